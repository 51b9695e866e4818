"""Resume signatures: what must stay fixed when a run is resumed and what may change.

A checkpoint stores ``signature = {"settings": ..., "data": manifest}``.  On resume the new
signature must be identical, unless ``--reconfigure`` is given, in which case only *execution*
settings may differ, the data manifest must match, and the number of global tokens per update
(``seq_len * micro_batch * grad_accum * world_size``) must be unchanged -- the objective and the
optimizer schedule are never re-interpreted (reference run_40b.py:361-420).

Keys and defaults of the reference's signature are kept so that its ``warpstate-server-v1``
checkpoints resume here; this framework adds its own execution keys (`kernels`, `grad_sync`,
`shard_optimizer`, `residual_dtype`).
"""
from __future__ import annotations

OBJECTIVE_KEYS = ("seq_len", "micro_batch", "grad_accum", "train_tokens", "lr", "min_lr", "warmup_steps",
                  "weight_decay", "seed", "activation_checkpointing", "loss_chunk_size", "compile")

# Execution settings with the value assumed when a stored signature predates the key.
EXECUTION_DEFAULTS = {
    "world_size": 1, "compile_core": False, "loss_mode": "checkpointed", "compile_mode": "default",
    "bf16_residuals": False, "activation_mode": "baseline", "gradient_mode": "eager",
    "overlap_swap_collectives": False, "overlap_runtime_estimates": False, "overlap_memory_budget": 0.0,
    "overlap_producer_schedule": False, "matmul_execution": None, "backward_layout_execution": None,
    "cache_core_weight_casts": False, "ddp_bucket_cap_mb": 128, "ddp_batched_grad_copy": False,
    # keys introduced by this framework
    "kernels": "library", "grad_sync": "ddp", "shard_optimizer": False,
}

EXECUTION_KEYS = set(EXECUTION_DEFAULTS) | {"micro_batch", "grad_accum", "activation_checkpointing",
                                            "loss_chunk_size", "compile"}


def train_signature(a, manifest: dict) -> dict:
    settings = {k: getattr(a, k) for k in OBJECTIVE_KEYS}
    for key, default in EXECUTION_DEFAULTS.items():
        settings[key] = getattr(a, key, default)
    settings["matmul_execution"] = getattr(a, "matmul_metadata", None)
    settings["backward_layout_execution"] = getattr(a, "backward_layout_metadata", None)
    return {"settings": settings, "data": manifest}


def _normalized(signature: dict) -> dict:
    settings = dict(signature["settings"])
    for key, default in EXECUTION_DEFAULTS.items():
        settings.setdefault(key, default)
    return {"settings": settings, "data": signature["data"]}


def global_batch_tokens(settings: dict) -> int:
    return settings["seq_len"] * settings["micro_batch"] * settings["grad_accum"] * settings["world_size"]


def check_resume_signature(old: dict, new: dict, reconfigure: bool = False) -> bool:
    """Returns False when nothing changed, True for an accepted execution-only change."""
    old, new = _normalized(old), _normalized(new)
    if old == new:
        return False
    message = "Resume settings/data differ; keep original settings or use --reconfigure for execution-only changes"
    if not reconfigure or old["data"] != new["data"]:
        raise ValueError(message)
    objective = lambda s: {k: v for k, v in s.items() if k not in EXECUTION_KEYS}
    if (objective(old["settings"]) != objective(new["settings"])
            or global_batch_tokens(old["settings"]) != global_batch_tokens(new["settings"])):
        raise ValueError(message + "; objective and global tokens per update must stay fixed")
    return True
