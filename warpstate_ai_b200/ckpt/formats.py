"""Checkpoint formats (single ``torch.save`` files, same keys as the reference).

* ``warpstate-server-v1`` (pretraining, reference run_40b.py:680-686): format, signature, origin,
  execution_history, config (``vars(cfg)``), model (FP32 state dict with canonical keys),
  optimizer (torch AdamW state dict: per-parameter step / exp_avg / exp_avg_sq, one group),
  step, tokens_seen, val_loss, val_step, val_tokens, rng_by_rank, rng_torch, rng_cuda,
  rng_numpy, rng_python.
* ``warpstate-posttrain-v1`` / ``warpstate-dpo-v1`` add sample_cursor, assistant_tokens_seen or
  response_tokens_seen, completed, total_steps, validation (reference posttrain.py:436-440,
  dpo.py:540-545).
* ``warpstate-chat-v1`` (inference export, reference chat.py:68-74): format, inference_only,
  config, step, tokens_seen, val_loss, tokenizer_sha256, captured_at_utc, source, [stage,
  origin], model -- plus a ``snapshot.json`` sidecar with the file's SHA-256 and size.

State-dict keys never carry wrapper prefixes (``module.``, ``_orig_mod.``).
"""
from __future__ import annotations

import json
import os
import random
from pathlib import Path

import numpy as np
import torch

from ..utils.io import atomic_json, digest, utc_timestamp

SERVER_FORMAT = "warpstate-server-v1"
POSTTRAIN_FORMAT = "warpstate-posttrain-v1"
DPO_FORMAT = "warpstate-dpo-v1"
CHAT_FORMAT = "warpstate-chat-v1"


# --------------------------------------------------------------------------- RNG
def capture_rng(device: torch.device | None = None) -> dict:
    state = {"torch": torch.get_rng_state(), "numpy": np.random.get_state(), "python": random.getstate()}
    if device is not None and device.type == "cuda":
        state["cuda"] = torch.cuda.get_rng_state(device)
    else:
        state["cuda"] = torch.zeros(0, dtype=torch.uint8)
    return state


def restore_rng(state: dict, device: torch.device | None = None) -> None:
    torch.set_rng_state(state["torch"])
    if device is not None and device.type == "cuda" and state.get("cuda") is not None and state["cuda"].numel():
        torch.cuda.set_rng_state(state["cuda"], device)
    np.random.set_state(state["numpy"])
    random.setstate(state["python"])


def seed_everything(seed: int, rank: int = 0, device: torch.device | None = None) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if device is not None and device.type == "cuda":
        torch.cuda.manual_seed(seed + rank)


# --------------------------------------------------------------------------- model state
def clean_state_dict(model: torch.nn.Module) -> dict:
    """State dict with canonical keys, whatever wrappers surround the model."""
    out = {}
    for key, value in model.state_dict().items():
        for prefix in ("module.", "_orig_mod."):
            while key.startswith(prefix):
                key = key[len(prefix):]
        out[key.replace("._orig_mod.", ".").replace(".module.", ".")] = value
    return out


def load_checkpoint(path, map_location="cpu"):
    return torch.load(path, map_location=map_location, mmap=True, weights_only=False)


def model_from_checkpoint(checkpoint: dict, device: torch.device, dtype=torch.float32):
    """Meta-device construction + ``assign=True`` load (no second host copy of 8 GB of weights)."""
    from ..config import WarpStateConfig
    from ..models.warpstate import WarpStateLM
    cfg = WarpStateConfig(**checkpoint["config"])
    cfg.validate()
    with torch.device("meta"):
        model = WarpStateLM(cfg)
    model.load_state_dict(checkpoint["model"], assign=True, strict=True)
    model.to(device=device, dtype=dtype)
    return model, cfg


def server_state(*, signature, origin, history, cfg, model, optimizer, step, tokens_seen, val_loss, val_step,
                 val_tokens, rng_by_rank, model_state=None) -> dict:
    """``model_state``: an already assembled unsharded state dict (sharded parameters), else ``model``'s own."""
    own = rng_by_rank[0]
    weights = model_state if model_state is not None else clean_state_dict(model)
    return {"format": SERVER_FORMAT, "signature": signature, "origin": origin, "execution_history": history,
            "config": vars(cfg).copy(), "model": weights, "optimizer": optimizer.state_dict(),
            "step": step, "tokens_seen": tokens_seen, "val_loss": val_loss, "val_step": val_step,
            "val_tokens": val_tokens, "rng_by_rank": rng_by_rank, "rng_torch": own["torch"],
            "rng_cuda": [own["cuda"]], "rng_numpy": own["numpy"], "rng_python": own["python"]}


# --------------------------------------------------------------------------- chat export
def export_chat_snapshot(checkpoint: dict, destination: Path, tokenizer: Path, source_info: dict,
                         stage: str | None = None) -> dict:
    """Model-only inference snapshot + ``snapshot.json``: the metadata stored inside the export, plus the export's
    SHA-256 and size (reference chat.py:37-102; stage exports ops/dpo_handoff.py:219-232, ops/archive_dpo.py:193-206,
    which also carry the stage's own token counter and the run's ancestry)."""
    from .writer import atomic_torch_save
    destination = Path(destination)
    destination.mkdir(parents=True, exist_ok=True)
    metadata = {"format": CHAT_FORMAT, "inference_only": True}
    if stage is not None:
        metadata["stage"] = stage
    metadata.update(config=dict(checkpoint["config"]), step=checkpoint.get("step"), tokens_seen=checkpoint.get("tokens_seen"))
    for counter in ("assistant_tokens_seen", "response_tokens_seen"):      # SFT resp. DPO checkpoints
        if stage is not None and counter in checkpoint:
            metadata[counter] = checkpoint[counter]
    metadata.update(val_loss=checkpoint.get("val_loss"), tokenizer_sha256=digest(tokenizer))
    if stage is not None:
        metadata["origin"] = checkpoint.get("origin")
    metadata.update(captured_at_utc=utc_timestamp(), source=source_info)
    model_path = destination / "model.pt"
    atomic_torch_save(model_path, {**metadata, "model": checkpoint["model"]})
    meta = {**metadata, "snapshot_sha256": digest(model_path), "snapshot_bytes": model_path.stat().st_size}
    atomic_json(destination / "snapshot.json", meta)
    return meta


def verify_chat_snapshot(directory: Path, tokenizer: Path | None = None) -> dict:
    directory = Path(directory)
    meta = json.loads((directory / "snapshot.json").read_text())
    model_path = directory / "model.pt"
    if model_path.stat().st_size != meta["snapshot_bytes"] or digest(model_path) != meta["snapshot_sha256"]:
        raise ValueError("Snapshot file does not match snapshot.json (size or SHA-256)")
    if tokenizer is not None and digest(tokenizer) != meta["tokenizer_sha256"]:
        raise ValueError("Tokenizer does not match the snapshot")
    return meta
