"""Direct preference optimisation (the engine behind ``dpo.py``).

The stage-specific half of a DPO run; the run itself is `train.stage.StageRun`.  What DPO adds, following
the reference's runner (reference dpo.py:38-647):

* it starts from an SFT export (``warpstate-chat-v1`` with ``stage == 'sft'``) that matches the plan's
  ``sft`` section (step, token count, tokenizer, and the base model's step and token count);
* sequences are scored by a head that returns per-sequence sums of response log-probabilities and never
  keeps vocabulary logits (`WarpStateLM.sequence_logps`; fused LM-head kernels on a GPU);
* the loss of a pair is ``-log sigmoid(r_chosen - r_rejected)`` with ``r = beta * (policy - reference)``,
  both scores divided by the response length for the length-normalised objective, averaged over the global
  pair count; reported with reward margin, reward accuracy and the chosen response's NLL per token;
* learning rate: linear warm-up, then linear decay to ``min_lr``;
* the frozen reference is scored once into a `ReferenceScoreCache` (resumable, multi-rank) -- or, with
  ``reference_mode = "resident"`` (this framework's addition), kept as a BF16 copy on the GPU and scored
  inside every update; the cache is built either way because it is what makes resume cheap;
* checkpoints are ``warpstate-dpo-v1``, completion records ``warpstate-dpo-completion-v1``.
"""
from __future__ import annotations

import gc
import json
import math
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..ckpt.formats import CHAT_FORMAT, DPO_FORMAT, capture_rng, restore_rng
from ..data import dpo as D
from ..data.sft import RENDER_FORMAT, renderer_sha256
from ..utils.io import digest
from .plans import DPO_PLAN
from .reference_cache import CACHE_FORMAT, ReferenceScoreCache, atomic_array, identity_digest  # noqa: F401
from .sft import source_identity as sft_sources
from .stage import StageRun, run_stage_cli, schedule_position, workspace

FORMAT = DPO_FORMAT
STOP = False
DEFAULTS = DPO_PLAN.defaults
METRICS = ("loss", "reward_margin", "reward_accuracy", "chosen_nll")
SCORING_SETTINGS = ("sequence_length", "micro_batch", "head_chunk_size", "compile_core", "bf16_residuals",
                    "deterministic", "workers")


def load_plan(path):
    """-> (plan document, effective training settings)"""
    return DPO_PLAN.read(path)


def source_identity() -> dict:
    package = Path(__file__).resolve().parents[1]
    mine = ("train/dpo.py", "train/reference_cache.py", "data/dpo.py")
    return {**sft_sources(), **{name: digest(package / name) for name in mine}}


def learning_rate(step: int, total_steps: int, s: dict) -> float:
    """Linear warm-up, then linear decay; a function of the step alone, so pauses do not bend it."""
    phase, x = schedule_position(step, total_steps, s["warmup_ratio"])
    if phase == "warmup":
        return s["lr"] * (step + 1) / x
    return s["min_lr"] + (s["lr"] - s["min_lr"]) * (1.0 - x)


def preference_metrics(policy, reference, counts, beta: float, objective: str):
    """Per-pair (loss, margin, accuracy) from ``[pairs, 2]`` score sums; gradients flow through ``policy`` only."""
    if objective not in ("length-normalized-dpo", "summed-dpo"):
        raise ValueError(f"unknown DPO objective {objective!r}")
    reference = reference.detach().to(policy.dtype)
    if objective == "length-normalized-dpo":
        lengths = counts.clamp_min(1)
        policy, reference = policy / lengths, reference / lengths
    reward = (policy - reference) * beta
    margin = reward[:, 0] - reward[:, 1]
    return -F.logsigmoid(margin), margin, (margin > 0).to(policy.dtype)


def reference_identity(weights_hash, manifest_hash, tokenizer_hash, s, device, world) -> dict:
    """Everything that determines the frozen reference's scores."""
    return dict(format=CACHE_FORMAT, weights_sha256=weights_hash, data_sha256=manifest_hash,
                tokenizer_sha256=tokenizer_hash, renderer_sha256=renderer_sha256(), mask_format=D.MASK_FORMAT,
                sources=source_identity(), settings={key: s[key] for key in SCORING_SETTINGS}, dropout=0.0,
                logps="response-token-sum-float32", dtype="bfloat16", device_type=device.type, world_size=world,
                torch_version=torch.__version__)


def validate_cache(directory, identity, sizes):
    return ReferenceScoreCache(directory, identity, sizes).verify()


def score_pairs(model, x, y, device, head_chunk_size: int):
    from .engine import autocast_for
    with autocast_for(device):
        return model.sequence_logps(x, y, head_chunk_size)


def _pair_statistics(logps, reference, y, active, s):
    """(per-pair losses, 4 weighted sums: loss, margin, accuracy, chosen NLL per token)"""
    counts = (y != -100).sum(dim=1).reshape(-1, 2)
    losses, margins, accuracy = preference_metrics(logps, reference, counts, s["beta"], s["objective"])
    nll = -logps[:, 0] / counts[:, 0].clamp_min(1)
    weight = active.double()
    sums = torch.stack([(t.detach().double() * weight).sum() for t in (losses, margins, accuracy, nll)])
    return losses, sums


def training_update(trainer, microbatches, global_pairs: int, s: dict, lr: float, resident=None, control=None):
    """One DPO update; ``microbatches`` hold ``(x, y, active, reference score sums [pairs, 2])``.
    -> ({loss, reward_margin, reward_accuracy, chosen_nll} as global pair means, gradient norm)"""
    device, world = trainer.device, trainer.world_size
    sums = torch.zeros(5, dtype=torch.float64, device=device)
    trainer.begin_update()
    for position, batch in enumerate(microbatches):
        x, y, active, reference = (t.to(device) for t in batch)
        if resident is not None:
            with torch.no_grad():
                reference = score_pairs(resident, x, y, device, s["head_chunk_size"]).reshape(-1, 2)

        def loss_fn(x=x, y=y, active=active, reference=reference):
            nonlocal sums
            logps = trainer.model.sequence_logps(x, y, s["head_chunk_size"]).reshape(-1, 2)
            losses, four = _pair_statistics(logps, reference, y, active, s)
            sums = sums + torch.cat([four, active.double().sum().reshape(1)])
            # the gradient synchroniser averages over ranks: world / global pairs turns the local sum into
            # this rank's share of the global pair mean
            return (losses * active).sum(), world / global_pairs, 0.0

        trainer.micro_step(loss_fn, last=position + 1 == len(microbatches))
    stats = trainer.finish_update(lr)
    if world > 1:
        dist.all_reduce(sums)
    _, norm, _ = trainer.read_update_scalars(stats)
    host = sums.tolist()
    if int(host[4]) != global_pairs:
        raise RuntimeError(f"the ranks scored {int(host[4])} pairs but the update holds {global_pairs}")
    means = [value / host[4] for value in host[:4]]
    if not (all(map(math.isfinite, means)) and math.isfinite(norm)):
        raise RuntimeError("non-finite DPO loss or gradient norm")
    return dict(zip(METRICS, means)), norm


@torch.no_grad()
def evaluate(trainer, records, reference, s, pad_id, *, full=False, resident=None):
    """Pair means of loss, margin, accuracy and chosen NLL over the hold-out pairs (all, or the first
    ``eval_batches`` micro-batches).  ``reference``: cached score sums aligned with ``records``."""
    model, device = trainer.model, trainer.device
    mb = s["micro_batch"]
    take = len(records) if full else min(len(records), s["eval_batches"] * mb)
    rng = capture_rng(device)
    training = model.training
    model.eval()
    sums = torch.zeros(4, dtype=torch.float64, device=device)
    try:
        for begin in range(0, take, mb):
            rows = list(records[begin:min(begin + mb, take)])
            real = len(rows)
            x, y, active = (t.to(device) for t in D.collate_pairs(rows + [None] * (mb - real), s["sequence_length"], pad_id))
            if resident is not None:
                ref = score_pairs(resident, x, y, device, s["head_chunk_size"]).reshape(-1, 2)
            else:
                ref = torch.zeros((mb, 2), device=device)
                ref[:real] = torch.as_tensor(np.array(reference[begin:begin + real]), device=device)
            logps = score_pairs(model, x, y, device, s["head_chunk_size"]).reshape(-1, 2)
            sums += _pair_statistics(logps, ref, y, active, s)[1]
    finally:
        model.train(training)
        restore_rng(rng, device)
    means = (sums / take).tolist()
    if not all(map(math.isfinite, means)):
        raise RuntimeError("non-finite DPO validation")
    return {"val_loss": means[0], **dict(zip(METRICS[1:], means[1:])), "evaluated_samples": take}


def validate_resume(checkpoint, signature, world):
    if checkpoint.get("format") != FORMAT or checkpoint.get("signature") != signature:
        raise ValueError("the checkpoint belongs to a DPO run with another signature; use a new output directory")
    if len(checkpoint.get("rng_by_rank", [])) != world:
        raise ValueError("the checkpoint does not hold one RNG state per rank")


def validate_reference_path(args) -> Path:
    """The cache directory: inside the workspace, disjoint from outputs, data and the weights' directory."""
    root = workspace()
    cache = Path(args.reference_cache_dir).resolve()
    if cache == root or not cache.is_relative_to(root):
        raise ValueError("the reference cache must be a directory inside the workspace")
    for other in (Path(p).resolve() for p in (args.work_dir, args.data_dir, Path(args.weights).parent)):
        if cache == other or cache.is_relative_to(other) or other.is_relative_to(cache):
            raise ValueError(f"the reference cache {cache} overlaps {other}; keep it apart from outputs and inputs")
    return cache


def load_model(checkpoint, s, device, tokenizer, dtype=torch.float32):
    """A model for scoring under DPO's rules (dropout off) from a checkpoint dict: (model, config)."""
    from ..config import WarpStateConfig
    from ..models.warpstate import WarpStateLM
    cfg = WarpStateConfig(**checkpoint["config"])
    cfg.gradient_checkpointing, cfg.dropout = s["gradient_checkpointing"], 0.0
    cfg.validate()
    if cfg.vocab_size != tokenizer.vocab_size() or s["sequence_length"] % cfg.chunk_size:
        raise ValueError("the model does not fit the tokenizer's vocabulary, or sequence_length is not a whole number "
                         "of chunks")
    with torch.device("meta"):
        model = WarpStateLM(cfg)
    model.load_state_dict(checkpoint["model"], strict=True, assign=True)
    model = model.to(device=device, dtype=dtype)
    if device.type == "cpu":
        for p in model.parameters():
            p.data = p.data.clone()
    model.bf16_residuals = bool(s["bf16_residuals"])
    return model, cfg


def prepare_reference(args, identity, records, s, device, rank, world, tokenizer, control=None, stop=None):
    """Create or reuse the reference-score cache: (train scores, validation scores, manifest hash), or None when
    a stop request interrupted the scoring (the shards stay and the next launch continues)."""
    from ..ckpt.formats import load_checkpoint
    cache = ReferenceScoreCache(args.reference_cache_dir, identity, [len(rows) for rows in records])
    if cache.sealed:
        return cache.verify()
    frozen, _ = load_model(load_checkpoint(args.weights), s, device, tokenizer)
    frozen.requires_grad_(False).eval()
    pad_id = tokenizer.pad_id() if tokenizer.pad_id() >= 0 else tokenizer.eos_id()
    mb = s["micro_batch"]

    def score_batch(rows):
        x, y, _ = D.collate_pairs(list(rows) + [None] * (mb - len(rows)), s["sequence_length"], pad_id)
        with torch.no_grad():
            sums = score_pairs(frozen, x.to(device), y.to(device), device, s["head_chunk_size"])
        return sums.reshape(-1, 2).double().cpu().numpy()[:len(rows)]

    def barrier():
        if world > 1:
            dist.barrier(group=control)

    try:
        return cache.build(records, score_batch, mb, rank, world, stop or (lambda: False), barrier)
    finally:
        del frozen
        gc.collect()
        if device.type == "cuda":
            torch.cuda.empty_cache()


class DpoStage(StageRun):
    stage = "dpo"
    checkpoint_format = FORMAT
    completion_format = "warpstate-dpo-completion-v1"
    scored_key = "response_tokens_seen"
    schema = DPO_PLAN

    def __init__(self, args, stop_flag):
        super().__init__(args, stop_flag)
        self.cache_dir = validate_reference_path(args)
        self.resident = None

    def lock_directories(self) -> list:
        return [self.work, self.cache_dir]

    def adjust_config(self, cfg) -> None:
        cfg.dropout = 0.0      # policy and reference are compared under one deterministic scoring rule

    def load_data(self):
        return D.load_data(self.data_dir, self.sp, self.tokenizer_hash, self.s["sequence_length"])

    def check_source(self, export: dict) -> None:
        good = (export.get("format") == CHAT_FORMAT and export.get("inference_only") is True
                and export.get("stage") == "sft" and export.get("tokenizer_sha256") == self.tokenizer_hash)
        if not good:
            raise ValueError("DPO starts from an SFT model export made with this tokenizer")
        promised = self.plan.get("sft", self.plan.get("base", {}))
        for key in ("step", "tokens_seen", "tokenizer_sha256"):
            if key in promised and promised[key] != export.get(key):
                raise ValueError(f"the plan expects SFT {key} = {promised[key]!r}; the export says {export.get(key)!r}")
        ancestor = export.get("origin") or {}
        for key in ("base_step", "base_tokens_seen"):
            if key in promised and promised[key] != ancestor.get(key[5:], ancestor.get(key)):
                raise ValueError(f"the plan expects {key} = {promised[key]!r}; the export's origin disagrees")

    def before_training(self) -> bool:
        s = self.s
        self.identity = reference_identity(self.base_hash, self.manifest_hash, self.tokenizer_hash, s, self.device,
                                           self.world)
        result = prepare_reference(self.args, self.identity, (self.train_data, self.val_data), s, self.device,
                                   self.rank, self.world, self.sp, self.control, stop=self.stop_requested)
        if result is None:
            print(json.dumps(dict(event="reference_paused", rank=self.rank)), flush=True)
            return False
        self.reference_train, self.reference_val, self.reference_hash = result
        if getattr(self.args, "reference_only", False):
            print(json.dumps(dict(event="reference_complete", reference_sha256=self.reference_hash)), flush=True)
            return False
        return True

    def signature_fields(self) -> dict:
        return dict(renderer=RENDER_FORMAT, mask=D.MASK_FORMAT, base_sha256=self.base_hash,
                    reference_sha256=self.reference_hash, sources=source_identity())

    def after_trainer(self) -> None:
        if self.s["reference_mode"] == "resident":
            from ..ckpt.formats import load_checkpoint
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            self.resident, _ = load_model(load_checkpoint(self.weights), self.s, self.device, self.sp, dtype=dtype)
            self.resident.requires_grad_(False).eval()

    def learning_rate(self, step: int) -> float:
        return learning_rate(step, self.total_steps, self.s)

    def count_tokens(self, indices):
        rows = [self.train_data[i] for i in indices]
        return sum(map(D.pair_tokens, rows)), sum(map(D.pair_targets, rows))

    def run_update(self, indices, lr: float) -> dict:
        s, mb = self.s, self.s["micro_batch"]
        batches = []
        for micro in range(s["grad_accum"]):
            first = (micro * self.world + self.rank) * mb
            mine = indices[first:first + mb]
            rows = [self.train_data[i] for i in mine] + [None] * (mb - len(mine))
            x, y, active = D.collate_pairs(rows, s["sequence_length"], self.pad_id)
            scores = torch.zeros((mb, 2), dtype=torch.float32)
            if mine:
                scores[:len(mine)] = torch.as_tensor(np.array(self.reference_train[mine]), dtype=torch.float32)
            batches.append((x, y, active, scores))
        values, norm = training_update(self.trainer, batches, len(indices), s, lr, self.resident, self.control)
        return dict(values, grad_norm=norm)

    def rate_fields(self, indices, scored: int, seconds: float) -> dict:
        return dict(pairs_per_second=len(indices) / seconds)

    def validate(self, full: bool) -> dict:
        return evaluate(self.trainer, self.val_data, self.reference_val, self.s, self.pad_id, full=full,
                        resident=self.resident)

    def event_fields(self) -> dict:
        return dict(objective=self.s["objective"])

    def evaluation_fields(self, values: dict) -> dict:
        return dict(reference_sha256=self.reference_hash, mask_format=D.MASK_FORMAT)

    def checkpoint_fields(self) -> dict:
        return dict(validation=self.last_validation)

    def completion_fields(self) -> dict:
        return dict(sample_cursor=self.progress.sample_cursor, reference_sha256=self.reference_hash)

    def after_training(self) -> None:
        ReferenceScoreCache(self.cache_dir, self.identity, (len(self.train_data), len(self.val_data))).verify()
        if digest(self.weights) != self.base_hash:
            raise RuntimeError("the SFT export this run started from changed on disk during the run")


def train(args) -> None:
    DpoStage(args, lambda: STOP).execute()


def main(argv=None) -> None:
    import signal
    import sys
    run_stage_cli(DpoStage, sys.modules[__name__], argv, "WarpState DPO", extra_dirs=("reference-cache-dir",),
                  extra_flags=("--reference-only",), signals=(signal.SIGUSR1,))


if __name__ == "__main__":
    main()
