"""Assistant-only supervised fine-tuning (the engine behind ``posttrain.py``).

The stage-specific half of an SFT run; the run itself (workspace rules, plan, resume, loop, records,
checkpoints) is `train.stage.StageRun`.  What SFT adds, following the reference's runner
(reference posttrain.py:34-543):

* it starts from a model-only ``warpstate-chat-v1`` export whose tokenizer hash, step and token count
  match the plan's ``base`` section;
* the objective is the mean loss over all assistant tokens of the *global* batch: a micro-batch's mean
  loss enters with weight ``local_targets * world / global_targets`` (rank averaging divides by world);
* learning rate: linear warm-up over ``warmup_ratio`` of the run, cosine to ``min_lr``;
* validation reports loss, perplexity and the number of assistant tokens evaluated;
* checkpoints are ``warpstate-posttrain-v1``, completion records ``warpstate-posttrain-completion-v1``.

The update runs on the `Trainer` (fused kernels on a GPU, arena AdamW, fused gradient synchronisation).
"""
from __future__ import annotations

import math

import torch

from ..ckpt.formats import CHAT_FORMAT, POSTTRAIN_FORMAT, capture_rng, restore_rng
from ..data import sft as D
from ..utils.io import digest
from .plans import SFT_PLAN
from .stage import (StageRun, base_pipeline_lock, run_stage_cli, schedule_position, shared_pipeline_lock,  # noqa: F401
                    validate_paths, workspace)

FORMAT = POSTTRAIN_FORMAT
STOP = False
DEFAULTS = SFT_PLAN.defaults


def load_plan(path):
    """-> (plan document, effective training settings)"""
    return SFT_PLAN.read(path)


def learning_rate(step: int, total_steps: int, s: dict) -> float:
    phase, x = schedule_position(step, total_steps, s["warmup_ratio"])
    if phase == "warmup":
        return s["lr"] * (step + 1) / x
    return s["min_lr"] + (s["lr"] - s["min_lr"]) * 0.5 * (1.0 + math.cos(math.pi * x))


def token_weighted_loss(mean_loss, local_targets: int, global_targets: int, world_size: int):
    """A micro-batch's mean loss scaled so that the rank-average of the gradients is the gradient of the
    global assistant-token mean."""
    if global_targets < 1:
        raise ValueError("the update contains no supervised tokens")
    return mean_loss * (local_targets * world_size / global_targets)


def source_identity() -> dict:
    """Hashes of the source files that define the objective and the data rendering."""
    from pathlib import Path
    package = Path(__file__).resolve().parents[1]
    names = ("train/sft.py", "train/stage.py", "train/plans.py", "data/sft.py", "ckpt/writer.py", "train/engine.py",
             "models/warpstate.py", "config.py")
    return {name: digest(package / name) for name in names}


def training_update(trainer, microbatches, global_targets: int, lr: float):
    """One SFT update on the engine: (assistant-token mean loss over all ranks, gradient norm)."""
    if global_targets < 1:
        raise ValueError("the update contains no supervised tokens")
    scale = trainer.world_size / global_targets
    trainer.begin_update()
    for position, (x, y) in enumerate(microbatches):
        count = int((y != D.IGNORE_INDEX).sum())
        x, y = x.to(trainer.device), y.to(trainer.device)

        def loss_fn(x=x, y=y, count=count):
            _, loss = trainer.model(x, y, return_logits=False)
            return loss, count * scale, float(count)       # backward weight, and the weight of the reported sum

        trainer.micro_step(loss_fn, last=position + 1 == len(microbatches))
    stats = trainer.finish_update(lr)
    weighted_sum, norm, _ = trainer.read_update_scalars(stats)   # sum over ranks of mean loss x targets
    if not (math.isfinite(weighted_sum) and math.isfinite(norm)):
        raise RuntimeError("non-finite SFT loss or gradient norm")
    return weighted_sum / global_targets, norm


@torch.no_grad()
def evaluate(trainer, records, s: dict, pad_id: int, *, full: bool = False):
    """(assistant-token mean loss, assistant tokens) over the hold-out records (all of them, or the first
    ``eval_batches`` micro-batches).  Leaves the RNG streams and the training mode as it found them."""
    from .engine import autocast_for
    model, device = trainer.model, trainer.device
    mb = s["micro_batch"]
    take = len(records) if full else min(len(records), s["eval_batches"] * mb)
    rng = capture_rng(device)
    training = model.training
    model.eval()
    weighted, counted = 0.0, 0
    try:
        for begin in range(0, take, mb):
            x, y = D.collate(records[begin:min(begin + mb, take)], s["sequence_length"], pad_id)
            count = int((y != D.IGNORE_INDEX).sum())
            with autocast_for(device):
                _, loss = model(x.to(device), y.to(device), return_logits=False)
            weighted += float(loss) * count
            counted += count
    finally:
        model.train(training)
        restore_rng(rng, device)
    mean = weighted / counted
    if not math.isfinite(mean):
        raise RuntimeError("non-finite SFT validation loss")
    return mean, counted


def validate_resume(checkpoint, signature, world_size):
    if checkpoint.get("format") != FORMAT or checkpoint.get("signature") != signature:
        raise ValueError("the checkpoint belongs to a run with another signature; use a new output directory")
    if len(checkpoint.get("rng_by_rank", [])) != world_size:
        raise ValueError("the checkpoint does not hold one RNG state per rank")


class SftStage(StageRun):
    stage = "sft"
    checkpoint_format = FORMAT
    completion_format = "warpstate-posttrain-completion-v1"
    scored_key = "assistant_tokens_seen"
    schema = SFT_PLAN

    def load_data(self):
        return D.load_data(self.data_dir, self.sp, self.tokenizer_hash, self.s["sequence_length"])

    def check_source(self, export: dict) -> None:
        if export.get("format") != CHAT_FORMAT or export.get("inference_only") is not True:
            raise ValueError(f"SFT starts from a model-only {CHAT_FORMAT} export, not from {export.get('format')!r}")
        if export.get("tokenizer_sha256") != self.tokenizer_hash:
            raise ValueError("the base export was made with another tokenizer")
        promised = self.plan.get("base", {})
        for key in ("step", "tokens_seen", "tokenizer_sha256"):
            if key in promised and promised[key] != export.get(key):
                raise ValueError(f"plan.base.{key} = {promised[key]!r} but the export says {export.get(key)!r}")

    def signature_fields(self) -> dict:
        return dict(renderer=D.RENDER_FORMAT, base_sha256=self.base_hash, sources=source_identity())

    def learning_rate(self, step: int) -> float:
        return learning_rate(step, self.total_steps, self.s)

    def count_tokens(self, indices):
        rows = [self.train_data[i] for i in indices]
        return sum(len(r["input_ids"]) - 1 for r in rows), sum(D.supervised_count(r) for r in rows)

    def run_update(self, indices, lr: float) -> dict:
        s = self.s
        targets = sum(D.supervised_count(self.train_data[i]) for i in indices)
        per_step = D.rank_microbatches(indices, self.train_data, s["micro_batch"], s["grad_accum"], self.world, self.rank)
        batches = [D.collate(rows, s["sequence_length"], self.pad_id) for rows in per_step]
        loss, norm = training_update(self.trainer, batches, targets, lr)
        return dict(loss=loss, grad_norm=norm)

    def rate_fields(self, indices, scored: int, seconds: float) -> dict:
        return dict(assistant_tokens_per_second=scored / seconds)

    def validate(self, full: bool) -> dict:
        loss, tokens = evaluate(self.trainer, self.val_data, self.s, self.pad_id, full=full)
        return dict(val_loss=loss, val_perplexity=math.exp(loss), validation_assistant_tokens=tokens)

    def evaluation_fields(self, values: dict) -> dict:
        window = self.s["eval_batches"] * self.s["micro_batch"]
        seen = len(self.val_data) if values.get("full_holdout") else min(len(self.val_data), window)
        return dict(evaluated_samples=seen, base_step=self.origin["step"], objective="assistant-token-mean",
                    renderer_format=D.RENDER_FORMAT)

    def completion_fields(self) -> dict:
        return dict(base_step=self.origin["step"])


def train(args) -> None:
    SftStage(args, lambda: STOP).execute()


def main(argv=None) -> None:
    import sys
    run_stage_cli(SftStage, sys.modules[__name__], argv, "WarpState assistant-only SFT")


if __name__ == "__main__":
    main()
