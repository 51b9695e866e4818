"""Assistant-only supervised fine-tuning (the engine behind ``posttrain.py``).

Behaviour follows the reference SFT runner (posttrain.py:34-543): a JSON plan
(``warpstate-posttrain-plan-v1``) whose ``training`` section overrides `DEFAULTS`; inputs and
outputs confined to one workspace root and kept apart from each other; initialisation from a
model-only ``warpstate-chat-v1`` export; token-weighted loss (each micro-batch's mean loss times
``local_targets * world / global_targets``); deterministic epoch order with a resumable sample
cursor; warm-up-ratio + cosine learning rate; a full hold-out evaluation before the first
update and at the end, a subset in between; checkpoints ``warpstate-posttrain-v1`` through the
distributed async writer; JSON-lines events on stdout and in ``metrics.jsonl``;
``completion.json`` when all steps are done.

The workspace root defaults to ``/workspace/WarpState`` and can be moved with the
``WARPSTATE_WORKSPACE`` environment variable.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import math
import os
import random
import signal
import time
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from ..ckpt.formats import CHAT_FORMAT, POSTTRAIN_FORMAT, capture_rng, clean_state_dict, restore_rng
from ..data import sft as D
from ..utils.io import atomic_json, digest, process_lock

FORMAT = POSTTRAIN_FORMAT
STOP = False
DEFAULTS = dict(sequence_length=2048, micro_batch=4, grad_accum=4, lr=5e-6, min_lr=0.0, warmup_ratio=0.03, epochs=1,
                max_steps=None, weight_decay=0.0, seed=42, eval_every=100, save_every=100, eval_batches=32,
                compile_core=True, loss_mode="compiled-full", bf16_residuals=True, gradient_checkpointing=False,
                workers=4, deterministic=True, clip_grad_norm=1.0)


def workspace() -> Path:
    return Path(os.environ.get("WARPSTATE_WORKSPACE", "/workspace/WarpState")).resolve()


# --------------------------------------------------------------------------- plan / paths
def _positive_int(settings, names):
    for name in names:
        if type(settings[name]) is not int or settings[name] < 1:
            raise ValueError(f"{name} must be a positive integer")


def _finite_nonneg(settings, names):
    for name in names:
        v = settings[name]
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v < 0:
            raise ValueError(f"{name} must be finite and nonnegative")


def load_plan(path):
    plan = json.loads(Path(path).read_text())
    if plan.get("format") != "warpstate-posttrain-plan-v1" or plan.get("stage") != "sft":
        raise ValueError("Expected warpstate-posttrain-plan-v1 stage sft")
    supplied = plan.get("training", {})
    unknown = set(supplied) - set(DEFAULTS)
    if unknown:
        raise ValueError(f"Unknown training settings: {sorted(unknown)}")
    s = DEFAULTS | supplied
    _positive_int(s, ("sequence_length", "micro_batch", "grad_accum", "epochs", "eval_every", "save_every",
                      "eval_batches", "workers"))
    ratio = s["warmup_ratio"]
    if isinstance(ratio, bool) or not isinstance(ratio, (int, float)) or not 0 <= ratio < 1:
        raise ValueError("warmup_ratio must be in [0, 1)")
    if s["max_steps"] is not None and (type(s["max_steps"]) is not int or s["max_steps"] < 1):
        raise ValueError("max_steps must be null or a positive integer")
    _finite_nonneg(s, ("lr", "min_lr", "weight_decay", "clip_grad_norm"))
    if not 0 < s["lr"] or s["min_lr"] > s["lr"] or not s["clip_grad_norm"]:
        raise ValueError("Require 0 <= min_lr <= lr and positive lr/clip_grad_norm")
    if type(s["seed"]) is not int or s["seed"] < 0:
        raise ValueError("seed must be a nonnegative integer")
    for name in ("compile_core", "bf16_residuals", "gradient_checkpointing", "deterministic"):
        if type(s[name]) is not bool:
            raise ValueError(f"{name} must be a boolean")
    if s["loss_mode"] not in ("full", "compiled-full", "checkpointed"):
        raise ValueError("Unsupported loss_mode")
    return plan, s


def validate_paths(work_dir, data_dir, weights, tokenizer, config):
    root = workspace()
    paths = [Path(p).resolve() for p in (work_dir, data_dir, weights, tokenizer, config)]
    if any(not p.is_relative_to(root) for p in paths):
        raise ValueError(f"All inputs and outputs must stay inside {root}")
    work, data, source, tok, plan = paths
    if work == root or any(p == work or p.is_relative_to(work) for p in (data, source, tok, plan)):
        raise ValueError("Training outputs must be separate from every input")
    if work.is_relative_to(data) or work.is_relative_to(source.parent):
        raise ValueError("Training outputs must not be inside data or source-weight directories")
    for p in (source, tok, plan):
        if not p.is_file():
            raise ValueError(f"Missing required input: {p}")
    if not data.is_dir():
        raise ValueError(f"Missing prepared data directory: {data}")
    return paths


@contextlib.contextmanager
def shared_pipeline_lock(path):
    """Every post-training rank holds the base job's ``pipeline.lock`` shared, so pretraining
    cannot start while any of them -- even an orphan -- is alive."""
    path = Path(path).resolve()
    if not path.is_relative_to(workspace()):
        raise ValueError("Pipeline lock must stay inside the workspace")
    try:
        with process_lock(path, shared=True):
            yield
    except Exception as error:
        if type(error).__name__ == "LockHeld":
            raise RuntimeError("Pretraining or its handoff currently owns pipeline.lock") from error
        raise


@contextlib.contextmanager
def base_pipeline_lock(plan):
    base = plan.get("handoff", {}).get("base_work_dir")
    if base is None:
        yield
        return
    root = workspace()
    path = (root / base).resolve()
    if not path.is_relative_to(root) or path == root or not path.is_dir():
        raise ValueError("handoff.base_work_dir must be an existing workspace directory")
    with shared_pipeline_lock(path / "pipeline.lock"):
        yield


# --------------------------------------------------------------------------- numerics helpers
def learning_rate(step: int, total_steps: int, s: dict) -> float:
    warmup = min(math.ceil(s["warmup_ratio"] * total_steps), max(0, total_steps - 1))
    if step < warmup:
        return s["lr"] * (step + 1) / warmup
    progress = min(1.0, (step - warmup) / max(1, total_steps - warmup - 1))
    return s["min_lr"] + 0.5 * (s["lr"] - s["min_lr"]) * (1 + math.cos(math.pi * progress))


def token_weighted_loss(mean_loss, local_targets: int, global_targets: int, world_size: int):
    """Rank averaging divides by world, so each local token *sum* is scaled by world/global."""
    if global_targets < 1:
        raise ValueError("Update has no supervised tokens")
    return mean_loss * (local_targets * world_size / global_targets)


def validate_resume(checkpoint, signature, world_size):
    if checkpoint.get("format") != FORMAT or checkpoint.get("signature") != signature:
        raise ValueError("Posttraining resume signature differs; use a new output directory")
    if len(checkpoint.get("rng_by_rank", [])) != world_size:
        raise ValueError("Checkpoint lacks exact per-rank RNG state")


def source_identity() -> dict:
    """Hashes of the source files that define the objective and the data rendering."""
    root = Path(__file__).resolve().parents[1]
    files = [Path(__file__), root / "data/sft.py", root / "ckpt/writer.py", root / "train/engine.py",
             root / "models/warpstate.py", root / "config.py"]
    return {str(p.relative_to(root)): digest(p) for p in files}


def training_update(trainer, microbatches, global_targets: int, lr: float):
    """One SFT update on the engine.  Returns (token-mean loss over all ranks, grad norm)."""
    world = trainer.world_size
    trainer.begin_update()
    local_targets = 0
    for index, (x, y) in enumerate(microbatches):
        targets = int(y.ne(-100).sum())
        local_targets += targets
        x, y = x.to(trainer.device), y.to(trainer.device)

        def loss_fn(x=x, y=y, targets=targets):
            _, loss = trainer.model(x, y, return_logits=False)
            if global_targets < 1:
                raise ValueError("Update has no supervised tokens")
            return loss, targets * world / global_targets, float(targets)

        trainer.micro_step(loss_fn, last=index == len(microbatches) - 1)
    stats = trainer.finish_update(lr)  # loss_sum now holds sum over ranks of loss*targets
    loss_sum, norm, _ = trainer.read_update_scalars(stats)
    if not math.isfinite(loss_sum) or not math.isfinite(norm):
        raise RuntimeError("Non-finite SFT training loss or gradient norm")
    return loss_sum / global_targets, norm


@torch.no_grad()
def evaluate(trainer, records, s: dict, pad_id: int, *, full: bool = False):
    from .engine import autocast_for
    model, device = trainer.model, trainer.device
    was_training = model.training
    state = capture_rng(device)
    model.eval()
    total_loss, total_targets = 0.0, 0
    try:
        limit = len(records) if full else s["eval_batches"] * s["micro_batch"]
        for start in range(0, min(len(records), limit), s["micro_batch"]):
            batch = records[start:min(start + s["micro_batch"], limit)]
            x, y = D.collate(batch, s["sequence_length"], pad_id)
            targets = int(y.ne(-100).sum())
            with autocast_for(device):
                _, loss = model(x.to(device), y.to(device), return_logits=False)
            total_loss += float(loss) * targets
            total_targets += targets
    finally:
        model.train(was_training)
        restore_rng(state, device)
    value = total_loss / total_targets
    if not math.isfinite(value):
        raise RuntimeError("Non-finite SFT validation loss")
    return value, total_targets


# --------------------------------------------------------------------------- the run
def train(args) -> None:
    import sentencepiece as spm
    from ..ckpt.formats import load_checkpoint
    from ..ckpt.writer import DistributedCheckpointWriter, host_control_group
    from ..config import WarpStateConfig
    from ..models.warpstate import WarpStateLM
    from .engine import Trainer

    work, data_dir, weights, tokenizer_path, config = validate_paths(args.work_dir, args.data_dir, args.weights,
                                                                     args.tokenizer, args.config)
    plan, s = load_plan(config)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank) if args.device == "cuda" else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
        if not torch.cuda.is_available() or not torch.cuda.is_bf16_supported():
            raise RuntimeError("BF16-capable CUDA GPU required")
    torch.set_num_threads(s["workers"])
    random.seed(s["seed"] + rank)
    np.random.seed(s["seed"] + rank)
    torch.manual_seed(s["seed"] + rank)
    tokenizer_hash = digest(tokenizer_path)
    sp = spm.SentencePieceProcessor(model_file=str(tokenizer_path))
    train_data, val_data, manifest, manifest_hash = D.load_data(data_dir, sp, tokenizer_hash, s["sequence_length"])
    base_hash = digest(weights)
    signature = dict(plan=plan, settings=s, data_sha256=manifest_hash, tokenizer_sha256=tokenizer_hash,
                     renderer=D.RENDER_FORMAT, base_sha256=base_hash, world_size=world, device_type=device.type,
                     torch_version=torch.__version__, sources=source_identity())
    latest = work / "latest.pt"
    resuming = latest.exists()
    checkpoint = load_checkpoint(latest if resuming else weights)
    if resuming:
        validate_resume(checkpoint, signature, world)
        origin = checkpoint["origin"]
    else:
        if checkpoint.get("format") != CHAT_FORMAT or checkpoint.get("inference_only") is not True:
            raise ValueError("Initialize SFT from an independent warpstate-chat-v1 model-only export")
        if checkpoint.get("tokenizer_sha256") != tokenizer_hash:
            raise ValueError("Base model export tokenizer differs")
        for key in ("step", "tokens_seen", "tokenizer_sha256"):
            if key in plan.get("base", {}) and plan["base"][key] != checkpoint.get(key):
                raise ValueError(f"Base model {key} differs from plan")
        origin = {k: v for k, v in checkpoint.items() if k != "model"}
        origin.update(weights_sha256=base_hash, weights_path=str(weights))
    cfg = WarpStateConfig(**checkpoint["config"])
    cfg.gradient_checkpointing = s["gradient_checkpointing"]
    cfg.validate()
    if cfg.vocab_size != sp.vocab_size() or s["sequence_length"] % cfg.chunk_size:
        raise ValueError("Model/tokenizer vocabulary or sequence/chunk mismatch")
    with torch.device("meta"):
        raw = WarpStateLM(cfg)
    raw.load_state_dict(checkpoint["model"], strict=True, assign=True)
    raw = raw.to(device=device, dtype=torch.float32).requires_grad_(True)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if device.type == "cuda":
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group("gloo")
    control = host_control_group() if world > 1 else None
    trainer = Trainer(raw, device=device, rank=rank, world_size=world, lr=s["lr"], weight_decay=s["weight_decay"],
                      max_grad_norm=s["clip_grad_norm"])
    optimizer = trainer.optimizer
    step = cursor = tokens_seen = assistant_tokens_seen = 0
    if resuming:
        optimizer.load_state_dict(checkpoint["optimizer"])
        step, cursor = checkpoint["step"], checkpoint["sample_cursor"]
        tokens_seen, assistant_tokens_seen = checkpoint["tokens_seen"], checkpoint["assistant_tokens_seen"]
        restore_rng(checkpoint["rng_by_rank"][rank], device)
    del checkpoint
    global_batch = s["micro_batch"] * s["grad_accum"] * world
    total_steps = math.ceil(len(train_data) / global_batch) * s["epochs"]
    if s["max_steps"] is not None:
        total_steps = min(total_steps, s["max_steps"])
    end_step = min(total_steps, step + args.max_steps) if args.max_steps is not None else total_steps
    work.mkdir(parents=True, exist_ok=True)
    if rank == 0:
        (work / "settings.json").write_text(json.dumps(dict(signature=signature, origin=origin, total_steps=total_steps,
                                                            train_rows=len(train_data), val_rows=len(val_data)),
                                                       indent=2, default=str) + "\n")
        if step < total_steps:
            (work / "completion.json").unlink(missing_ok=True)
    pad_id = sp.pad_id() if sp.pad_id() >= 0 else sp.eos_id()
    last_validation = last_validation_step = None

    def validation(*, full=False):
        values = [evaluate(trainer, val_data, s, pad_id, full=full) if rank == 0 else None]
        if world > 1:
            dist.broadcast_object_list(values, src=0, group=control)
        return values[0]

    def metric(values):
        if rank != 0:
            return
        values.update(timestamp=time.time(), stage="sft", step=step, tokens_seen=tokens_seen,
                      assistant_tokens_seen=assistant_tokens_seen, sample_cursor=cursor)
        with (work / "metrics.jsonl").open("a") as stream:
            stream.write(json.dumps(values, allow_nan=False) + "\n")
        if values.get("event") == "validation":
            count = len(val_data) if values.get("full_holdout") else min(len(val_data), s["eval_batches"] * s["micro_batch"])
            atomic_json(work / "evaluation.json", dict(
                values, evaluated_samples=count, available_validation_samples=len(val_data), data_sha256=manifest_hash,
                base_sha256=base_hash, base_step=origin["step"], objective="assistant-token-mean",
                tokenizer_sha256=tokenizer_hash, renderer_format=D.RENDER_FORMAT))
        print(json.dumps(values, allow_nan=False), flush=True)

    def save(writer):
        state = capture_rng(device)
        rank_states = [state]
        if world > 1:
            rank_states = [None] * world
            dist.all_gather_object(rank_states, state, group=control)
        writer.submit(state_factory=lambda: dict(
            format=FORMAT, signature=signature, origin=origin, config=vars(cfg).copy(), model=clean_state_dict(raw),
            optimizer=optimizer.state_dict(), step=step, sample_cursor=cursor, tokens_seen=tokens_seen,
            assistant_tokens_seen=assistant_tokens_seen, val_loss=last_validation, val_step=last_validation_step,
            rng_by_rank=rank_states, completed=step >= total_steps, total_steps=total_steps))

    def stop_requested():
        flag = STOP or bool(args.stop_file and args.stop_file.exists())
        if world > 1:
            t = torch.tensor([int(flag)])
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=control)
            return bool(t.item())
        return flag

    with DistributedCheckpointWriter(latest, rank=rank, device=device, distributed=world > 1,
                                     control_group=control) as writer:
        last_validation, eval_tokens = validation(full=True)
        last_validation_step = step
        metric(dict(event="validation", val_loss=last_validation, val_perplexity=math.exp(last_validation),
                    validation_assistant_tokens=eval_tokens, full_holdout=True))
        last_saved_step = step if resuming else -1
        raw.train()
        while step < end_step and not stop_requested():
            writer.check()
            indices, next_cursor = D.update_indices(len(train_data), s["seed"], cursor, s["epochs"], global_batch)
            if not indices:
                break
            global_targets = sum(D.supervised_count(train_data[i]) for i in indices)
            rows = D.rank_microbatches(indices, train_data, s["micro_batch"], s["grad_accum"], world, rank)
            microbatches = [D.collate(r, s["sequence_length"], pad_id) for r in rows]
            lr = learning_rate(step, total_steps, s)
            started = time.perf_counter()
            loss, grad_norm = training_update(trainer, microbatches, global_targets, lr)
            seconds = time.perf_counter() - started
            step += 1
            cursor = next_cursor
            actual_tokens = sum(len(train_data[i]["input_ids"]) - 1 for i in indices)
            tokens_seen += actual_tokens
            assistant_tokens_seen += global_targets
            metric(dict(event="train", loss=loss, lr=lr, grad_norm=grad_norm, update_seconds=seconds,
                        tokens_per_second=actual_tokens / seconds,
                        assistant_tokens_per_second=global_targets / seconds, update_samples=len(indices)))
            if step % s["eval_every"] == 0 or step == end_step:
                full = step >= total_steps
                last_validation, eval_tokens = validation(full=full)
                last_validation_step = step
                metric(dict(event="validation", val_loss=last_validation, val_perplexity=math.exp(last_validation),
                            validation_assistant_tokens=eval_tokens, full_holdout=full))
            if step % s["save_every"] == 0 or step == end_step:
                save(writer)
                last_saved_step = step
        if last_saved_step != step:
            save(writer)
        writer.flush()
        if rank == 0 and step >= total_steps:
            atomic_json(work / "completion.json", dict(
                format="warpstate-posttrain-completion-v1", stage="sft", completed=True, paused_for_evaluation=True,
                step=step, total_steps=total_steps, base_step=origin["step"], tokens_seen=tokens_seen,
                assistant_tokens_seen=assistant_tokens_seen, val_loss=last_validation,
                evaluation_file=str(work / "evaluation.json"), checkpoint=str(latest), timestamp=time.time()))
        metric(dict(event="complete" if step >= total_steps else "paused", total_steps=total_steps,
                    checkpoint=str(latest)))
    if world > 1:
        dist.destroy_process_group()


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description="WarpState assistant-only SFT")
    for name in ("config", "work-dir", "data-dir", "weights", "tokenizer"):
        parser.add_argument("--" + name, type=Path, required=True)
    parser.add_argument("--max-steps", type=int, help="pause after this many additional updates; schedule unchanged")
    parser.add_argument("--stop-file", type=Path, help="defaults to work-dir/control/training-stop-request")
    parser.add_argument("--device", choices=("cuda", "cpu"), default="cuda")
    args = parser.parse_args(argv)
    if args.stop_file is None:
        args.stop_file = args.work_dir / "control/training-stop-request"
    if args.max_steps is not None and args.max_steps < 1:
        parser.error("--max-steps must be positive")
    if not args.stop_file.resolve().is_relative_to(workspace()):
        parser.error("--stop-file must stay inside the workspace")

    def stop(signum, frame):
        global STOP
        STOP = True

    signal.signal(signal.SIGTERM, stop)
    signal.signal(signal.SIGINT, stop)
    rank = int(os.environ.get("RANK", "0"))
    validate_paths(args.work_dir, args.data_dir, args.weights, args.tokenizer, args.config)
    lock_dir = args.work_dir.resolve()
    lock_dir.mkdir(parents=True, exist_ok=True)
    plan, _ = load_plan(args.config)
    # one lock file per rank: a duplicate launch of a rank is refused without serialising the ranks
    with process_lock(lock_dir / f"rank-{rank}.lock"), base_pipeline_lock(plan):
        train(args)


if __name__ == "__main__":
    main()
