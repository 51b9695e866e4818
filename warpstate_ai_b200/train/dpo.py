"""Direct preference optimisation (the engine behind ``dpo.py``).

Behaviour follows the reference DPO runner (dpo.py:38-647): plan ``warpstate-dpo-plan-v1`` with
`DEFAULTS` (beta 5, length-normalised objective, micro-batch 2 x accumulation 8, lr 5e-7, linear
warm-up / decay); initialisation from an SFT ``warpstate-chat-v1`` export (``stage == 'sft'``);
per-sequence response log-probabilities from a head that never keeps vocabulary logits; the
frozen reference scored ONCE into a cache (float64 ``train.npy`` / ``val.npy`` bound to an
identity hash, built from resumable per-rank shards); loss ``-log sigmoid(r_chosen - r_rejected)``
with ``r = beta * (pi - ref)`` (divided by response length when length-normalised), averaged
over the global pair count; metrics loss / reward_margin / reward_accuracy / chosen_nll;
checkpoints ``warpstate-dpo-v1``.

Added here: ``reference_mode = "resident"`` keeps a frozen BF16 copy of the reference on the GPU
and scores it every step instead of reading the cache (the two modes are interchangeable; the
cache is still what makes a run resumable without re-scoring).
"""
from __future__ import annotations

import argparse
import gc
import hashlib
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
import torch.nn.functional as F

from ..ckpt.formats import CHAT_FORMAT, DPO_FORMAT, capture_rng, clean_state_dict, restore_rng
from ..data import dpo as D
from ..data.sft import RENDER_FORMAT, renderer_sha256, update_indices
from ..utils.io import atomic_json, digest, process_lock
from .sft import base_pipeline_lock, validate_paths, workspace
from .sft import source_identity as sft_sources

FORMAT = DPO_FORMAT
CACHE_FORMAT = "warpstate-dpo-reference-v1"
STOP = False
DEFAULTS = dict(sequence_length=2048, micro_batch=2, grad_accum=8, lr=5e-7, min_lr=0.0, warmup_ratio=0.1, epochs=1,
                max_steps=None, weight_decay=0.0, seed=42, eval_every=100, save_every=100, eval_batches=32,
                compile_core=True, bf16_residuals=True, gradient_checkpointing=False, workers=4, deterministic=True,
                clip_grad_norm=1.0, beta=5.0, objective="length-normalized-dpo", head_chunk_size=256,
                reference_mode="cached")


def load_plan(path):
    plan = json.loads(Path(path).read_text())
    if plan.get("format") != "warpstate-dpo-plan-v1" or plan.get("stage") != "dpo":
        raise ValueError("Expected warpstate-dpo-plan-v1 stage dpo")
    supplied = plan.get("training", {})
    unknown = set(supplied) - set(DEFAULTS)
    if unknown:
        raise ValueError(f"Unknown DPO training settings: {sorted(unknown)}")
    s = DEFAULTS | supplied
    for key in ("sequence_length", "micro_batch", "grad_accum", "epochs", "eval_every", "save_every", "eval_batches",
                "workers", "head_chunk_size"):
        if type(s[key]) is not int or s[key] < 1:
            raise ValueError(f"{key} must be a positive integer")
    if s["max_steps"] is not None and (type(s["max_steps"]) is not int or s["max_steps"] < 1):
        raise ValueError("max_steps must be null or a positive integer")
    for key in ("lr", "min_lr", "warmup_ratio", "weight_decay", "clip_grad_norm", "beta"):
        v = s[key]
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v < 0:
            raise ValueError(f"{key} must be finite and nonnegative")
    if not 0 <= s["warmup_ratio"] < 1 or not 0 <= s["min_lr"] <= s["lr"]:
        raise ValueError("Invalid LR schedule")
    if not s["lr"] or not s["clip_grad_norm"] or not s["beta"]:
        raise ValueError("lr, clip_grad_norm and beta must be positive")
    for key in ("compile_core", "bf16_residuals", "gradient_checkpointing", "deterministic"):
        if type(s[key]) is not bool:
            raise ValueError(f"{key} must be a boolean")
    if type(s["seed"]) is not int or s["seed"] < 0:
        raise ValueError("seed must be a nonnegative integer")
    if s["objective"] not in ("length-normalized-dpo", "summed-dpo"):
        raise ValueError("Unsupported DPO objective")
    if s["reference_mode"] not in ("cached", "resident"):
        raise ValueError("reference_mode must be 'cached' or 'resident'")
    return plan, s


def source_identity() -> dict:
    root = Path(__file__).resolve().parents[1]
    return sft_sources() | {str(p.relative_to(root)): digest(p) for p in (Path(__file__), root / "data/dpo.py")}


def identity_digest(identity) -> str:
    return hashlib.sha256(json.dumps(identity, sort_keys=True, separators=(",", ":"), allow_nan=False).encode()).hexdigest()


def learning_rate(step: int, total_steps: int, s: dict) -> float:
    """Linear warm-up then linear decay, independent of pause boundaries."""
    warmup = min(math.ceil(s["warmup_ratio"] * total_steps), max(0, total_steps - 1))
    if step < warmup:
        return s["lr"] * (step + 1) / warmup
    progress = min(1.0, (step - warmup) / max(1, total_steps - warmup - 1))
    return s["min_lr"] + (s["lr"] - s["min_lr"]) * (1.0 - progress)


def preference_metrics(policy, reference, counts, beta: float, objective: str):
    """Per-pair (loss, margin, accuracy); gradients flow through the policy scores only."""
    reference = reference.detach().to(policy.dtype)
    if objective == "length-normalized-dpo":
        policy = policy / counts.clamp_min(1)
        reference = reference / counts.clamp_min(1)
    elif objective != "summed-dpo":
        raise ValueError("Unsupported DPO objective")
    rewards = beta * (policy - reference)
    margin = rewards[:, 0] - rewards[:, 1]
    return -F.logsigmoid(margin), margin, (margin > 0).to(policy.dtype)


def reference_identity(weights_hash, manifest_hash, tokenizer_hash, s, device, world) -> dict:
    keys = ("sequence_length", "micro_batch", "head_chunk_size", "compile_core", "bf16_residuals", "deterministic",
            "workers")
    return dict(format=CACHE_FORMAT, weights_sha256=weights_hash, data_sha256=manifest_hash,
                tokenizer_sha256=tokenizer_hash, renderer_sha256=renderer_sha256(), mask_format=D.MASK_FORMAT,
                sources=source_identity(), settings={k: s[k] for k in keys}, dropout=0.0,
                logps="response-token-sum-float32", dtype="bfloat16", device_type=device.type, world_size=world,
                torch_version=torch.__version__)


def validate_cache(directory, identity, sizes):
    directory = Path(directory)
    manifest = json.loads((directory / "manifest.json").read_text())
    if (manifest.get("format") != CACHE_FORMAT or manifest.get("complete") is not True
            or manifest.get("identity") != identity or manifest.get("identity_sha256") != identity_digest(identity)):
        raise ValueError("Reference cache identity/completion differs")
    arrays = []
    for name, size in zip(("train.npy", "val.npy"), sizes):
        path = directory / name
        info = manifest.get("files", {}).get(name, {})
        if not path.is_file() or path.is_symlink() or digest(path) != info.get("sha256") or info.get("rows") != size:
            raise ValueError(f"Reference cache file changed: {name}")
        values = np.load(path, allow_pickle=False, mmap_mode="r")
        if values.shape != (size, 2) or values.dtype != np.float64 or not np.isfinite(values).all():
            raise ValueError(f"Invalid reference log probabilities: {name}")
        arrays.append(values)
    return arrays[0], arrays[1], digest(directory / "manifest.json")


def stop_requested(args, world: int, control=None) -> bool:
    value = STOP or bool(args.stop_file and Path(args.stop_file).exists())
    if world > 1:
        t = torch.tensor([int(value)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=control)
        value = bool(t.item())
    return value


def load_model(checkpoint, s, device, tokenizer, dtype=torch.float32):
    from ..config import WarpStateConfig
    from ..models.warpstate import WarpStateLM
    cfg = WarpStateConfig(**checkpoint["config"])
    cfg.gradient_checkpointing = s["gradient_checkpointing"]
    cfg.dropout = 0.0  # policy and reference are compared under a deterministic scoring rule
    cfg.validate()
    if cfg.vocab_size != tokenizer.vocab_size() or s["sequence_length"] % cfg.chunk_size:
        raise ValueError("Model/tokenizer vocabulary or sequence/chunk mismatch")
    with torch.device("meta"):
        raw = WarpStateLM(cfg)
    raw.load_state_dict(checkpoint["model"], strict=True, assign=True)
    raw = raw.to(device=device, dtype=dtype)
    if device.type == "cpu":
        for p in raw.parameters():  # an mmap-backed initialisation must not alias training state
            p.data = p.data.clone()
    return raw, cfg


def score_pairs(model, x, y, device, head_chunk_size: int):
    from .engine import autocast_for
    with autocast_for(device):
        return model.sequence_logps(x, y, head_chunk_size)


def atomic_array(path, array) -> None:
    temporary = Path(str(path) + ".tmp")
    with temporary.open("wb") as stream:
        np.save(stream, array, allow_pickle=False)
        stream.flush()
        os.fsync(stream.fileno())
    os.replace(temporary, path)


# --------------------------------------------------------------------------- frozen reference cache
def prepare_reference(args, identity, records, s, device, rank, world, tokenizer, control=None):
    """Create or reuse the reference-score cache.  Every rank scores the batches
    ``rank*mb, rank*mb + world*mb, ...`` of each split into a resumable ``.npz`` shard; rank 0
    merges the shards, seals ``train.npy`` / ``val.npy`` + manifest.  Returns ``None`` if a stop
    request interrupted scoring (shards are kept)."""
    from ..ckpt.formats import load_checkpoint
    directory = Path(args.reference_cache_dir)
    if (directory / "manifest.json").exists():
        return validate_cache(directory, identity, [len(rows) for rows in records])
    directory.mkdir(parents=True, exist_ok=True)
    marker = directory / "identity.json"
    if marker.exists() and json.loads(marker.read_text()) != identity:
        raise ValueError("Partial reference cache identity differs")
    if rank == 0:
        atomic_json(marker, identity)
    if world > 1:
        dist.barrier(group=control)
    raw, _ = load_model(load_checkpoint(args.weights), s, device, tokenizer)
    raw.requires_grad_(False).eval()
    pad_id = tokenizer.pad_id() if tokenizer.pad_id() >= 0 else tokenizer.eos_id()
    started = time.monotonic()
    mb = s["micro_batch"]
    try:
        for split, rows in zip(("train", "val"), records):
            starts = list(range(rank * mb, len(rows), world * mb))
            shard = directory / f"{split}-rank-{rank}.npz"
            done, scored, scores = 0, [], []
            if shard.exists():
                with np.load(shard, allow_pickle=False) as old:
                    if str(old["identity"]) != identity_digest(identity):
                        raise ValueError("Partial reference shard identity differs")
                    done, scored, scores = int(old["batches"]), old["indices"].tolist(), old["scores"].tolist()
                expected = [i for st in starts[:done] for i in range(st, min(st + mb, len(rows)))]
                if scored != expected or len(scores) != len(scored):
                    raise ValueError("Partial reference shard cursor differs")

            def save_shard():
                temporary = Path(str(shard) + ".tmp")
                with temporary.open("wb") as stream:
                    np.savez(stream, identity=identity_digest(identity), batches=done,
                             indices=np.asarray(scored, dtype=np.int64),
                             scores=np.asarray(scores, dtype=np.float64).reshape(-1, 2))
                    stream.flush()
                    os.fsync(stream.fileno())
                os.replace(temporary, shard)

            # every rank runs the same number of stop checks, also on an uneven final shard
            for batch in range(math.ceil(len(rows) / (world * mb))):
                if stop_requested(args, world, control):
                    save_shard()
                    return None
                if batch < done or batch >= len(starts):
                    continue
                chosen = list(range(starts[batch], min(starts[batch] + mb, len(rows))))
                padded = [rows[i] for i in chosen] + [None] * (mb - len(chosen))
                x, y, _ = D.collate_pairs(padded, s["sequence_length"], pad_id)
                with torch.no_grad():
                    logps = score_pairs(raw, x.to(device), y.to(device), device, s["head_chunk_size"])
                values = logps.reshape(-1, 2).double().cpu().numpy()[:len(chosen)]
                if not np.isfinite(values).all():
                    raise RuntimeError("Non-finite frozen reference scores")
                scored.extend(chosen)
                scores.extend(values.tolist())
                done = batch + 1
                if done % 128 == 0 or done == len(starts):
                    save_shard()
                    print(json.dumps(dict(event="reference_progress", rank=rank, split=split, batches=done,
                                          total_batches=len(starts), scored_pairs=len(scores),
                                          elapsed_seconds=time.monotonic() - started)), flush=True)
            save_shard()
        if world > 1:
            dist.barrier(group=control)
        if rank == 0:
            files = {}
            for split, rows in zip(("train", "val"), records):
                combined = np.full((len(rows), 2), np.nan, dtype=np.float64)
                seen = np.zeros(len(rows), dtype=np.bool_)
                for owner in range(world):
                    with np.load(directory / f"{split}-rank-{owner}.npz", allow_pickle=False) as part:
                        if str(part["identity"]) != identity_digest(identity):
                            raise ValueError("Reference shard identity differs")
                        index = part["indices"]
                        if seen[index].any():
                            raise ValueError("Duplicate reference indices")
                        combined[index] = part["scores"]
                        seen[index] = True
                if not seen.all() or not np.isfinite(combined).all():
                    raise ValueError("Reference cache is incomplete")
                path = directory / f"{split}.npy"
                atomic_array(path, combined)
                files[path.name] = dict(sha256=digest(path), rows=len(rows))
            atomic_json(directory / "manifest.json", dict(format=CACHE_FORMAT, complete=True, identity=identity,
                                                          identity_sha256=identity_digest(identity), files=files))
        if world > 1:
            dist.barrier(group=control)
        return validate_cache(directory, identity, [len(rows) for rows in records])
    finally:
        del raw
        gc.collect()
        if device.type == "cuda":
            torch.cuda.empty_cache()


# --------------------------------------------------------------------------- update / evaluation
def training_update(trainer, microbatches, global_pairs: int, s: dict, lr: float, resident=None, control=None):
    """One DPO update.  ``microbatches`` hold (x, y, active, reference_logps[mb,2])."""
    world, device = trainer.world_size, trainer.device
    totals = torch.zeros(5, device=device, dtype=torch.float64)
    trainer.begin_update()
    for index, (x, y, active, reference) in enumerate(microbatches):
        x, y, active, reference = (v.to(device) for v in (x, y, active, reference))
        counts = y.ne(-100).sum(dim=1).reshape(-1, 2)
        if resident is not None:
            with torch.no_grad():
                reference = score_pairs(resident, x, y, device, s["head_chunk_size"]).reshape(-1, 2)

        def loss_fn(x=x, y=y, active=active, reference=reference, counts=counts):
            logps = trainer.model.sequence_logps(x, y, s["head_chunk_size"]).reshape(-1, 2)
            losses, margins, accuracy = preference_metrics(logps, reference, counts, s["beta"], s["objective"])
            nonlocal totals
            totals = totals + torch.stack((
                (losses.detach() * active).double().sum(), (margins.detach() * active).double().sum(),
                (accuracy.detach() * active).double().sum(),
                ((-logps[:, 0].detach() / counts[:, 0].clamp_min(1)) * active).double().sum(), active.double().sum()))
            # rank averaging divides by world: scale so the result is the global pair mean
            return (losses * active).sum(), world / global_pairs, 0.0

        trainer.micro_step(loss_fn, last=index == len(microbatches) - 1)
    stats = trainer.finish_update(lr)
    if world > 1:
        dist.all_reduce(totals)
    _, norm, _ = trainer.read_update_scalars(stats)
    host = totals.tolist()
    if int(host[-1]) != global_pairs:
        raise RuntimeError("Distributed DPO pair count differs")
    values = [v / host[-1] for v in host[:4]]
    if not all(math.isfinite(v) for v in values) or not math.isfinite(norm):
        raise RuntimeError("Non-finite DPO training loss")
    return dict(zip(("loss", "reward_margin", "reward_accuracy", "chosen_nll"), values)), norm


@torch.no_grad()
def evaluate(trainer, records, reference, s, pad_id, *, full=False, resident=None):
    model, device = trainer.model, trainer.device
    state = capture_rng(device)
    was_training = model.training
    model.eval()
    totals = torch.zeros(4, dtype=torch.float64, device=device)
    count = 0
    mb = s["micro_batch"]
    limit = len(records) if full else min(len(records), s["eval_batches"] * mb)
    try:
        for start in range(0, limit, mb):
            chosen = list(records[start:min(start + mb, limit)])
            n = len(chosen)
            chosen += [None] * (mb - n)
            x, y, active = D.collate_pairs(chosen, s["sequence_length"], pad_id)
            x, y, active = x.to(device), y.to(device), active.to(device)
            if resident is not None:
                ref = score_pairs(resident, x, y, device, s["head_chunk_size"]).reshape(-1, 2)
            else:
                ref = torch.zeros((mb, 2), device=device)
                ref[:n] = torch.tensor(np.array(reference[start:start + n]), device=device)
            logps = score_pairs(model, x, y, device, s["head_chunk_size"]).reshape(-1, 2)
            counts = y.ne(-100).sum(dim=1).reshape(-1, 2)
            losses, margins, accuracy = preference_metrics(logps, ref, counts, s["beta"], s["objective"])
            totals += torch.stack(((losses * active).double().sum(), (margins * active).double().sum(),
                                   (accuracy * active).double().sum(),
                                   ((-logps[:, 0] / counts[:, 0].clamp_min(1)) * active).double().sum()))
            count += n
    finally:
        model.train(was_training)
        restore_rng(state, device)
    values = (totals / count).tolist()
    if not all(math.isfinite(v) for v in values):
        raise RuntimeError("Non-finite DPO validation")
    return dict(zip(("val_loss", "reward_margin", "reward_accuracy", "chosen_nll"), values)) | dict(evaluated_samples=count)


def validate_resume(checkpoint, signature, world):
    if checkpoint.get("format") != FORMAT or checkpoint.get("signature") != signature:
        raise ValueError("DPO resume signature differs; use a new output directory")
    if len(checkpoint.get("rng_by_rank", [])) != world:
        raise ValueError("DPO checkpoint lacks exact per-rank RNG state")


def validate_reference_path(args):
    root = workspace()
    cache = Path(args.reference_cache_dir).resolve()
    others = [Path(p).resolve() for p in (args.work_dir, args.data_dir, args.weights.parent)]
    if not cache.is_relative_to(root) or cache == root:
        raise ValueError("Reference cache must stay inside the workspace")
    if any(cache == p or cache.is_relative_to(p) or p.is_relative_to(cache) for p in others):
        raise ValueError("Reference cache must be separate from training outputs and inputs")
    return cache


# --------------------------------------------------------------------------- the run
def train(args) -> None:
    import sentencepiece as spm
    from ..ckpt.formats import load_checkpoint
    from ..ckpt.writer import DistributedCheckpointWriter, host_control_group
    from .engine import Trainer

    work, data_dir, weights, tokenizer_path, config = validate_paths(args.work_dir, args.data_dir, args.weights,
                                                                     args.tokenizer, args.config)
    cache = validate_reference_path(args)
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
    tokenizer_hash, base_hash = digest(tokenizer_path), digest(weights)
    sp = spm.SentencePieceProcessor(model_file=str(tokenizer_path))
    train_data, val_data, manifest, manifest_hash = D.load_data(data_dir, sp, tokenizer_hash, s["sequence_length"])
    source = load_checkpoint(weights)
    if (source.get("format") != CHAT_FORMAT or source.get("inference_only") is not True
            or source.get("stage") != "sft" or source.get("tokenizer_sha256") != tokenizer_hash):
        raise ValueError("Initialize DPO from an independent, tokenizer-matched SFT model export")
    expected = plan.get("sft", plan.get("base", {}))
    for key in ("step", "tokens_seen", "tokenizer_sha256"):
        if key in expected and expected[key] != source.get(key):
            raise ValueError(f"SFT source {key} differs from plan")
    ancestor = source.get("origin") or {}
    for key in ("step", "tokens_seen"):
        expected_key = "base_" + key
        if expected_key in expected and expected[expected_key] != ancestor.get(key, ancestor.get(expected_key)):
            raise ValueError(f"SFT source {expected_key} differs from plan")
    origin = {k: v for k, v in source.items() if k != "model"}
    origin.update(weights_sha256=base_hash, weights_path=str(weights))
    del source
    identity = reference_identity(base_hash, manifest_hash, tokenizer_hash, s, device, world)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if device.type == "cuda":
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group("gloo")
    control = host_control_group() if world > 1 else None
    try:
        reference = prepare_reference(args, identity, (train_data, val_data), s, device, rank, world, sp, control)
        if reference is None:
            print(json.dumps(dict(event="reference_paused", rank=rank)), flush=True)
            return
        reference_train, reference_val, reference_hash = reference
        if getattr(args, "reference_only", False):
            print(json.dumps(dict(event="reference_complete", reference_sha256=reference_hash)), flush=True)
            return
        signature = dict(plan=plan, settings=s, data_sha256=manifest_hash, tokenizer_sha256=tokenizer_hash,
                         renderer=RENDER_FORMAT, mask=D.MASK_FORMAT, base_sha256=base_hash,
                         reference_sha256=reference_hash, world_size=world, device_type=device.type,
                         torch_version=torch.__version__, sources=source_identity())
        latest = work / "latest.pt"
        resuming = latest.exists()
        saved = load_checkpoint(latest if resuming else weights)
        if resuming:
            validate_resume(saved, signature, world)
            origin = saved["origin"]
        raw, cfg = load_model(saved, s, device, sp)
        raw.requires_grad_(True)
        resident = None
        if s["reference_mode"] == "resident":
            resident, _ = load_model(load_checkpoint(weights), s, device, sp,
                                     dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
            resident.requires_grad_(False).eval()
        trainer = Trainer(raw, device=device, rank=rank, world_size=world, lr=s["lr"], weight_decay=s["weight_decay"],
                          max_grad_norm=s["clip_grad_norm"])
        optimizer = trainer.optimizer
        step = cursor = tokens_seen = response_tokens_seen = 0
        if resuming:
            optimizer.load_state_dict(saved["optimizer"])
            step, cursor = saved["step"], saved["sample_cursor"]
            tokens_seen, response_tokens_seen = saved["tokens_seen"], saved["response_tokens_seen"]
            restore_rng(saved["rng_by_rank"][rank], device)
        del saved
        global_batch = s["micro_batch"] * s["grad_accum"] * world
        total_steps = math.ceil(len(train_data) / global_batch) * s["epochs"]
        if s["max_steps"] is not None:
            total_steps = min(total_steps, s["max_steps"])
        end_step = min(total_steps, step + args.max_steps) if args.max_steps is not None else total_steps
        work.mkdir(parents=True, exist_ok=True)
        if rank == 0:
            (work / "settings.json").write_text(json.dumps(dict(signature=signature, origin=origin,
                                                                total_steps=total_steps, train_rows=len(train_data),
                                                                val_rows=len(val_data)), indent=2, default=str))
            if step < total_steps:
                (work / "completion.json").unlink(missing_ok=True)
        pad_id = sp.pad_id() if sp.pad_id() >= 0 else sp.eos_id()
        last_validation = last_validation_step = None

        def validation(full=False):
            values = [evaluate(trainer, val_data, reference_val, s, pad_id, full=full, resident=resident)
                      if rank == 0 else None]
            if world > 1:
                dist.broadcast_object_list(values, src=0, group=control)
            return values[0]

        def metric(values):
            if rank != 0:
                return
            values.update(timestamp=time.time(), stage="dpo", step=step, tokens_seen=tokens_seen,
                          response_tokens_seen=response_tokens_seen, sample_cursor=cursor, objective=s["objective"])
            with (work / "metrics.jsonl").open("a") as stream:
                stream.write(json.dumps(values, allow_nan=False) + "\n")
            if values.get("event") == "validation":
                atomic_json(work / "evaluation.json", dict(
                    values, data_sha256=manifest_hash, base_sha256=base_hash, reference_sha256=reference_hash,
                    tokenizer_sha256=tokenizer_hash, mask_format=D.MASK_FORMAT,
                    available_validation_samples=len(val_data)))
            print(json.dumps(values, allow_nan=False), flush=True)

        def save(writer):
            state = capture_rng(device)
            states = [state]
            if world > 1:
                states = [None] * world
                dist.all_gather_object(states, state, group=control)
            writer.submit(state_factory=lambda: dict(
                format=FORMAT, signature=signature, origin=origin, config=vars(cfg).copy(),
                model=clean_state_dict(raw), optimizer=optimizer.state_dict(), step=step, sample_cursor=cursor,
                tokens_seen=tokens_seen, response_tokens_seen=response_tokens_seen,
                val_loss=last_validation["val_loss"], validation=last_validation, val_step=last_validation_step,
                rng_by_rank=states, completed=step >= total_steps, total_steps=total_steps))

        with DistributedCheckpointWriter(latest, rank=rank, device=device, distributed=world > 1,
                                         control_group=control) as writer:
            last_validation = validation(full=True)
            last_validation_step = step
            metric(dict(event="validation", full_holdout=True, **last_validation))
            last_saved_step = step if resuming else -1
            raw.train()
            while step < end_step and not stop_requested(args, world, control):
                writer.check()
                indices, next_cursor = update_indices(len(train_data), s["seed"], cursor, s["epochs"], global_batch)
                if not indices:
                    break
                microbatches = []
                for micro in range(s["grad_accum"]):
                    offset = (micro * world + rank) * s["micro_batch"]
                    chosen = indices[offset:offset + s["micro_batch"]]
                    padded = [train_data[i] for i in chosen] + [None] * (s["micro_batch"] - len(chosen))
                    x, y, active = D.collate_pairs(padded, s["sequence_length"], pad_id)
                    ref = torch.zeros((s["micro_batch"], 2), dtype=torch.float32)
                    if chosen:
                        ref[:len(chosen)] = torch.tensor(np.array(reference_train[chosen]), dtype=torch.float32)
                    microbatches.append((x, y, active, ref))
                lr = learning_rate(step, total_steps, s)
                started = time.perf_counter()
                values, norm = training_update(trainer, microbatches, len(indices), s, lr, resident, control)
                seconds = time.perf_counter() - started
                step += 1
                cursor = next_cursor
                actual_tokens = sum(D.pair_tokens(train_data[i]) for i in indices)
                tokens_seen += actual_tokens
                response_tokens_seen += sum(D.pair_targets(train_data[i]) for i in indices)
                metric(dict(event="train", **values, lr=lr, grad_norm=norm, update_seconds=seconds,
                            tokens_per_second=actual_tokens / seconds, pairs_per_second=len(indices) / seconds,
                            update_samples=len(indices)))
                if step % s["eval_every"] == 0 or step == end_step:
                    full = step >= total_steps
                    last_validation = validation(full=full)
                    last_validation_step = step
                    metric(dict(event="validation", full_holdout=full, **last_validation))
                if step % s["save_every"] == 0 or step == end_step:
                    save(writer)
                    last_saved_step = step
            if last_saved_step != step:
                save(writer)
            writer.flush()
            if rank == 0 and step >= total_steps:
                atomic_json(work / "completion.json", dict(
                    format="warpstate-dpo-completion-v1", stage="dpo", completed=True, paused_for_evaluation=True,
                    step=step, total_steps=total_steps, sample_cursor=cursor, tokens_seen=tokens_seen,
                    response_tokens_seen=response_tokens_seen, val_loss=last_validation["val_loss"],
                    evaluation_file=str(work / "evaluation.json"), checkpoint=str(latest),
                    reference_sha256=reference_hash, timestamp=time.time()))
            metric(dict(event="complete" if step >= total_steps else "paused", total_steps=total_steps,
                        checkpoint=str(latest)))
        validate_cache(cache, identity, (len(train_data), len(val_data)))
        if digest(weights) != base_hash:
            raise RuntimeError("Frozen SFT initialization changed during DPO")
    finally:
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description="WarpState DPO")
    for name in ("config", "work-dir", "data-dir", "weights", "tokenizer", "reference-cache-dir"):
        parser.add_argument("--" + name, required=True, type=Path)
    parser.add_argument("--max-steps", type=int)
    parser.add_argument("--stop-file", type=Path)
    parser.add_argument("--device", choices=("cuda", "cpu"), default="cuda")
    parser.add_argument("--reference-only", action="store_true")
    args = parser.parse_args(argv)
    if args.max_steps is not None and args.max_steps < 1:
        parser.error("--max-steps must be positive")
    if args.stop_file is None:
        args.stop_file = args.work_dir / "control/training-stop-request"
    if not args.stop_file.resolve().is_relative_to(workspace()):
        parser.error("--stop-file must stay inside the workspace")

    def stop(signum, frame):
        global STOP
        STOP = True

    for signum in (signal.SIGTERM, signal.SIGINT, signal.SIGUSR1):
        signal.signal(signum, stop)
    validate_paths(args.work_dir, args.data_dir, args.weights, args.tokenizer, args.config)
    validate_reference_path(args)
    args.work_dir.mkdir(parents=True, exist_ok=True)
    args.reference_cache_dir.mkdir(parents=True, exist_ok=True)
    plan, _ = load_plan(args.config)
    rank = int(os.environ.get("RANK", "0"))
    with process_lock(args.work_dir / f"rank-{rank}.lock"), \
            process_lock(args.reference_cache_dir / f"rank-{rank}.lock"), base_pipeline_lock(plan):
        train(args)


if __name__ == "__main__":
    main()
