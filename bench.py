"""Headline benchmark: 2.005 B WarpState pretraining update, tokens/sec.

    python bench.py --gpus 1 --steps 5 --warmup 3            # this framework
    python bench.py --impl reference --gpus 1 ...             # the unmodified reference (baseline/_ref)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (both arms): 2,005,111,424-parameter model, seq 2048, micro-batch 8 x accumulation 4 per
GPU (65,536 tokens per GPU per update; weak scaling), BF16 compute with FP32 master weights,
gradients and AdamW moments, uniform-random tokens, normal(0, 0.02) random-init weights.

Two timed regions, each of exactly --steps updates after --warmup untimed ones, bracketed by a
barrier and a device synchronize, max over ranks:
  * `value`: CUDA-event time of updates whose micro-batches are already resident on the device;
  * `e2e`: wall-clock time of `Trainer.pretrain_update`, the public call, which every step copies
    its micro-batches from pinned host memory and reads loss and gradient norm back to the host.
Inputs are larger than L2 by construction (8 GB of gradients, 4 GB of BF16 weights and tens of GB
of activations stream through every update).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
BASELINE_TOKS = 72499.0  # published 1xB200 median (reference ops/B200_PERFORMANCE.md:54), mb16 x acc4


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", choices=["2b", "smoke"], default="2b")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--grad-accum", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--grad-sync", default="auto", help="auto | fused | nccl (multi-GPU gradient path)")
    ap.add_argument("--shard-optimizer", action="store_true",
                    help="multi-GPU: sharded AdamW state with the fused update-and-broadcast kernel")
    ap.add_argument("--ref-compile-mode", default=os.environ.get("WARPSTATE_REF_COMPILE_MODE", "default"))
    return ap.parse_args()


def dist_setup(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
        args.gpus = world
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    return rank, world, local, device


def barrier_sync(world):
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, world: int, device) -> float:
    import torch
    import torch.distributed as dist
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def model_config(name: str):
    from warpstate_ai_b200.config import warpstate_2b, warpstate_smoke
    cfg = warpstate_2b() if name == "2b" else warpstate_smoke()
    cfg.gradient_checkpointing = False
    return cfg


def emit(args, rank, world, metric_value, ms_per_step, e2e_value, clocks, launches, impl, extra_cfg, h2d, d2h):
    if rank != 0:
        return
    global_batch = args.micro_batch * args.grad_accum * world
    line = {
        "metric": "train tokens/sec @2.005B seq2048 (max over ranks)" if args.model == "2b" else "train tokens/sec (smoke model)",
        "value": metric_value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (metric_value / BASELINE_TOKS) if args.model == "2b" else None,
        "dtype": "bf16", "data": "synthetic uniform-random tokens; random-init normal(0,0.02) weights",
        "impl": impl,
        "config": dict({"model": "warpstate-2.005B" if args.model == "2b" else "warpstate-smoke",
                        "global_batch": global_batch, "seq_len": args.seq_len,
                        "micro_batch": args.micro_batch, "grad_accum": args.grad_accum,
                        "tokens_per_update": global_batch * args.seq_len,
                        "parallelism": f"dp{world}", "master_dtype": "fp32", "grad_dtype": "fp32",
                        "l2": "working set per update (weights 4 GB bf16 + grads 8 GB + activations) far exceeds the 126 MB L2"},
                       **extra_cfg),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------- ours
def run_ours(args):
    import torch
    sys.path.insert(0, str(ROOT))
    rank, world, local, device = dist_setup(args)
    from warpstate_ai_b200 import WarpStateLM
    from warpstate_ai_b200.data.tokens import HostBatcher, SyntheticTokens, update_slices, host_batch
    from warpstate_ai_b200.ops import _ext
    from warpstate_ai_b200.train.engine import Trainer
    from warpstate_ai_b200.utils.clocks import ClockSampler

    _ext.require()
    cfg = model_config(args.model)
    torch.manual_seed(1337)
    with torch.device(device):
        model = WarpStateLM(cfg)
    model.train()
    sync = None
    if world > 1:
        from warpstate_ai_b200.parallel.grad_sync import make_grad_sync
        sync = make_grad_sync(device, world, rank, None, kind=args.grad_sync)
    trainer = Trainer(model, device=device, rank=rank, world_size=world, lr=1.5e-4, weight_decay=0.1,
                      grad_sync=sync, shard_optimizer=args.shard_optimizer)
    mb, T, acc = args.micro_batch, args.seq_len, args.grad_accum
    update_tokens = mb * T * acc * world
    data = SyntheticTokens(update_tokens * 3 + 1, cfg.vocab_size, seed=7)
    batcher = HostBatcher(mb, T, device)
    lr = 1.5e-4

    # ---- device-resident inputs for the kernel-timed region
    resident = []
    for offset, valid in update_slices(update_tokens, mb * T, world, rank):
        x, y = host_batch(data, offset, mb, T, valid)
        resident.append((x.to(device), y.to(device), valid))

    def resident_update():
        trainer.begin_update()
        for index, (x, y, valid) in enumerate(resident):
            def loss_fn(x=x, y=y, valid=valid):
                _, loss = model(x, y, return_logits=False)
                return loss, valid * world / update_tokens, valid / update_tokens
            trainer.micro_step(loss_fn, last=index == len(resident) - 1)
        return trainer.finish_update(lr)

    cursor = 0
    for _ in range(args.warmup):
        trainer.pretrain_update(data, cursor, update_tokens, mb, T, lr, batcher)
        cursor += update_tokens
    # ---- region 1: device-timed
    barrier_sync(world)
    sampler = ClockSampler()
    if rank == 0:
        sampler.start()
    launches0 = _ext.launch_count()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        stats = resident_update()
    stop.record()
    barrier_sync(world)
    launches = _ext.launch_count() - launches0
    dev_s = max_over_ranks(start.elapsed_time(stop) / 1e3, world, device)
    norm = float(stats[0])
    # ---- region 2: end to end through the public API
    barrier_sync(world)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        result = trainer.pretrain_update(data, cursor % update_tokens, update_tokens, mb, T, lr, batcher)
    barrier_sync(world)
    e2e_s = max_over_ranks(time.perf_counter() - t0, world, device)
    clocks = sampler.stop(gpu_indices=None) if rank == 0 else {}
    from warpstate_ai_b200.ops.gemm import check_device_errors
    check_device_errors()
    tokens = update_tokens * args.steps
    h2d = batcher.bytes_per_batch * acc * world
    emit(args, rank, world, tokens / dev_s, dev_s / args.steps * 1e3, tokens / e2e_s, clocks, launches, "ours",
         {"last_loss": result.loss, "last_grad_norm": norm, "grad_sync": getattr(sync, "kind", "none"),
          "optimizer": "sharded" if (args.shard_optimizer and world > 1) else "replicated",
          "peak_mem_gib": torch.cuda.max_memory_allocated(device) / 2**30}, h2d, 12 * world)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------- reference
def run_reference(args):
    """Runs the unmodified reference (its model, compiled cores, compiled full loss, DDP with its
    own kwargs, fused AdamW, its batch/slice helpers) with the update loop of run_40b.train."""
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "warpstate" / "model.py").exists():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}), flush=True)
        return
    sys.path.insert(0, str(ref_root))
    if str(ROOT) in sys.path:
        sys.path.remove(str(ROOT))
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != ROOT]
    sys.path.insert(0, str(ref_root))
    import contextlib
    import numpy as np
    import torch
    import torch.distributed as dist
    try:
        from warpstate import WarpStateConfig, WarpStateLM  # reference package
        import run_40b as ref_run
        from ops.distributed_execution import ddp_kwargs, ddp_runtime_settings
        from ops.gradient_execution import make_backward, scale_loss
        from ops.loss_experiment import apply_loss_execution
    except Exception as error:  # pragma: no cover - depends on the installed torch
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {error!r}"[:300]}), flush=True)
        return
    assert "baseline/_ref" in str(Path(sys.modules["warpstate"].__file__))
    rank, world, local, device = dist_setup(args)
    sys.path.append(str(ROOT))
    from warpstate_ai_b200.utils.clocks import ClockSampler  # telemetry only; not on the reference path
    if args.model == "2b":
        cfg = WarpStateConfig(vocab_size=32768, d_model=2048, n_heads=32, n_cores=28, logical_depth=28,
                              ffn_hidden=7168, chunk_size=128, dropout=0.0, rms_eps=1e-5,
                              gradient_checkpointing=False, parallel_memory=True, loss_chunk_size=128)
    else:
        cfg = WarpStateConfig(vocab_size=32768, d_model=256, n_heads=4, n_cores=2, logical_depth=4,
                              ffn_hidden=688, chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    torch.manual_seed(1337)
    with torch.device(device):
        model = WarpStateLM(cfg)
    model = model.to(device)  # also moves the rope tables, which the reference builds on the CPU
    model.train()
    optimizer = torch.optim.AdamW(model.parameters(), lr=1.5e-4, betas=(0.9, 0.95), eps=1e-8,
                                  weight_decay=0.1, fused=True)
    raw = model
    backward = make_backward("eager", distributed=world > 1, overlap_settings=None)
    ref_run.compile_training_cores(raw, mode=args.ref_compile_mode)
    apply_loss_execution(raw, "compiled-full")
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(
            model, device_ids=[local], output_device=local, **ddp_kwargs(ddp_runtime_settings(bucket_cap_mb=128)))
    mb, T, acc = args.micro_batch, args.seq_len, args.grad_accum
    update_tokens = mb * T * acc * world
    rng = np.random.default_rng(7)
    data = rng.integers(0, cfg.vocab_size, size=update_tokens * 3 + 1, dtype=np.uint16)

    def update(seen):
        optimizer.zero_grad(set_to_none=True)
        loss_sum = torch.zeros((), device=device)
        slices = list(ref_run.update_slices(update_tokens, mb * T, world, rank))
        for index, (offset, valid) in enumerate(slices):
            x, y = ref_run.batches(data, seen + offset, mb, T, valid, device)
            sync = model.no_sync() if world > 1 and index < len(slices) - 1 else contextlib.nullcontext()
            with sync:
                with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=True):
                    _, loss = model(x, y, return_logits=False)
                backward(scale_loss(loss, valid * world / update_tokens, "eager"))
            loss_sum += loss.detach() * (valid / update_tokens)
        norm = torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0, error_if_nonfinite=True)
        optimizer.step()
        if world > 1:
            dist.all_reduce(loss_sum, op=dist.ReduceOp.SUM)
        return float(loss_sum), float(norm)

    seen = 0
    for _ in range(args.warmup):
        update(seen)
        seen += update_tokens
    barrier_sync(world)
    sampler = ClockSampler()
    if rank == 0:
        sampler.start()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(args.steps):
        loss, norm = update(seen % update_tokens)
    stop.record()
    barrier_sync(world)
    wall = max_over_ranks(time.perf_counter() - t0, world, device)
    dev_s = max_over_ranks(start.elapsed_time(stop) / 1e3, world, device)
    clocks = sampler.stop() if rank == 0 else {}
    tokens = update_tokens * args.steps
    emit(args, rank, world, tokens / dev_s, dev_s / args.steps * 1e3, tokens / wall, clocks, 0, "reference",
         {"last_loss": loss, "last_grad_norm": norm, "compile_mode": args.ref_compile_mode,
          "loss_mode": "compiled-full", "ddp_bucket_cap_mb": 128,
          "peak_mem_gib": torch.cuda.max_memory_allocated(device) / 2**30},
         2 * mb * T * 8 * acc * world, 8 * world)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        try:
            run_reference(a)
        except Exception as error:
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"run failed: {error!r}"[:400]}), flush=True)
    else:
        run_ours(a)
