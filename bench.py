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
of activations stream through every update).  Every update (warm-up and timed, both regions, both
arms) reads the next window of the token stream, so no batch is seen twice.

The JSON line keeps the workload definition in `config` (identical in both arms), what the arm is
built from in `arm`, and what the run produced (loss, gradient norm, peak memory) in `result`.
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
    ap.add_argument("--shard-params", choices=["off", "stream", "resident"], default="off",
                    help="fully sharded parameters, gradients and optimizer state for the core projections "
                         "(stream: re-gather every use; resident: keep the gathered BF16 weights for the update)")
    ap.add_argument("--activation-checkpointing", action="store_true")
    ap.add_argument("--bf16-residuals", action="store_true")
    ap.add_argument("--ref-compile-mode", default=os.environ.get("WARPSTATE_REF_COMPILE_MODE", "max-autotune-no-cudagraphs"),
                    help="torch.compile mode of the reference arm's cores; the default is the reference's own B200 preset "
                         "(its ops/train-b200.sh), whose compilation takes about a minute here")
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


def emit(args, rank, world, metric_value, ms_per_step, e2e_value, clocks, launches, impl, arm, result, h2d, d2h):
    """One JSON line from rank 0.  `config` names the workload and is the same dict in both arms; `arm` says
    what this arm is built from; `result` is what the run produced."""
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
        "config": {"model": "warpstate-2.005B" if args.model == "2b" else "warpstate-smoke",
                   "global_batch": global_batch, "seq_len": args.seq_len,
                   "micro_batch": args.micro_batch, "grad_accum": args.grad_accum,
                   "tokens_per_update": global_batch * args.seq_len,
                   "parallelism": f"dp{world}", "master_dtype": "fp32", "grad_dtype": "fp32",
                   "batches": "a fresh window of the token stream every update",
                   "l2": "working set per update (weights 4 GB bf16 + grads 8 GB + activations) far exceeds the 126 MB L2",
                   "value_region": "device-timed updates on micro-batches already resident on the device",
                   "e2e_region": "public update call: pinned-host inputs copied every step, loss and norm read back"},
        "arm": arm,
        "result": result,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
    }
    print(json.dumps(line), flush=True)


def stream_tokens(args, world: int) -> int:
    """Length of the synthetic stream: one window per update of either region plus warm-up."""
    update_tokens = args.micro_batch * args.seq_len * args.grad_accum * world
    return update_tokens * (args.warmup + 2 * args.steps) + 1


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
    cfg.gradient_checkpointing = bool(args.activation_checkpointing)
    torch.manual_seed(1337)
    with torch.device(device):
        model = WarpStateLM(cfg)
    model.train()
    if args.bf16_residuals:
        model.bf16_residuals = True
    sync = None
    if world > 1:
        from warpstate_ai_b200.parallel.grad_sync import make_grad_sync
        sync = make_grad_sync(device, world, rank, None, kind=args.grad_sync)
    trainer = Trainer(model, device=device, rank=rank, world_size=world, lr=1.5e-4, weight_decay=0.1,
                      grad_sync=sync, shard_optimizer=args.shard_optimizer,
                      shard_params=None if args.shard_params == "off" else args.shard_params)
    mb, T, acc = args.micro_batch, args.seq_len, args.grad_accum
    update_tokens = mb * T * acc * world
    data = SyntheticTokens(stream_tokens(args, world), cfg.vocab_size, seed=7)
    batcher = HostBatcher(mb, T, device)
    lr = 1.5e-4

    cursor = 0
    for _ in range(args.warmup):
        trainer.pretrain_update(data, cursor, update_tokens, mb, T, lr, batcher)
        cursor += update_tokens

    # ---- device-resident inputs for the kernel-timed region: a different window for every step
    resident = []
    for step in range(args.steps):
        micro = []
        for offset, valid in update_slices(update_tokens, mb * T, world, rank):
            x, y = host_batch(data, cursor + offset, mb, T, valid)
            micro.append((x.to(device), y.to(device), valid))
        resident.append(micro)
        cursor += update_tokens

    def resident_update(micro):
        trainer.begin_update()
        for index, (x, y, valid) in enumerate(micro):
            def loss_fn(x=x, y=y, valid=valid):
                _, loss = model(x, y, return_logits=False)
                return loss, valid * world / update_tokens, valid / update_tokens
            trainer.micro_step(loss_fn, last=index == len(micro) - 1)
        return trainer.finish_update(lr)

    # ---- region 1: device-timed
    barrier_sync(world)
    sampler = ClockSampler()
    if rank == 0:
        sampler.start()
    launches0 = _ext.launch_count()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for micro in resident:
        stats = resident_update(micro)
    stop.record()
    barrier_sync(world)
    launches = _ext.launch_count() - launches0
    dev_s = max_over_ranks(start.elapsed_time(stop) / 1e3, world, device)
    trainer.read_update_scalars(stats)  # raises if the device reported a communication error
    # ---- region 2: end to end through the public API
    barrier_sync(world)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        result = trainer.pretrain_update(data, cursor, update_tokens, mb, T, lr, batcher)
        cursor += update_tokens
    barrier_sync(world)
    e2e_s = max_over_ranks(time.perf_counter() - t0, world, device)
    clocks = sampler.stop(gpu_indices=None) if rank == 0 else {}
    from warpstate_ai_b200.ops.gemm import check_device_errors
    check_device_errors()
    tokens = update_tokens * args.steps
    h2d = batcher.bytes_per_batch * acc * world
    sharded = args.shard_params != "off"
    arm = {"grad_sync": getattr(trainer.sync, "kind", "none"),
           "optimizer": "sharded" if ((args.shard_optimizer or sharded) and world > 1) else "replicated",
           "params": f"sharded-{args.shard_params}" if sharded else "replicated",
           "activation_checkpointing": bool(args.activation_checkpointing),
           "bf16_residuals": bool(args.bf16_residuals)}
    emit(args, rank, world, tokens / dev_s, dev_s / args.steps * 1e3, tokens / e2e_s, clocks, launches, "ours", arm,
         {"last_loss": result.loss, "last_grad_norm": result.grad_norm,
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
    data = rng.integers(0, cfg.vocab_size, size=stream_tokens(args, world), dtype=np.uint16)
    slices = list(ref_run.update_slices(update_tokens, mb * T, world, rank))

    def update(micro):
        """``micro``: per accumulation step a callable returning the (x, y) pair on the device, and its
        number of valid tokens."""
        optimizer.zero_grad(set_to_none=True)
        loss_sum = torch.zeros((), device=device)
        for index, (fetch, valid) in enumerate(micro):
            x, y = fetch()
            sync = model.no_sync() if world > 1 and index < len(micro) - 1 else contextlib.nullcontext()
            with sync:
                with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=True):
                    _, loss = model(x, y, return_logits=False)
                backward(scale_loss(loss, valid * world / update_tokens, "eager"))
            loss_sum += loss.detach() * (valid / update_tokens)
        norm = torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0, error_if_nonfinite=True)
        optimizer.step()
        if world > 1:
            dist.all_reduce(loss_sum, op=dist.ReduceOp.SUM)
        return loss_sum, norm

    def from_host(seen):
        """The reference's own loader: pinned host window -> device, inside the step."""
        return [((lambda o=offset, v=valid: ref_run.batches(data, seen + o, mb, T, v, device)), valid)
                for offset, valid in slices]

    seen = 0
    for _ in range(args.warmup):
        update(from_host(seen))
        seen += update_tokens
    # device-resident micro-batches for the device-timed region, produced by the reference's loader
    resident = []
    for _ in range(args.steps):
        micro = []
        for offset, valid in slices:
            pair = ref_run.batches(data, seen + offset, mb, T, valid, device)
            micro.append(((lambda p=pair: p), valid))
        resident.append(micro)
        seen += update_tokens
    barrier_sync(world)
    sampler = ClockSampler()
    if rank == 0:
        sampler.start()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for micro in resident:
        update(micro)
    stop.record()
    barrier_sync(world)
    dev_s = max_over_ranks(start.elapsed_time(stop) / 1e3, world, device)
    barrier_sync(world)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        loss_t, norm_t = update(from_host(seen))
        loss, norm = float(loss_t), float(norm_t)  # the reference reads both every update (run_40b.py:757-764)
        seen += update_tokens
    barrier_sync(world)
    wall = max_over_ranks(time.perf_counter() - t0, world, device)
    clocks = sampler.stop() if rank == 0 else {}
    tokens = update_tokens * args.steps
    emit(args, rank, world, tokens / dev_s, dev_s / args.steps * 1e3, tokens / wall, clocks, 0, "reference",
         {"compile_mode": args.ref_compile_mode, "loss_mode": "compiled-full", "ddp_bucket_cap_mb": 128,
          "optimizer": "torch.optim.AdamW(fused=True)"},
         {"last_loss": loss, "last_grad_norm": norm,
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
