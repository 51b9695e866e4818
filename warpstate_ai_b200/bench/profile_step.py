"""Kernel-level profile of one optimizer update (torch.profiler, CUDA activities).

Equivalent of the reference's ``ops/benchmark_training.py --profile`` (kernel table + name-based
categories, ops/benchmark_training.py:199-255): prints per-kernel total device time and the
share of each category for one measured update after warm-up.  Numbers taken under the profiler
are for *shares* only; throughput is measured by bench.py.

    python -m warpstate_ai_b200.bench.profile_step --model 2b --micro-batch 8 --grad-accum 1
"""
from __future__ import annotations

import argparse
import os
import json
from collections import defaultdict

import torch

CATEGORIES = [
    ("gemm", ("gemm_kernel", "gemm2_kernel")),
    ("attention", ("attn_fwd_kernel", "attn_bwd_kernel", "chunk_writes_kernel", "dstate_kernel", "memory_scan")),
    ("lm_head", ("lmhead", "ce_")),
    ("norm", ("rmsnorm", "colsum")),
    ("communication", ("nccl", "grad_reduce", "bucket_ready", "norm_exchange", "node_barrier", "gather_cast", "adamw_shard_push")),
    ("optimizer", ("adamw_kernel", "sumsq_kernel", "clip_coef")),
    ("embedding", ("embed_",)),
    ("cast", ("cast_f32_bf16",)),
    ("communication", ("nccl", "grad_reduce", "bucket_ready", "norm_exchange", "node_barrier", "gather_cast", "adamw_shard_push",
                       "allreduce", "allgather", "all_gather")),
    ("copies", ("Memcpy", "memcpy", "Memset", "memset")),
]


def category(name: str) -> str:
    for cat, keys in CATEGORIES:
        if any(k in name for k in keys):
            return cat
    return "other (library / eager PyTorch)"


def idle_gaps(intervals: list[tuple[float, float, str]], top: int = 12) -> dict:
    """``intervals``: (start_us, end_us, kernel name) of every device activity of one update.

    Returns the span from the first start to the last end, the time in which at least one kernel
    ran (union of the intervals, so kernels overlapping on two streams count once), the idle rest,
    and the ``top`` longest idle gaps with the kernels on either side (the place to look for host
    synchronisations and launch-bound stretches).  The interval-union arithmetic is that of the
    reference's trace analysis (ops/analyze_communication_profile.py:38-80).
    """
    if not intervals:
        return {"span_ms": 0.0, "busy_ms": 0.0, "idle_ms": 0.0, "gaps": []}
    ordered = sorted(intervals)
    span0, frontier, frontier_name = ordered[0][0], ordered[0][1], ordered[0][2]
    busy = 0.0
    run_start = ordered[0][0]
    gaps = []
    for start, end, name in ordered[1:]:
        if start > frontier:
            busy += frontier - run_start
            gaps.append((start - frontier, frontier_name, name, frontier - span0))
            run_start = start
        if end > frontier:
            frontier, frontier_name = end, name
    busy += frontier - run_start
    span = frontier - span0
    gaps.sort(key=lambda g: -g[0])
    return {"span_ms": span / 1e3, "busy_ms": busy / 1e3, "idle_ms": (span - busy) / 1e3, "n_gaps": len(gaps),
            "gaps": [{"idle_us": g[0], "after": g[1][:80], "before": g[2][:80], "at_ms": g[3] / 1e3} for g in gaps[:top]]}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="2b", choices=["2b", "smoke"])
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--grad-accum", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--top", type=int, default=40)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    # A programmatic dependent launch starts before its predecessor ends and waits inside the kernel, so a
    # profiler would book that wait as the kernel's own time: profile with plain launches (read once, at the
    # library's first launch).
    os.environ.setdefault("WS_TRAIN_PDL", "0")
    from .. import WarpStateLM, warpstate_2b, warpstate_smoke
    from ..data.tokens import SyntheticTokens
    from ..train.engine import Trainer

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    cfg = warpstate_2b() if args.model == "2b" else warpstate_smoke()
    cfg.gradient_checkpointing = False
    torch.manual_seed(0)
    with torch.device(device):
        model = WarpStateLM(cfg)
    trainer = Trainer(model, device=device)
    tokens = args.micro_batch * args.seq_len * args.grad_accum
    data = SyntheticTokens(tokens * 2 + 1, cfg.vocab_size)
    for _ in range(2):
        trainer.pretrain_update(data, 0, tokens, args.micro_batch, args.seq_len, 1e-4)
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA,
                                            torch.profiler.ProfilerActivity.CPU]) as prof:
        trainer.pretrain_update(data, 0, tokens, args.micro_batch, args.seq_len, 1e-4)
        torch.cuda.synchronize()
    per_kernel = defaultdict(lambda: [0.0, 0])
    intervals = []
    for event in prof.events():
        if event.device_type == torch.autograd.DeviceType.CUDA:
            per_kernel[event.name][0] += event.device_time
            per_kernel[event.name][1] += 1
            intervals.append((float(event.time_range.start), float(event.time_range.end), event.name))
    gaps = idle_gaps(intervals)
    total = sum(v[0] for v in per_kernel.values())
    cats = defaultdict(float)
    for name, (us, _count) in per_kernel.items():
        cats[category(name)] += us
    rows = sorted(per_kernel.items(), key=lambda kv: -kv[1][0])
    print(f"total device time {total / 1e3:.2f} ms over {sum(v[1] for v in per_kernel.values())} kernels")
    for cat, us in sorted(cats.items(), key=lambda kv: -kv[1]):
        print(f"  {cat:36s} {us / 1e3:9.2f} ms  {100 * us / total:5.1f} %")
    print("top kernels:")
    for name, (us, count) in rows[:args.top]:
        print(f"  {us / 1e3:9.3f} ms  x{count:5d}  {name[:110]}")
    print(f"device span {gaps['span_ms']:.2f} ms: busy {gaps['busy_ms']:.2f} ms, idle {gaps['idle_ms']:.2f} ms "
          f"in {gaps['n_gaps']} gaps; longest:")
    for g in gaps["gaps"]:
        print(f"  {g['idle_us']:8.1f} us at {g['at_ms']:8.2f} ms  after {g['after'][:48]:48s} before {g['before'][:48]}")
    if args.out:
        with open(args.out, "w") as f:
            json.dump({"total_ms": total / 1e3, "idle": gaps, "categories": {k: v / 1e3 for k, v in cats.items()},
                       "kernels": [{"name": n, "ms": v[0] / 1e3, "count": v[1]} for n, v in rows]}, f, indent=1)


if __name__ == "__main__":
    main()
