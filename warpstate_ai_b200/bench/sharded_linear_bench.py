"""Fused all-gather + cast + GEMM against its unfused formulation (row-sharded FP32 weight).

Runs on N ranks of one node (``torchrun --nproc-per-node N -m warpstate_ai_b200.bench.sharded_linear_bench``)
or on one GPU (shards emulated on the device: no link traffic, the cast and flag protocol only).
Three arms on the in_proj shape of the 2.005 B model (16384 x 10240 x 2048 by default):

* ``fused``     one launch: gather (peer loads) + FP32->BF16 cast + tcgen05 GEMM (`ShardedWeight.forward`)
* ``unfused``   NCCL all_gather_into_tensor of the FP32 shards, cast kernel, GEMM kernel (three launches)
* ``gemm_only`` the GEMM on an already gathered BF16 weight (the floor: no gather at all)

Times are CUDA-event times on the launching stream, max over ranks, median of the iterations, with
an L2 flush between iterations.  The roofline target of the fused arm is the slower of
(FLOPs / measured BF16 GEMM peak) and (remote FP32 bytes / 770 GB/s per direction).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    # long names: under torchrun a bare --n is read as an abbreviation of torchrun's own options
    ap.add_argument("--m", "--tokens", dest="m", type=int, default=16384)
    ap.add_argument("--n", "--out-features", dest="n", type=int, default=10240)
    ap.add_argument("--k", "--in-features", dest="k", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--emulate-world", type=int, default=4, help="shards on one device when run without torchrun")
    ap.add_argument("--swiglu", action="store_true",
                    help="up/gate weight [2n, k] with the SwiGLU epilogue (n = hidden width; try --out-features 7168)")
    args = ap.parse_args()
    from ..ops import _ext, gemm as G
    from ..parallel.sharded_linear import ShardedWeight, rows_per_shard

    distributed = "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1
    rank = int(os.environ.get("LOCAL_RANK", "0")) if distributed else 0
    world = int(os.environ["WORLD_SIZE"]) if distributed else 1
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    if distributed:
        dist.init_process_group("nccl", device_id=device)
    _ext.require()
    torch.manual_seed(0)
    w_rows = 2 * args.n if args.swiglu else args.n
    w = torch.randn(w_rows, args.k, device=device) * 0.02
    torch.manual_seed(1 + rank)
    x = torch.randn(args.m, args.k, device=device).bfloat16()
    if distributed:
        sw = ShardedWeight.from_full(w, rank, world, swiglu=args.swiglu)
        shards = world
    else:
        sw = ShardedWeight.emulated(w, args.emulate_world, swiglu=args.swiglu)
        shards = args.emulate_world
    per = rows_per_shard(w_rows, shards)
    linear = G.linear_swiglu if args.swiglu else G.linear
    gathered32 = torch.empty(per * shards, args.k, device=device)
    wb = w.bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def unfused():
        if distributed:
            dist.all_gather_into_tensor(gathered32.view(-1), sw.shard.view(-1)[:per * args.k])
            src = gathered32[:w_rows]
        else:
            src = w
        return linear(x, torch.ops.ws_b200.cast_bf16(src, None))

    arms = {"fused": lambda: sw.forward(x), "unfused": unfused, "gemm_only": lambda: linear(x, wb)}
    result = {}
    for name, fn in arms.items():
        times = []
        for it in range(args.warmup + args.iters):
            flush.fill_(it & 0xFF)
            if distributed:
                dist.barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                times.append(start.elapsed_time(end))
        t = torch.tensor([statistics.median(times)], device=device)
        if distributed:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        result[name] = float(t.item())
    G.check_device_errors()
    if rank == 0:
        flops = 2.0 * args.m * w_rows * args.k
        remote_bytes = 4.0 * w_rows * args.k * (world - 1) / world
        peaks = {}
        try:
            with open(os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except OSError:
            pass
        peak_tflops = float(peaks.get("bf16_tflops", 1590.0))
        target_ms = max(flops / (peak_tflops * 1e12), remote_bytes / 770e9) * 1e3
        print(json.dumps({"shape": [args.m, w_rows, args.k], "swiglu": args.swiglu, "ranks": world, "shards": shards, "ms": result,
                          "fused_tflops": flops / result["fused"] / 1e9, "remote_fp32_mb": remote_bytes / 1e6,
                          "roofline_target_ms": target_ms, "fused_fraction_of_roofline": target_ms / result["fused"],
                          "peak_tflops_used": peak_tflops, "timing": "cuda events, median, max over ranks, L2 flushed"}),
              flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
