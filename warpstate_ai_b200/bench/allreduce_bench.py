"""In-kernel gradient all-reduce (`bucket_ready_kernel` + `grad_reduce_kernel`, ops/csrc/comm.cu) against NCCL all_reduce.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29561 \
        -m warpstate_ai_b200.bench.allreduce_bench [--mib 128 1024] [--ctas 16 32 64]

For every buffer size: the fused kernel (reduce over peer memory or inside NVSwitch with `multimem`, scale by
1/world, broadcast, sum of squares of the result in the same pass) with each CTA count, through plain peer
loads and -- when the fabric offers a multicast address -- through NVLS, and `dist.all_reduce` + a separate
scale on the same bytes.  Times are CUDA events on the launching stream, median of the iterations, max over
ranks.  Reported: algorithmic bandwidth bytes / t and bus bandwidth 2 (N-1)/N bytes / t, the figure that
compares with the node's measured NCCL all-reduce bus bandwidth (725 GB/s at 1 GiB on 8 ranks) and with the
770 GB/s per direction of a peer copy.

The reference reduces its gradients with DDP's NCCL all-reduce on FP32 buckets of 128 MiB
(ops/distributed_execution.py:16-79); the 128 MiB default here is that bucket.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist


def timed(fn, iters: int, warmup: int, device) -> float:
    times = []
    for it in range(warmup + iters):
        dist.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(start.elapsed_time(end))
    t = torch.tensor([statistics.median(times)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, nargs="+", default=[128, 1024])
    ap.add_argument("--ctas", type=int, nargs="+", default=[16, 32, 64])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    from ..ops import _ext
    from ..parallel import symm

    rank, world = int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=device)
    _ext.require()
    # The kernel's completion counters advance by (CTAs per launch) every call, so one flag bucket serves one
    # CTA count: every (size, path, CTA count) arm below gets a bucket of its own with its own sequence number.
    max_arms = 2 * len(args.mib) * len(args.ctas)
    flags = symm.allocate(2 * 8 * max_arms, torch.int32, device)
    status = torch.zeros(8, dtype=torch.int32, device=device)
    sumsq = torch.zeros(64, dtype=torch.float32, device=device)   # one partial per CTA
    rows = []
    arm = 0
    for mib in args.mib:
        n = mib * (1 << 20) // 4
        buf = symm.allocate(n, torch.float32, device)
        buf.tensor.normal_()
        plain = torch.randn(n, device=device)
        bytes_ = 4.0 * n

        def record(name, ms, ctas=None):
            rows.append({"mib": mib, "arm": name, "ctas": ctas, "ms": ms, "alg_gbs": bytes_ / ms / 1e6,
                         "bus_gbs": 2.0 * (world - 1) / world * bytes_ / ms / 1e6})

        def nccl():
            dist.all_reduce(plain)
            plain.mul_(1.0 / world)

        record("nccl all_reduce + scale", timed(nccl, args.iters, args.warmup, device))
        for use_nvls in (False, True):
            mc = buf.multicast_ptr if use_nvls else 0
            if use_nvls and not mc:
                continue
            for ctas in args.ctas:
                bucket, counter = arm, [0]
                arm += 1

                def fused():
                    counter[0] += 1
                    torch.ops.ws_b200.grad_allreduce(buf.peer_ptrs, flags.peer_ptrs, mc, rank, world, 0, n, bucket,
                                                     counter[0], 1.0 / world, True, ctas, sumsq, status, 2.0)

                ms = timed(fused, args.iters, args.warmup, device)
                if int(status[0]) != 0:
                    raise RuntimeError(f"grad_allreduce reported {status.tolist()}")
                record("fused multimem (NVLS)" if use_nvls else "fused peer loads", ms, ctas)
        del buf
    if rank == 0:
        print(json.dumps({"ranks": world, "rows": rows,
                          "timing": "cuda events, median, max over ranks; buffers far larger than L2"}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
