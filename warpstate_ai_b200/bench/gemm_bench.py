"""Isolated timing of the tcgen05 GEMM on the production shapes of the 2.005 B model.

Covers the same four projection families and three directions (forward, dX, dW) as the
reference's ops/benchmark_gemm.py:26-50, with CUDA-event timing, warm-up and an L2 flush
between iterations; prints one JSON line per case with the achieved TFLOP/s next to
torch.matmul (cuBLAS) on the same operands.

    python -m warpstate_ai_b200.bench.gemm_bench --tokens 16384
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import gemm as G

FAMILIES = {"in_proj": (2048, 10240), "out_proj": (2048, 2048), "up_gate": (2048, 14336), "down": (7168, 2048)}


def time_fn(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(stop)
    return total / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", type=str, default=None)
    args = ap.parse_args()
    m = args.tokens
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    rows = []
    for name, (k, n) in FAMILIES.items():
        x = torch.randn(m, k, device="cuda").bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
        dy = torch.randn(m, n, device="cuda").bfloat16()
        grad = torch.zeros(n, k, device="cuda")
        flops = 2.0 * m * n * k
        cases = {
            "fwd": (lambda: G.linear(x, w), lambda: torch.matmul(x, w.T)),
            "dx": (lambda: G.grad_input(dy, w), lambda: torch.matmul(dy, w)),
            "dw": (lambda: G.grad_weight_accumulate(dy, x, grad), lambda: torch.matmul(dy.T, x)),
        }
        for direction, (ours, lib) in cases.items():
            t_ours = time_fn(ours, args.iters, flush)
            t_lib = time_fn(lib, args.iters, flush)
            row = {"family": name, "direction": direction, "m": m, "n": n, "k": k,
                   "ms": round(t_ours, 4), "tflops": round(flops / t_ours / 1e9, 1),
                   "cublas_ms": round(t_lib, 4), "cublas_tflops": round(flops / t_lib / 1e9, 1)}
            rows.append(row)
            print(json.dumps(row), flush=True)
    G.check_device_errors()
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
