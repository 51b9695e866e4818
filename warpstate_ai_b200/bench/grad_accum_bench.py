"""Weight-gradient GEMM + FP32 accumulation: the reference's three steps against the fused forms.

What a training step needs per weight is ``grad_fp32 += dy^T x``.  The reference evaluates
three ways of doing it (ops/benchmark_gradient_accumulation.py): a BF16 dW GEMM followed by
autograd's cast and FP32 add (baseline), a fused cast-add, and a direct FP32 ``addmm``.  This
benchmark times those with cuBLAS and compares them with this library's forms on the four
projection families:

* ``fused``    one tcgen05 GEMM whose epilogue does the FP32 read-modify-write (no BF16 rounding
               of the product, no extra pass over the gradient);
* ``grouped``  all four families in ONE persistent launch (shared waves).

    python -m warpstate_ai_b200.bench.grad_accum_bench --tokens 16384

One JSON line per variant with milliseconds for the four weights of a layer, the achieved
TFLOP/s and the error against the FP32 product.
"""
from __future__ import annotations

import argparse
import json

import torch

from .gemm_bench import FAMILIES, time_fn


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    from ..ops import gemm as G
    device = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    torch.manual_seed(0)
    problems = []
    for name, (k, n) in FAMILIES.items():
        dy = torch.randn(a.tokens, n, device=device).bfloat16()
        x = torch.randn(a.tokens, k, device=device).bfloat16()
        problems.append((name, dy, x, torch.zeros(n, k, device=device)))
    flops = sum(2 * a.tokens * dy.shape[1] * x.shape[1] for _, dy, x, _ in problems)

    def baseline():
        for _, dy, x, grad in problems:
            grad.add_((dy.T @ x).to(torch.float32))       # BF16 GEMM, cast, FP32 add

    def addmm_fp32():
        for _, dy, x, grad in problems:
            grad.addmm_(dy.T.float(), x.float())           # direct FP32 accumulate (TF32/FP32 GEMM)

    def fused():
        for _, dy, x, grad in problems:
            G.grad_weight_accumulate(dy, x, grad, accumulate=True)

    def grouped():
        G.grad_weight_accumulate_group([(dy, x, grad, True) for _, dy, x, grad in problems])

    variants = {"cublas_bf16_cast_add": baseline, "fused_epilogue": fused, "grouped_launch": grouped}
    if a.tokens <= 4096:
        variants["cublas_fp32_addmm"] = addmm_fp32  # needs FP32 copies of the operands
    for label, fn in variants.items():
        for _, _, _, grad in problems:
            grad.zero_()
        fn()
        torch.cuda.synchronize()
        worst = 0.0
        for _, dy, x, grad in problems:
            ref = dy.float().T @ x.float()
            worst = max(worst, float((grad - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()))
        ms = time_fn(fn, a.iters, flush)
        print(json.dumps({"variant": label, "tokens": a.tokens, "ms_per_layer": round(ms, 4),
                          "tflops": round(flops / ms / 1e9, 1), "relative_rms_error": worst}), flush=True)
    G.check_device_errors()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
