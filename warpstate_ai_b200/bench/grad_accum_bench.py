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
import statistics
from pathlib import Path

from .gemm_bench import ALIASES, FAMILIES, add_library_arm_flags, apply_library_arm_flags, burn_in, time_fn

VARIANTS = ("cublas_bf16_cast_add", "cublas_fp32_addmm", "fused_epilogue", "grouped_launch")


def arguments(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--families", nargs="+", choices=[*FAMILIES, *ALIASES], default=list(FAMILIES))
    ap.add_argument("--variants", nargs="+", choices=VARIANTS,
                    help="default: all; the direct FP32 addmm only up to 4096 rows (it needs FP32 copies of the operands)")
    ap.add_argument("--rows", "--tokens", dest="rows", type=int, default=16384, help="micro-batch times sequence length")
    ap.add_argument("--accumulation-steps", type=int, default=1,
                    help="micro-batches accumulated into the same FP32 gradient per timed launch group")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", "--iters", dest="repeats", type=int, default=10)
    ap.add_argument("--trials", type=int, default=1, help="the median over this many trials is reported")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--output-dir", type=Path, help="write results.json here")
    ap.add_argument("--list-shapes", action="store_true", help="print the dW problems and exit (no GPU needed)")
    ap.add_argument("--burnin-seconds", type=float, default=0.0, help="keep the GPU busy this long before the first variant")
    add_library_arm_flags(ap)
    a = ap.parse_args(argv)
    if min(a.rows, a.accumulation_steps, a.repeats, a.trials) < 1 or a.warmup < 0 or a.burnin_seconds < 0:
        ap.error("rows, accumulation steps, repeats and trials must be positive; warmup must not be negative")
    a.families = list(dict.fromkeys(ALIASES.get(f, f) for f in a.families))
    if a.variants is None:
        a.variants = [v for v in VARIANTS if v != "cublas_fp32_addmm" or a.rows <= 4096]
    return a


def problems_of(families, rows: int) -> list[dict]:
    """The weight-gradient product of each family: ``grad[n, k] += dy[rows, n]^T x[rows, k]``."""
    return [{"family": f, "rows": rows, "n": FAMILIES[f][1], "k": FAMILIES[f][0], "flops": 2 * rows * FAMILIES[f][0] * FAMILIES[f][1]}
            for f in families]


def main(argv=None) -> int:
    a = arguments(argv)
    shapes = problems_of(a.families, a.rows)
    if a.list_shapes:
        print(json.dumps(shapes, indent=1))
        return 0
    import torch
    from ..ops import gemm as G
    device = torch.device("cuda", a.device)
    torch.cuda.set_device(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    torch.manual_seed(a.seed)
    library_arm = apply_library_arm_flags(a)
    burn_in(a.burnin_seconds)
    problems = []
    for shape in shapes:
        dy = torch.randn(a.rows, shape["n"], device=device).bfloat16()
        x = torch.randn(a.rows, shape["k"], device=device).bfloat16()
        problems.append((shape["family"], dy, x, torch.zeros(shape["n"], shape["k"], device=device)))
    steps = a.accumulation_steps
    flops = steps * sum(shape["flops"] for shape in shapes)

    def baseline():
        for _ in range(steps):
            for _, dy, x, grad in problems:
                grad.add_((dy.T @ x).to(torch.float32))       # BF16 GEMM, cast, FP32 add

    def addmm_fp32():
        for _ in range(steps):
            for _, dy, x, grad in problems:
                grad.addmm_(dy.T.float(), x.float())           # direct FP32 accumulate (TF32/FP32 GEMM)

    def fused():
        for _ in range(steps):
            for _, dy, x, grad in problems:
                G.grad_weight_accumulate(dy, x, grad, accumulate=True)

    def grouped():
        for _ in range(steps):
            G.grad_weight_accumulate_group([(dy, x, grad, True) for _, dy, x, grad in problems])

    launch = {"cublas_bf16_cast_add": baseline, "cublas_fp32_addmm": addmm_fp32, "fused_epilogue": fused, "grouped_launch": grouped}
    rows = []
    for label in a.variants:
        fn = launch[label]
        for _, _, _, grad in problems:
            grad.zero_()
        fn()
        torch.cuda.synchronize()
        worst = 0.0
        for _, dy, x, grad in problems:
            ref = steps * (dy.float().T @ x.float())
            worst = max(worst, float((grad - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()))
        ms = statistics.median(time_fn(fn, a.repeats, flush, a.warmup) for _ in range(a.trials))
        rows.append({"variant": label, "tokens": a.rows, "accumulation_steps": steps, "families": a.families,
                     "ms_per_layer": round(ms / steps, 4), "tflops": round(flops / ms / 1e9, 1), "relative_rms_error": worst})
        print(json.dumps(rows[-1]), flush=True)
    G.check_device_errors()
    if a.output_dir is not None:
        a.output_dir.mkdir(parents=True, exist_ok=True)
        (a.output_dir / "results.json").write_text(json.dumps({
            "rows": rows, "problems": shapes, "library_arm": library_arm, "gpu": torch.cuda.get_device_name(device), "torch": torch.__version__}, indent=1) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
