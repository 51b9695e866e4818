"""Isolated timing of the tcgen05 GEMM on the production shapes of the 2.005 B model.

The four projection families and three operations (forward ``Y = X W^T``, ``dX = dY W``, ``dW = dY^T X``) of the
reference's ops/benchmark_gemm.py:26-117, timed with CUDA events after warm-up, an optional burn-in and an L2 flush
before every timed launch; one JSON line per case with the achieved TFLOP/s, next to ``torch.matmul`` (cuBLAS) on the
same operands when that arm is selected.

    python -m warpstate_ai_b200.bench.gemm_bench --rows 16384
    python -m warpstate_ai_b200.bench.gemm_bench --list-shapes          # the cases, no GPU needed
"""
from __future__ import annotations

import argparse
import json
import statistics
import time
from pathlib import Path

FAMILIES = {"in_proj": (2048, 10240), "out_proj": (2048, 2048), "up_gate": (2048, 14336), "down": (7168, 2048)}
ALIASES = {"ffn_up_gate": "up_gate", "ffn_down": "down"}                 # the reference's names for the two FFN families
OPERATIONS = ("fwd", "dx", "dw")
ARMS = ("ours", "cublas")


def projection_cases(families, rows: int, operations) -> list[dict]:
    """``[{name, family, operation, m, n, k, a_shape, b_shape, flops}]``: the GEMM each operation of a projection with
    ``rows`` tokens is, written as ``[m, k] x [k, n]``."""
    cases = []
    for family in families:
        family = ALIASES.get(family, family)
        features_in, features_out = FAMILIES[family]
        shapes = {"fwd": (rows, features_out, features_in), "dx": (rows, features_in, features_out),
                  "dw": (features_out, features_in, rows)}
        for operation in operations:
            m, n, k = shapes[operation]
            cases.append({"name": f"{family}.{operation}", "family": family, "operation": operation, "m": m, "n": n, "k": k,
                          "a_shape": [m, k], "b_shape": [k, n], "flops": 2 * m * n * k})
    return cases


def time_fn(fn, iters: int, flush, warmup: int = 3) -> float:
    """Mean milliseconds of ``fn`` over ``iters`` launches, each after ``flush`` (larger than L2) has been rewritten."""
    import torch
    for _ in range(warmup):
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


def add_library_arm_flags(ap) -> None:
    """How the cuBLAS arm is run (the arm this library's kernel is compared with; the kernel itself has neither choice)."""
    ap.add_argument("--blas-backend", choices=["default", "cublas", "cublaslt"], default="default",
                    help="PyTorch's BLAS preference for the cuBLAS arm; default keeps the process's own")
    ap.add_argument("--allow-reduced-precision-reduction", action=argparse.BooleanOptionalAction, default=True,
                    help="let the cuBLAS arm reduce in BF16 between split-K partial sums, as PyTorch does by default")


def apply_library_arm_flags(a) -> dict:
    """Apply the two cuBLAS-arm settings to this process; -> what is now in force (for the record)."""
    import torch
    if a.blas_backend != "default":
        torch.backends.cuda.preferred_blas_library(a.blas_backend)
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = bool(a.allow_reduced_precision_reduction)
    return {"blas_backend": a.blas_backend, "allow_bf16_reduced_precision_reduction": bool(a.allow_reduced_precision_reduction)}


def burn_in(seconds: float) -> None:
    """Keep the GPU busy for ``seconds`` so that the first case is not timed on cold clocks."""
    import torch
    if seconds <= 0:
        return
    a = torch.randn(8192, 8192, device="cuda").bfloat16()
    until = time.monotonic() + seconds
    while time.monotonic() < until:
        for _ in range(20):
            torch.matmul(a, a)
        torch.cuda.synchronize()


def arguments(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--families", nargs="+", choices=[*FAMILIES, *ALIASES], default=list(FAMILIES))
    ap.add_argument("--operations", nargs="+", choices=OPERATIONS, default=list(OPERATIONS))
    ap.add_argument("--rows", "--tokens", dest="rows", type=int, default=16384,
                    help="micro-batch times sequence length (the headline configuration: 8 x 2048)")
    ap.add_argument("--backends", nargs="+", choices=ARMS, default=list(ARMS), help="this library's kernel and/or cuBLAS")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", "--iters", dest="repeats", type=int, default=10, help="timed launches per trial")
    ap.add_argument("--trials", type=int, default=1, help="the median over this many trials is reported")
    ap.add_argument("--burnin-seconds", type=float, default=0.0, help="keep the GPU busy this long before the first case")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", type=int, default=0, help="CUDA device index")
    ap.add_argument("--output-dir", type=Path, help="write cases.json and results.json here")
    ap.add_argument("--out", type=str, default=None, help="write the result rows to this file")
    ap.add_argument("--list-shapes", action="store_true", help="print the cases and exit (no GPU needed)")
    add_library_arm_flags(ap)
    a = ap.parse_args(argv)
    if a.rows < 1 or a.warmup < 0 or a.repeats < 1 or a.trials < 1 or a.burnin_seconds < 0:
        ap.error("rows, repeats and trials must be positive; warmup and burn-in must not be negative")
    return a


def main(argv=None) -> int:
    args = arguments(argv)
    cases = projection_cases(args.families, args.rows, args.operations)
    if args.list_shapes:
        print(json.dumps(cases, indent=1))
        return 0
    import torch
    from ..ops import gemm as G
    torch.cuda.set_device(args.device)
    torch.manual_seed(args.seed)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    library_arm = apply_library_arm_flags(args)
    burn_in(args.burnin_seconds)
    rows = []
    m = args.rows
    for family in dict.fromkeys(ALIASES.get(f, f) for f in args.families):
        k, n = FAMILIES[family]
        x = torch.randn(m, k, device="cuda").bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
        dy = torch.randn(m, n, device="cuda").bfloat16()
        grad = torch.zeros(n, k, device="cuda")
        launches = {
            "fwd": (lambda: G.linear(x, w), lambda: torch.matmul(x, w.T)),
            "dx": (lambda: G.grad_input(dy, w), lambda: torch.matmul(dy, w)),
            "dw": (lambda: G.grad_weight_accumulate(dy, x, grad), lambda: torch.matmul(dy.T, x)),
        }
        flops = 2.0 * m * n * k
        for operation in args.operations:
            ours, library = launches[operation]
            row = {"family": family, "direction": operation, "m": m, "n": n, "k": k, "trials": args.trials, "repeats": args.repeats}
            if "ours" in args.backends:
                t = statistics.median(time_fn(ours, args.repeats, flush, args.warmup) for _ in range(args.trials))
                row.update(ms=round(t, 4), tflops=round(flops / t / 1e9, 1))
            if "cublas" in args.backends:
                t = statistics.median(time_fn(library, args.repeats, flush, args.warmup) for _ in range(args.trials))
                row.update(cublas_ms=round(t, 4), cublas_tflops=round(flops / t / 1e9, 1))
            rows.append(row)
            print(json.dumps(row), flush=True)
    G.check_device_errors()
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    if args.output_dir is not None:
        args.output_dir.mkdir(parents=True, exist_ok=True)
        (args.output_dir / "cases.json").write_text(json.dumps(cases, indent=1) + "\n")
        (args.output_dir / "results.json").write_text(json.dumps({
            "rows": rows, "arguments": {k: (str(v) if isinstance(v, Path) else v) for k, v in vars(args).items()},
            "library_arm": library_arm, "gpu": torch.cuda.get_device_name(args.device), "torch": torch.__version__}, indent=1) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
