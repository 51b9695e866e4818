"""Bracketed screening of GEMM kernel variants against cuBLAS, producing a candidate policy.

For each production problem (the four projection families x forward / dX / dW at ``--rows``
tokens) every candidate -- the CTA-pair kernel, the single-CTA kernel, and either of them
restricted to fewer SMs (what a concurrent collective kernel leaves) -- is timed in
control / candidate / control triples with CUDA events after a burn-in, with an L2 flush before
every timed launch.  A candidate is eligible only if its result is within
``--maximum-relative-rms`` of the FP32 product and its WORST triple still beats the mean of its
two adjacent controls by ``--minimum-gain``.  The best eligible candidate per problem goes into
``candidate-policy.json`` (loadable with ``ops.gemm.load_policy``); ``report.json`` keeps every
trial.  Entries are isolated-kernel candidates: validate them in a full step before adopting.

    python -m warpstate_ai_b200.bench.tune_gemm --rows 16384 --output-dir tune-out

Method of the reference's ops/tune_matmul.py:143-157,251-313 (there: Triton tile sweeps against
ATen; here: this library's tcgen05 kernels against cuBLAS).
"""
from __future__ import annotations

import argparse
import json
import math
import statistics
import time
from pathlib import Path

import torch

FAMILIES = {"in_proj": (2048, 10240), "out_proj": (2048, 2048), "up_gate": (2048, 14336), "down": (7168, 2048)}
CANDIDATES = [{"kernel": "pair", "sm_limit": 0}, {"kernel": "single", "sm_limit": 0},
              {"kernel": "pair", "sm_limit": 116}, {"kernel": "single", "sm_limit": 116}]


def paired_timing_metrics(trials: list, minimum_gain: float) -> dict:
    """Compare each candidate timing with its two adjacent controls; keep the worst trial."""
    if not trials or any(not math.isfinite(v) or v <= 0 for t in trials for v in t.values()):
        raise ValueError("paired timings must be finite and positive")
    controls = [(t["control_before_ms"] + t["control_after_ms"]) / 2 for t in trials]
    gains = [c / t["candidate_ms"] - 1 for c, t in zip(controls, trials)]
    return {"median_ms": statistics.median(t["candidate_ms"] for t in trials),
            "median_control_ms": statistics.median(controls), "paired_gain": statistics.median(gains),
            "minimum_trial_gain": min(gains), "timing_eligible": min(gains) >= minimum_gain,
            "maximum_control_drift_fraction": max(abs(t["control_after_ms"] - t["control_before_ms"]) / c
                                                  for c, t in zip(controls, trials))}


def cases(rows: int, operations, kind: str = "mm") -> list:
    """The problems of one screening: every family and operation, or (``kind="swiglu"``) the forward up/gate projection
    with the SwiGLU epilogue, which no other family has."""
    if kind == "swiglu":
        k, n = FAMILIES["up_gate"]
        return [{"family": "up_gate", "operation": "fwd", "kind": "swiglu", "tokens": rows, "in_features": k, "out_features": n}]
    out = []
    for name, (k, n) in FAMILIES.items():
        for op in operations:
            out.append({"family": name, "operation": op, "tokens": rows, "in_features": k, "out_features": n})
    return out


def candidates_of(algorithms, tiles) -> list:
    """The candidates of a screening: the default sweep restricted to ``algorithms`` (kernels), or exactly the
    ``KERNEL,SMS`` pairs given with ``--tile`` (tile shapes are fixed when the kernels are built; what can be chosen at
    run time is the kernel and how many SMs it may occupy, 0 = all)."""
    if tiles:
        chosen = []
        for text in tiles:
            kernel, _, sms = text.partition(",")
            if kernel not in ("pair", "single") or not sms.strip().isdigit() or int(sms) > 148:
                raise ValueError(f"--tile {text!r}: expected KERNEL,SMS with KERNEL pair or single and SMS from 0 (all) to 148")
            chosen.append({"kernel": kernel, "sm_limit": int(sms)})
        return chosen
    return [c for c in CANDIDATES if algorithms is None or c["kernel"] in algorithms]


def policy_key(case: dict) -> str:
    if case.get("kind") == "swiglu":           # the launch `ops.gemm.linear_swiglu` makes: one output tile per (up, gate) pair
        return f"fwd:{case['tokens']}x{case['out_features'] // 2}x{case['in_features']}"
    return f"{case['operation']}:{case['tokens']}x{case['out_features']}x{case['in_features']}"


def select_policy(results: list) -> dict:
    """Best eligible candidate per problem (by paired gain)."""
    best = {}
    for row in results:
        if row.get("status") != "ok" or not row.get("eligible"):
            continue
        key = policy_key(row["case"])
        if key not in best or row["paired_gain"] > best[key]["paired_gain"]:
            best[key] = row
    return {"format": "warpstate-gemm-policy-v1",
            "entries": [{"key": k, **r["candidate"], "paired_gain": r["paired_gain"], "tflops": r["tflops"]}
                        for k, r in sorted(best.items())]}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--kind", choices=["mm", "swiglu"], default="mm",
                   help="plain projections, or the forward up/gate projection with the SwiGLU epilogue")
    p.add_argument("--operations", nargs="+", choices=["fwd", "dx", "dw"], default=["fwd", "dx", "dw"])
    p.add_argument("--algorithms", nargs="+", choices=["pair", "single"],
                   help="kernels of the default sweep (CTA pair, single CTA); both when omitted")
    p.add_argument("--tile", action="append", metavar="KERNEL,SMS",
                   help="repeat to screen exactly these candidates instead of the default sweep, e.g. pair,116")
    p.add_argument("--rows", type=int, default=16384)
    p.add_argument("--repeats", type=int, default=10)
    p.add_argument("--trials", type=int, default=3)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--burnin-seconds", type=float, default=1.0)
    p.add_argument("--minimum-gain", type=float, default=0.01)
    p.add_argument("--maximum-relative-rms", type=float, default=0.003)
    p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--input-scale", type=float, default=1.0, help="standard deviation of the random activations and gradients")
    p.add_argument("--device", type=int, default=0, help="CUDA device index")
    p.add_argument("--list-cases", action="store_true")
    p.add_argument("--output-dir", type=Path, required=True)
    a = p.parse_args(argv)
    selected = cases(a.rows, a.operations, a.kind)
    try:
        candidates = candidates_of(a.algorithms, a.tile)
    except ValueError as problem:
        p.error(str(problem))
    if a.list_cases:
        print(json.dumps(selected, indent=1))
        return 0
    from ..ops import _ext, gemm as G
    lib = _ext.cdll()
    device = torch.device("cuda", a.device)
    torch.cuda.set_device(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    a.output_dir.mkdir(parents=True, exist_ok=True)
    report = {"started": time.time(), "device": torch.cuda.get_device_name(device), "arguments": vars(a) | {"output_dir": str(a.output_dir)},
              "results": []}

    def save():
        (a.output_dir / "report.json").write_text(json.dumps(report, indent=1, default=str) + "\n")
        (a.output_dir / "candidate-policy.json").write_text(json.dumps(select_policy(report["results"]), indent=1) + "\n")

    def elapsed_ms(fn) -> float:
        total = 0.0
        for _ in range(a.repeats):
            flush.zero_()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            stop.record()
            torch.cuda.synchronize()
            total += start.elapsed_time(stop)
        return total / a.repeats

    def warm(fn):
        end = time.monotonic() + a.burnin_seconds
        for _ in range(a.warmup):
            fn()
        while time.monotonic() < end:
            fn()
        torch.cuda.synchronize()

    gen = torch.Generator(device=device).manual_seed(a.seed)
    for case in selected:
        t, k, n = case["tokens"], case["in_features"], case["out_features"]
        x = (torch.randn(t, k, device=device, generator=gen) * a.input_scale).bfloat16()
        w = (torch.randn(n, k, device=device, generator=gen) * 0.02).bfloat16()
        dy = (torch.randn(t, n, device=device, generator=gen) * a.input_scale).bfloat16()
        grad = torch.zeros(n, k, device=device)
        if case.get("kind") == "swiglu":
            def control():
                up, gate = (x @ w.T).chunk(2, dim=-1)
                return torch.nn.functional.silu(gate) * up
            ours, flops = (lambda: G.linear_swiglu(x, w)[1]), 2 * t * n * k
        elif case["operation"] == "fwd":
            control, ours, flops = (lambda: x @ w.T), (lambda: G.linear(x, w)), 2 * t * n * k
        elif case["operation"] == "dx":
            control, ours, flops = (lambda: dy @ w), (lambda: G.grad_input(dy, w)), 2 * t * n * k
        else:
            control = lambda: grad.add_((dy.T @ x).float())  # noqa: E731  (BF16 product, cast, FP32 add)
            ours, flops = (lambda: G.grad_weight_accumulate(dy, x, grad, accumulate=False)), 2 * t * n * k
        if case.get("kind") == "swiglu":
            up, gate = (x.float() @ w.float().T).bfloat16().float().chunk(2, dim=-1)
            reference = torch.nn.functional.silu(gate) * up
            del up, gate
        else:
            reference = (x.float() @ w.float().T if case["operation"] == "fwd" else dy.float() @ w.float()
                         if case["operation"] == "dx" else dy.float().T @ x.float())
        for candidate in candidates:
            row = {"case": case, "candidate": candidate, "status": "running"}
            lib.ws_gemm_set_pair_mode(1 if candidate["kernel"] == "pair" else 0)
            lib.ws_gemm_set_sm_limit(candidate["sm_limit"])
            try:
                out = ours()
                torch.cuda.synchronize()
                err = float((out.float() - reference).pow(2).mean().sqrt() / reference.pow(2).mean().sqrt())
                row["relative_rms_error"] = err
                warm(control)
                warm(ours)
                triples = [{"control_before_ms": elapsed_ms(control), "candidate_ms": elapsed_ms(ours),
                            "control_after_ms": elapsed_ms(control)} for _ in range(a.trials)]
                row["trials"] = triples
                row.update(paired_timing_metrics(triples, a.minimum_gain))
                row["tflops"] = flops / (row["median_ms"] * 1e9)
                row["status"] = "ok"
                row["eligible"] = err <= a.maximum_relative_rms and row["timing_eligible"]
            except Exception as error:  # noqa: BLE001
                row["status"], row["error"] = "error", f"{type(error).__name__}: {str(error)[:2000]}"
            finally:
                lib.ws_gemm_set_pair_mode(-1)
                lib.ws_gemm_set_sm_limit(0)
            report["results"].append(row)
            save()
            print(json.dumps({k2: row.get(k2) for k2 in ("status", "median_ms", "paired_gain", "tflops", "relative_rms_error")}
                             | {"case": policy_key(case), **candidate}), flush=True)
        del x, w, dy, grad, reference
    report["finished"] = time.time()
    save()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
