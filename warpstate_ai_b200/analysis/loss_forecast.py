"""Loss-curve sensitivity study from a frozen validation log (CPU only).

Reads a JSONL snapshot with ``{"tokens": int, "loss": float}`` rows (the ``validation`` events of
``metrics.jsonl``), averages them over complete token bins (default 0.25 B tokens), and fits, for
several window starts, three families in loss space with equal weights:

* ``log``           L = a + b ln t
* ``power_free``    L = f + A t^-alpha with the floor f fitted in [0, min binned loss], A >= 0
* ``power_fixed:f`` the same with an assumed floor f (a sensitivity assumption, not a measurement)

For each fit it reports RMSE, the token count at which the curve crosses a target loss, the
predicted loss at given budgets, and hold-out checks (fit up to E, predict the next complete
billion).  These are illustrations of how strongly an extrapolation depends on the assumed
family; they are not confidence intervals or ETAs.

    python -m warpstate_ai_b200.analysis.loss_forecast --input val.jsonl --output forecast.json

Covers the reference's ops/loss_curve_forecast.py:27-150 (alpha is found here with a bounded
scalar minimiser on ln alpha; the linear parameters are solved in closed form for each alpha).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import platform
from pathlib import Path

import numpy as np
from scipy.optimize import minimize_scalar

ALPHA_RANGE = (1e-4, 3.0)


def linear_for_alpha(x, y, alpha: float, fixed_floor):
    """Closed-form (floor, amplitude, mse) of L = f + A x^-alpha for one alpha."""
    z = x ** (-alpha)
    if fixed_floor is None:
        zc = z - z.mean()
        denom = float(zc @ zc)
        amplitude = float(zc @ (y - y.mean()) / denom) if denom > 0 else 0.0
        floor = float(np.clip(y.mean() - amplitude * z.mean(), 0.0, y.min()))
    else:
        floor = float(fixed_floor)
    amplitude = max(0.0, float(z @ (y - floor) / (z @ z)))
    return floor, amplitude, float(np.mean((floor + amplitude * z - y) ** 2))


def fit(x, y, model: str) -> dict:
    if len(x) < 3:
        raise ValueError("each fitting window needs at least three complete bins")
    if model == "log":
        slope, intercept = np.polyfit(np.log(x), y, 1)
        mse = float(np.mean((intercept + slope * np.log(x) - y) ** 2))
        return {"model": model, "intercept": float(intercept), "slope": float(slope), "rmse": math.sqrt(mse)}
    fixed = None if model == "power_free" else float(model.split(":", 1)[1])
    lo, hi = math.log(ALPHA_RANGE[0]), math.log(ALPHA_RANGE[1])
    coarse = np.linspace(lo, hi, 200)  # the objective can have a flat shoulder: bracket the best coarse point
    errors = [linear_for_alpha(x, y, math.exp(v), fixed)[2] for v in coarse]
    best = int(np.argmin(errors))
    bracket = (coarse[max(best - 1, 0)], coarse[min(best + 1, len(coarse) - 1)])
    result = minimize_scalar(lambda v: linear_for_alpha(x, y, math.exp(v), fixed)[2], bounds=bracket, method="bounded",
                             options={"xatol": 1e-10})
    alpha = math.exp(float(result.x))
    floor, amplitude, mse = linear_for_alpha(x, y, alpha, fixed)
    return {"model": model, "floor": floor, "amplitude": amplitude, "alpha": alpha, "rmse": math.sqrt(mse),
            "alpha_at_search_boundary": best in (0, len(coarse) - 1)}


def predict(parameters: dict, tokens_b):
    t = np.asarray(tokens_b, dtype=np.float64)
    if parameters["model"] == "log":
        return parameters["intercept"] + parameters["slope"] * np.log(t)
    return parameters["floor"] + parameters["amplitude"] * t ** (-parameters["alpha"])


def crossing(parameters: dict, target: float):
    """Tokens (billions) at which the fitted curve reaches ``target``; None if it never does."""
    if parameters["model"] == "log":
        if parameters["slope"] >= 0:
            return None
        exponent = (target - parameters["intercept"]) / parameters["slope"]
    else:
        if parameters["floor"] >= target or parameters["amplitude"] <= 0:
            return None
        exponent = math.log(parameters["amplitude"] / (target - parameters["floor"])) / parameters["alpha"]
    return math.exp(exponent) if exponent < 700 else None


def bin_rows(rows, width_b: float, first_b: float):
    if not rows or any(b["tokens"] <= a["tokens"] for a, b in zip(rows, rows[1:])):
        raise ValueError("validation snapshot must have strictly increasing token counts")
    right = math.floor(rows[-1]["tokens"] / 1e9 / width_b) * width_b
    bins = []
    left = first_b
    while left < right - 1e-12:
        chosen = [r for r in rows if left <= r["tokens"] / 1e9 < left + width_b]
        if not chosen:
            raise ValueError(f"missing validation data in the bin starting at {left} B tokens")
        bins.append({"left_B": left, "right_B": left + width_b,
                     "tokens_B": float(np.mean([r["tokens"] / 1e9 for r in chosen])),
                     "loss": float(np.mean([r["loss"] for r in chosen])), "count": len(chosen)})
        left = round(left + width_b, 12)
    return bins, right


def analyze(raw: bytes, *, bin_width_b: float = 0.25, first_bin_b: float = 1.0, window_starts=(1, 2, 3, 4, 5),
            fixed_floors=(1.5, 1.8, 1.9, 2.0, 2.1), budgets_b=(40.0, 268.435456, 1073.741824), target: float = 2.0,
            holdout_ends=(4, 5, 6)) -> dict:
    rows = [json.loads(line) for line in raw.splitlines() if line.strip()]
    bins, right = bin_rows(rows, bin_width_b, first_bin_b)
    x = np.array([b["tokens_B"] for b in bins])
    y = np.array([b["loss"] for b in bins])
    models = ("log", "power_free") + tuple(f"power_fixed:{f}" for f in fixed_floors)
    fits = []
    for start in window_starts:
        chosen = x >= start
        if chosen.sum() < 3:
            continue
        for model in models:
            parameters = fit(x[chosen], y[chosen], model)
            fits.append({"start_B": start, "end_B": right, "bins": int(chosen.sum()), "parameters": parameters,
                         f"cross_{target:g}_tokens_B": crossing(parameters, target),
                         "endpoint_losses": {f"{b:g}B": float(predict(parameters, b)) for b in budgets_b}})
    holdouts = []
    for end in holdout_ends:
        train, test = (x >= 2) & (x < end), (x >= end) & (x < end + 1)
        if right < end + 1 or not test.any() or train.sum() < 3:
            continue
        for model in models:
            parameters = fit(x[train], y[train], model)
            error = predict(parameters, x[test]) - y[test]
            holdouts.append({"train_start_B": 2, "train_end_B": end, "test_end_B": end + 1, "parameters": parameters,
                             "actual_mean_loss": float(y[test].mean()),
                             "predicted_mean_loss": float(predict(parameters, x[test]).mean()),
                             "mean_bias": float(error.mean()), "rmse": float(np.sqrt(np.mean(error ** 2)))})
    return {"method": "equal-weight least squares in loss space on complete token bins; x is each bin's mean token "
                      "count in billions; power-law alpha minimised on [1e-4, 3] with closed-form floor/amplitude",
            "caveats": ["Illustrative extrapolations, not confidence intervals or ETAs.",
                        "Short hold-outs do not validate an extrapolation over orders of magnitude.",
                        "Learning-rate schedule, data repetition and distribution changes are not modelled.",
                        "Fixed floors are assumptions; a fitted floor above the target proves no architectural limit."],
            "source_sha256": hashlib.sha256(raw).hexdigest(), "source_rows": len(rows), "latest_validation": rows[-1],
            "complete_bins_end_B": right, "bins": bins, "fits": fits, "holdouts": holdouts}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--input", required=True, type=Path, help="frozen validation JSONL snapshot")
    p.add_argument("--output", required=True, type=Path)
    p.add_argument("--bin-width-b", type=float, default=0.25)
    p.add_argument("--target-loss", type=float, default=2.0)
    a = p.parse_args(argv)
    if a.input.resolve() == a.output.resolve():
        p.error("input and output must be different files")
    report = analyze(a.input.read_bytes(), bin_width_b=a.bin_width_b, target=a.target_loss)
    report["source_path"] = str(a.input)
    report["analysis_sha256"] = hashlib.sha256(Path(__file__).read_bytes()).hexdigest()
    report["versions"] = {"python": platform.python_version(), "numpy": np.__version__}
    a.output.parent.mkdir(parents=True, exist_ok=True)
    a.output.write_text(json.dumps(report, indent=2, allow_nan=False) + "\n")
    print(f"Analyzed {report['source_rows']} validation rows through {report['complete_bins_end_B']:g}B complete bins; "
          f"wrote {a.output}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
