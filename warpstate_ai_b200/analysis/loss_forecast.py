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
from dataclasses import dataclass
from pathlib import Path

import numpy as np
from scipy.optimize import minimize_scalar

ALPHA_RANGE = (1e-4, 3.0)
MIN_BINS = 3


# ----------------------------------------------------------------------------------- curve families
class LogCurve:
    """L = a + b ln t"""
    name = "log"

    def fit(self, t, loss) -> "Fitted":
        design = np.stack([np.ones_like(t), np.log(t)], axis=1)
        (a, b), *_ = np.linalg.lstsq(design, loss, rcond=None)
        residual = design @ np.array([a, b]) - loss
        return Fitted(self, {"model": self.name, "intercept": float(a), "slope": float(b),
                             "rmse": float(np.sqrt(np.mean(residual ** 2)))})

    def evaluate(self, p: dict, t):
        return p["intercept"] + p["slope"] * np.log(t)

    def log_crossing(self, p: dict, target: float):
        return (target - p["intercept"]) / p["slope"] if p["slope"] < 0 else None


class PowerCurve:
    """L = f + A t^-alpha with A >= 0; the floor f is fitted in [0, min loss] or fixed by assumption.
    For a given alpha the curve is linear in (f, A), so alpha is the only searched parameter."""

    def __init__(self, floor: float | None = None):
        self.floor = floor
        self.name = "power_free" if floor is None else f"power_fixed:{floor}"

    def _given_alpha(self, t, loss, alpha: float):
        basis = t ** (-alpha)
        if self.floor is None:
            centred = basis - basis.mean()
            spread = float(centred @ centred)
            slope = float(centred @ (loss - loss.mean())) / spread if spread > 0 else 0.0
            floor = float(min(max(loss.mean() - slope * basis.mean(), 0.0), loss.min()))
        else:
            floor = float(self.floor)
        amplitude = max(float(basis @ (loss - floor)) / float(basis @ basis), 0.0)
        return floor, amplitude, float(np.mean((floor + amplitude * basis - loss) ** 2))

    def fit(self, t, loss) -> "Fitted":
        def error(log_alpha):
            return self._given_alpha(t, loss, math.exp(log_alpha))[2]

        # the error can be flat on one side of its minimum: locate the best of a coarse grid, refine around it
        grid = np.linspace(math.log(ALPHA_RANGE[0]), math.log(ALPHA_RANGE[1]), 200)
        at = int(np.argmin([error(v) for v in grid]))
        around = (grid[max(at - 1, 0)], grid[min(at + 1, grid.size - 1)])
        refined = minimize_scalar(error, bounds=around, method="bounded", options={"xatol": 1e-10})
        alpha = math.exp(float(refined.x))
        floor, amplitude, mse = self._given_alpha(t, loss, alpha)
        return Fitted(self, {"model": self.name, "floor": floor, "amplitude": amplitude, "alpha": alpha,
                             "rmse": math.sqrt(mse), "alpha_at_search_boundary": at in (0, grid.size - 1)})

    def evaluate(self, p: dict, t):
        return p["floor"] + p["amplitude"] * t ** (-p["alpha"])

    def log_crossing(self, p: dict, target: float):
        if p["amplitude"] <= 0 or target <= p["floor"]:
            return None
        return math.log(p["amplitude"] / (target - p["floor"])) / p["alpha"]


@dataclass
class Fitted:
    family: object
    parameters: dict

    def predict(self, tokens_b):
        return self.family.evaluate(self.parameters, np.asarray(tokens_b, dtype=np.float64))

    def crossing(self, target: float):
        """Tokens (billions) at which the curve reaches ``target``; None if never (or beyond e^700)."""
        where = self.family.log_crossing(self.parameters, target)
        return math.exp(where) if where is not None and where < 700 else None


def family_of(model: str):
    if model == "log":
        return LogCurve()
    if model == "power_free":
        return PowerCurve()
    return PowerCurve(float(model.split(":", 1)[1]))


def fit(x, y, model: str) -> dict:
    if len(x) < MIN_BINS:
        raise ValueError(f"a fitting window needs at least {MIN_BINS} complete bins")
    return family_of(model).fit(np.asarray(x, dtype=np.float64), np.asarray(y, dtype=np.float64)).parameters


def predict(parameters: dict, tokens_b):
    return Fitted(family_of(parameters["model"]), parameters).predict(tokens_b)


def crossing(parameters: dict, target: float):
    return Fitted(family_of(parameters["model"]), parameters).crossing(target)


# ----------------------------------------------------------------------------------- binning
def bin_rows(rows, width_b: float, first_b: float):
    """Mean token count and mean loss per complete bin ``[left, left + width)`` (billions of tokens), from
    ``first_b`` to the last bin boundary the data reaches.  -> (bins, that boundary)"""
    tokens_b = np.array([row["tokens"] for row in rows], dtype=np.float64) / 1e9
    losses = np.array([row["loss"] for row in rows], dtype=np.float64)
    if tokens_b.size == 0 or np.any(np.diff(tokens_b) <= 0):
        raise ValueError("the validation rows must have strictly increasing token counts")
    end = math.floor(tokens_b[-1] / width_b) * width_b
    bins, left = [], first_b
    while left < end - 1e-12:
        inside = (tokens_b >= left) & (tokens_b < left + width_b)
        if not inside.any():
            raise ValueError(f"no validation row falls in the bin that starts at {left} B tokens")
        bins.append({"left_B": left, "right_B": left + width_b, "tokens_B": float(tokens_b[inside].mean()),
                     "loss": float(losses[inside].mean()), "count": int(inside.sum())})
        left = round(left + width_b, 12)
    return bins, end


CAVEATS = ["Illustrative extrapolations, not confidence intervals or ETAs.",
           "Short hold-outs do not validate an extrapolation over orders of magnitude.",
           "Learning-rate schedule, data repetition and distribution changes are not modelled.",
           "Fixed floors are assumptions; a fitted floor above the target proves no architectural limit."]
METHOD = ("equal-weight least squares in loss space on complete token bins; x is each bin's mean token count in "
          "billions; power-law alpha minimised on [1e-4, 3] with closed-form floor/amplitude")


def analyze(raw: bytes, *, bin_width_b: float = 0.25, first_bin_b: float = 1.0, window_starts=(1, 2, 3, 4, 5),
            fixed_floors=(1.5, 1.8, 1.9, 2.0, 2.1), budgets_b=(40.0, 268.435456, 1073.741824), target: float = 2.0,
            holdout_ends=(4, 5, 6)) -> dict:
    rows = [json.loads(line) for line in raw.splitlines() if line.strip()]
    bins, end = bin_rows(rows, bin_width_b, first_bin_b)
    t = np.array([b["tokens_B"] for b in bins])
    loss = np.array([b["loss"] for b in bins])
    families = [LogCurve(), PowerCurve(), *(PowerCurve(f) for f in fixed_floors)]
    fits = []
    for start in window_starts:
        window = t >= start
        if window.sum() < MIN_BINS:
            continue
        for family in families:
            curve = family.fit(t[window], loss[window])
            fits.append({"start_B": start, "end_B": end, "bins": int(window.sum()), "parameters": curve.parameters,
                         f"cross_{target:g}_tokens_B": curve.crossing(target),
                         "endpoint_losses": {f"{b:.12g}B": float(curve.predict(b)) for b in budgets_b}})
    holdouts = []
    for stop in holdout_ends:
        known, unseen = (t >= 2) & (t < stop), (t >= stop) & (t < stop + 1)
        if end < stop + 1 or known.sum() < MIN_BINS or not unseen.any():
            continue
        for family in families:
            curve = family.fit(t[known], loss[known])
            guess = curve.predict(t[unseen])
            holdouts.append({"train_start_B": 2, "train_end_B": stop, "test_end_B": stop + 1,
                             "parameters": curve.parameters, "actual_mean_loss": float(loss[unseen].mean()),
                             "predicted_mean_loss": float(guess.mean()), "mean_bias": float((guess - loss[unseen]).mean()),
                             "rmse": float(np.sqrt(np.mean((guess - loss[unseen]) ** 2)))})
    return {"method": METHOD, "caveats": CAVEATS, "source_sha256": hashlib.sha256(raw).hexdigest(),
            "source_rows": len(rows), "latest_validation": rows[-1], "complete_bins_end_B": end,
            "observed_validation": [{"tokens_B": r["tokens"] / 1e9, "loss": r["loss"]} for r in rows if r["tokens"] >= 1e9],
            "bins": bins,
            "fits": fits, "holdouts": holdouts}


# ----------------------------------------------------------------------------------- picture
PALETTE = ("#2469aa", "#ca6d12", "#238456", "#8051a5", "#cfa323", "#8f3333", "#444444")


def plot(report: dict, output: Path, target: float = 2.0) -> None:
    """The report as a picture, written as plain SVG (no plotting library): every validation, the bin means and, for the
    earliest fitting window, each family's curve drawn solid over the data and dashed beyond it, on a logarithmic token
    axis out to the largest budget.  How far apart the dashed lines end is the message of the study."""
    bins = report["bins"]
    if not bins or not report["fits"]:
        raise ValueError("nothing to plot: the report has no bins or no fits")
    end = report["complete_bins_end_B"]
    first = min(f["start_B"] for f in report["fits"])
    curves = [f for f in report["fits"] if f["start_B"] == first]
    budgets = sorted(float(name[:-1]) for name in curves[0]["endpoint_losses"])
    far = max(budgets + [end * 1.25])
    observed = report.get("observed_validation") or [{"tokens_B": b["tokens_B"], "loss": b["loss"]} for b in bins]
    seen = [row["loss"] for row in observed]
    low, high = min(min(seen), target) - 0.15, max(seen) + 0.1
    width, height, left, right, top, bottom = 960, 540, 70, 20, 40, 50

    def at(tokens_b: float, loss: float) -> str:
        x = left + (math.log(tokens_b) - math.log(first)) / (math.log(far) - math.log(first)) * (width - left - right)
        y = top + (high - min(max(loss, low), high)) / (high - low) * (height - top - bottom)
        return f"{x:.1f},{y:.1f}"

    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" viewBox="0 0 {width} {height}" '
             'font-family="sans-serif" font-size="12">', f'<rect width="{width}" height="{height}" fill="white"/>',
             f'<text x="{left}" y="22" font-size="14">Validation loss against tokens trained (billions, log axis): '
             'illustrative scenarios, not confidence intervals</text>']
    for budget in budgets:
        x = at(budget, low).split(",")[0]
        parts.append(f'<line x1="{x}" y1="{top}" x2="{x}" y2="{height - bottom}" stroke="#bbbbbb" stroke-dasharray="2,4"/>')
        parts.append(f'<text x="{x}" y="{height - bottom + 16}" text-anchor="middle">{budget:g}</text>')
    for tick in (first, end):
        x = at(tick, low).split(",")[0]
        parts.append(f'<text x="{x}" y="{height - bottom + 32}" text-anchor="middle" fill="#666666">{tick:g}</text>')
    steps = 6
    for k in range(steps + 1):
        value = low + (high - low) * k / steps
        y = at(first, value).split(",")[1]
        parts.append(f'<line x1="{left}" y1="{y}" x2="{width - right}" y2="{y}" stroke="#eeeeee"/>')
        parts.append(f'<text x="{left - 8}" y="{y}" text-anchor="end" dominant-baseline="middle">{value:.2f}</text>')
    y = at(first, target).split(",")[1]
    parts.append(f'<line x1="{left}" y1="{y}" x2="{width - right}" y2="{y}" stroke="#8f3333" stroke-dasharray="6,4"/>')
    for row in observed:
        if row["tokens_B"] >= first:
            x, y = at(row["tokens_B"], row["loss"]).split(",")
            parts.append(f'<circle cx="{x}" cy="{y}" r="1.6" fill="#999999"/>')
    parts.append('<polyline fill="none" stroke="black" stroke-width="1.5" points="'
                 + " ".join(at(b["tokens_B"], b["loss"]) for b in bins if b["tokens_B"] >= first) + '"/>')
    for index, fit_row in enumerate(curves):
        colour, parameters = PALETTE[index % len(PALETTE)], fit_row["parameters"]
        over = np.linspace(first, end, 60)
        beyond = np.geomspace(end, far, 120)
        for grid, dash in ((over, ""), (beyond, ' stroke-dasharray="7,4"')):
            points = " ".join(at(float(t), float(v)) for t, v in zip(grid, predict(parameters, grid)))
            parts.append(f'<polyline fill="none" stroke="{colour}" stroke-width="1.3"{dash} points="{points}"/>')
        parts.append(f'<text x="{width - right - 4}" y="{top + 14 + 15 * index}" text-anchor="end" fill="{colour}">'
                     f'{parameters["model"]} (fit {first:g}-{end:g} B, rmse {parameters["rmse"]:.4f})</text>')
    parts.append("</svg>")
    output.parent.mkdir(parents=True, exist_ok=True)
    output.write_text("\n".join(parts) + "\n")


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--input", required=True, type=Path, help="frozen validation JSONL snapshot")
    p.add_argument("--output", required=True, type=Path)
    p.add_argument("--bin-width-b", type=float, default=0.25)
    p.add_argument("--target-loss", type=float, default=2.0)
    p.add_argument("--plot", type=Path, help="also draw the report as an SVG picture here")
    a = p.parse_args(argv)
    if a.input.resolve() == a.output.resolve() or (a.plot is not None and a.plot.resolve() in (a.input.resolve(), a.output.resolve())):
        p.error("input, output and plot must be different files")
    report = analyze(a.input.read_bytes(), bin_width_b=a.bin_width_b, target=a.target_loss)
    report["source_path"] = str(a.input)
    report["analysis_sha256"] = hashlib.sha256(Path(__file__).read_bytes()).hexdigest()
    report["versions"] = {"python": platform.python_version(), "numpy": np.__version__}
    a.output.parent.mkdir(parents=True, exist_ok=True)
    a.output.write_text(json.dumps(report, indent=2, allow_nan=False) + "\n")
    if a.plot is not None:
        plot(report, a.plot, a.target_loss)
    print(f"Analyzed {report['source_rows']} validation rows through {report['complete_bins_end_B']:g}B complete bins; "
          f"wrote {a.output}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
