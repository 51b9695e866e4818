"""Paired comparison of two `train_bench` output directories (control vs candidate).

Two runs are comparable only if they measured the same thing: same model configuration,
checkpoint and data identity, geometry (world size, micro-batch, sequence length, tokens per
update), precision, optimizer-state choice and update counts, none of them profiled.  The tool
refuses anything else, then pairs update ``i`` of both runs and reports, per update, the
slowest-rank seconds of each run, the throughput ratio, and the per-rank loss / gradient-norm
differences (a change of the communication path must not change the numbers), plus timing
statistics (mean, median, population std, first-five vs last-five drift) and peak memory.

    python -m warpstate_ai_b200.bench.compare_runs --control dir_a --candidate dir_b --output cmp.json

Same checks and report as the reference's ops/compare_communication_benchmarks.py:50-234, over
this framework's benchmark records (rank-<r>.jsonl + summary.json).  A directory written by the
reference's own benchmark (``summary.json`` with a ``configuration`` and embedded ranks) is read as
well, so a run of the reference and a run of this framework from the same checkpoint and data can be
paired; between the two layouts the model is matched by its parameter count.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import statistics
from pathlib import Path

MUST_MATCH = ("world_size", "geometry", "precision", "optimizer_state", "warmup_updates", "measured_updates")
IDENTITIES = ("checkpoint", "data")
LIMITATIONS = [
    "Checkpoint and data identities are recorded path, size and modification time, not content hashes.",
    "Elapsed time of an update is the slowest rank's; ranks are never added up.",
    "Consecutive update pairs are neither randomised trials nor independent samples: no confidence interval follows.",
    "Recorded differences (gradient path, optimizer, sources, library, device) are disclosed, not judged.",
    "No threshold names a winner: read the drift, the numerical differences and the peak memory.",
]
MAY_DIFFER = ("grad_sync", "optimizer", "bucket_cap_mb", "reference_execution_flags", "source_sha256", "torch", "device")


def finite(value, name: str, positive: bool = False) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or (positive and value <= 0):
        raise ValueError(f"{name} must be a finite{' positive' if positive else ''} number")
    return float(value)


def load_run(directory: Path) -> dict:
    directory = Path(directory)
    inputs = []

    def read(path: Path) -> bytes:
        data = path.read_bytes()
        inputs.append({"path": str(path), "sha256": hashlib.sha256(data).hexdigest()})
        return data

    summary = json.loads(read(directory / "summary.json"))
    if "format" not in summary and "configuration" in summary:
        return _load_reference_run(directory, summary, read, inputs)
    if summary.get("format") != "warpstate-training-benchmark-v1":
        raise ValueError(f"{directory}: not a training-benchmark summary")
    world = summary["world_size"]
    geometry = summary["geometry"]
    if geometry["global_tokens_per_update"] != world * geometry["grad_accum"] * geometry["micro_batch"] * geometry["seq_len"]:
        raise ValueError("global batch does not match world size, accumulation, micro-batch and sequence length")
    if summary.get("profile") is not None:
        raise ValueError("comparisons need unprofiled runs")
    ranks = {}
    total = summary["warmup_updates"] + summary["measured_updates"]
    for rank in range(world):
        rows = [json.loads(line) for line in read(directory / f"rank-{rank}.jsonl").splitlines() if line.strip()]
        if len(rows) != total:
            raise ValueError(f"rank {rank}: {len(rows)} records, expected {total}")
        for index, row in enumerate(rows):
            if row["update"] != index or row["measured"] != (index >= summary["warmup_updates"]):
                raise ValueError("update records must describe one continuous benchmark")
            if row.get("profiled"):
                raise ValueError("profiled updates cannot be compared")
            finite(row["seconds"], "update seconds", positive=True)
            finite(row["loss"], "loss")
            finite(row["grad_norm"], "grad_norm")
            if row["tokens"] != geometry["global_tokens_per_update"]:
                raise ValueError("update token count differs from the geometry")
            if not math.isclose(row["tokens_per_second"], row["tokens"] / row["slowest_rank_seconds"], rel_tol=1e-9):
                raise ValueError("recorded throughput disagrees with tokens and elapsed time")
        ranks[rank] = rows
    return {"directory": str(directory), "summary": summary, "ranks": ranks, "input_files": inputs}


def _load_reference_run(directory: Path, summary: dict, read, inputs: list) -> dict:
    """A directory written by the reference's benchmark (ops/benchmark_training.py:455-590: ``configuration`` with the
    parsed ``args``, updates numbered from one with a ``phase``, peaks in GiB), brought to this comparator's terms, so
    that a run of the reference and a run of this framework from the same checkpoint and data can be paired."""
    config = summary["configuration"]
    args = config["args"]
    world, warmup, measured = config["world_size"], args["warmup_updates"], args["measured_updates"]
    tokens = args["global_tokens_per_update"]
    if tokens != world * config["grad_accum"] * args["micro_batch"] * args["seq_len"]:
        raise ValueError("global batch does not match world size, accumulation, micro-batch and sequence length")
    if args.get("profile") or config.get("checkpoint_writes"):
        raise ValueError("comparisons need unprofiled runs without checkpoint writes")
    sources = summary.get("ranks") or ([summary] if world == 1 else None)
    if sources is None:                      # older summaries: the per-rank files are the record
        sources = []
        for rank in range(world):
            rows = [json.loads(line) for line in read(directory / f"rank-{rank}.jsonl").splitlines() if line.strip()]
            sources.append({"configuration": {"rank": rank}, "updates": [row for row in rows if row.get("event") == "update"]})
    ranks = {}
    for source in sources:
        rank = source["configuration"].get("rank", 0)
        if type(rank) is not int or not 0 <= rank < world or rank in ranks:
            raise ValueError("rank records must be complete and distinct")
        if len(source["updates"]) != warmup + measured:
            raise ValueError(f"rank {rank}: {len(source['updates'])} records, expected {warmup + measured}")
        rows = []
        for index, update in enumerate(source["updates"]):
            if update.get("update") != index + 1 or update.get("phase") != ("warmup" if index < warmup else "measured"):
                raise ValueError("update records must describe one continuous benchmark")
            if update.get("profiled") is not False:
                raise ValueError("profiled updates cannot be compared")
            if update.get("global_tokens") != tokens:
                raise ValueError("update token count differs from the geometry")
            seconds = finite(update["seconds"], "update seconds", positive=True)
            if not math.isclose(update.get("tokens_per_second", 0), tokens / seconds, rel_tol=1e-9):
                raise ValueError("recorded throughput disagrees with tokens and elapsed time")
            rows.append({"update": index, "measured": index >= warmup, "seconds": seconds, "tokens": tokens,
                         "loss": finite(update["loss"], "loss"), "grad_norm": finite(update["grad_norm"], "grad_norm"),
                         "tokens_per_second": update["tokens_per_second"], "slowest_rank_seconds": seconds,
                         "peak_allocated_bytes": int(finite(update["peak_allocated_gib"], "peak_allocated_gib") * 2 ** 30),
                         "peak_reserved_bytes": int(finite(update["peak_reserved_gib"], "peak_reserved_gib") * 2 ** 30)})
        ranks[rank] = rows
    if len(ranks) != world:
        raise ValueError("rank records must be complete and distinct")

    def identity(entry):
        return None if entry is None else {"path": entry["path"], "bytes": entry["size"], "mtime_ns": entry["mtime_ns"]}

    dtype = {"float32": "fp32", "bfloat16": "bf16", "float16": "fp16"}
    view = {"format": "warpstate-training-benchmark-v1", "implementation": "reference", "world_size": world,
            "device": config.get("gpu"), "model": {"parameters": config["parameters"], "config": None},
            "geometry": {"micro_batch": args["micro_batch"], "seq_len": args["seq_len"], "global_tokens_per_update": tokens,
                         "grad_accum": config["grad_accum"]},
            "precision": {"compute": dtype.get(config["autocast_dtype"], config["autocast_dtype"]),
                          "master": dtype.get(config["parameter_dtype"], config["parameter_dtype"]),
                          "grads": dtype.get(config["parameter_dtype"], config["parameter_dtype"]),
                          "residual_stream": "bf16" if args.get("bf16_residuals") else "fp32"},
            "grad_sync": "ddp", "optimizer": config.get("optimizer"), "bucket_cap_mb": args.get("ddp_bucket_cap_mb"),
            "checkpoint": identity(config.get("checkpoint")), "data": identity(config.get("data")),
            "optimizer_state": args["optimizer_state"], "warmup_updates": warmup, "measured_updates": measured,
            "source_sha256": config.get("source_sha256"), "torch": config.get("torch"), "profile": None}
    return {"directory": str(directory), "summary": view, "ranks": ranks, "input_files": inputs}


def differences(left: dict, right: dict) -> dict:
    """Keys whose values differ, or that only one side recorded (an absent key is not the same as a recorded ``None``)."""
    table = {}
    for key in sorted(set(left) | set(right)):
        if (key in left) != (key in right) or left.get(key) != right.get(key):
            table[key] = {"control": left.get(key), "candidate": right.get(key),
                          "control_recorded": key in left, "candidate_recorded": key in right}
    return table


def timing_statistics(seconds: list, tokens: int) -> dict:
    early, late = statistics.mean(seconds[:5]), statistics.mean(seconds[-5:])
    return {"updates": len(seconds), "mean_seconds": statistics.mean(seconds), "median_seconds": statistics.median(seconds),
            "std_seconds": statistics.pstdev(seconds), "std_definition": "population",
            "tokens_per_second": len(seconds) * tokens / sum(seconds), "first_five_mean_seconds": early,
            "last_five_mean_seconds": late, "first_to_last_seconds_drift_fraction": late / early - 1,
            "drift_windows_overlap": len(seconds) < 10}


def compare(control: dict, candidate: dict) -> dict:
    a, b = control["summary"], candidate["summary"]
    for key in MUST_MATCH:
        if a.get(key) != b.get(key):
            raise ValueError(f"incompatible runs: {key} differs ({a.get(key)} vs {b.get(key)})")
    if "reference" in (a.get("implementation"), b.get("implementation")):      # its record has no model configuration
        if a["model"]["parameters"] != b["model"]["parameters"]:
            raise ValueError("incompatible runs: parameter count differs")
    elif a["model"]["config"] != b["model"]["config"]:
        raise ValueError("incompatible runs: model configuration differs")
    for key in IDENTITIES:
        if a.get(key) != b.get(key):
            raise ValueError(f"incompatible runs: {key} identity differs")
    start, tokens = a["warmup_updates"], a["geometry"]["global_tokens_per_update"]
    paired = []
    for index in range(start, start + a["measured_updates"]):
        per_rank = []
        for rank in sorted(control["ranks"]):
            x, y = control["ranks"][rank][index], candidate["ranks"][rank][index]
            per_rank.append({"rank": rank, "control_loss": x["loss"], "candidate_loss": y["loss"],
                             "loss_difference": y["loss"] - x["loss"], "control_grad_norm": x["grad_norm"],
                             "candidate_grad_norm": y["grad_norm"], "grad_norm_difference": y["grad_norm"] - x["grad_norm"],
                             "grad_norm_relative_difference": abs(y["grad_norm"] - x["grad_norm"]) / max(abs(x["grad_norm"]), 1e-30)})
        cs = max(rows[index]["seconds"] for rows in control["ranks"].values())
        ds = max(rows[index]["seconds"] for rows in candidate["ranks"].values())
        paired.append({"update": index + 1, "control_seconds": cs, "candidate_seconds": ds, "throughput_ratio": cs / ds,
                       "ranks": per_rank})
    ct = timing_statistics([p["control_seconds"] for p in paired], tokens)
    dt = timing_statistics([p["candidate_seconds"] for p in paired], tokens)
    memory = []
    for rank in sorted(control["ranks"]):
        row = {"rank": rank}
        for label, run in (("control", control), ("candidate", candidate)):
            rows = run["ranks"][rank][start:]
            row[label] = {k: max((r.get(k) or 0) for r in rows) for k in ("peak_allocated_bytes", "peak_reserved_bytes")}
        memory.append(row)
    return {"control_timing": ct, "candidate_timing": dt, "throughput_ratio": dt["tokens_per_second"] / ct["tokens_per_second"],
            "maximum_absolute_loss_difference": max(abs(r["loss_difference"]) for p in paired for r in p["ranks"]),
            "maximum_relative_grad_norm_difference": max(r["grad_norm_relative_difference"] for p in paired for r in p["ranks"]),
            "paired_updates": paired, "rank_peak_memory": memory,
            "recorded_differences": differences({k: a[k] for k in MAY_DIFFER if k in a}, {k: b[k] for k in MAY_DIFFER if k in b})}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--control", required=True, type=Path)
    p.add_argument("--candidate", required=True, type=Path, nargs="+", action="append",
                   help="one or more run directories; the flag may be repeated")
    p.add_argument("--output", required=True, type=Path)
    a = p.parse_args(argv)
    if a.output.suffix != ".json" or a.output.exists():
        p.error("the report is a new .json file; this path exists already or has another suffix")
    control = load_run(a.control)
    report = {"format": "warpstate-benchmark-comparison-v1", "control": {k: control[k] for k in ("directory", "input_files")},
              "comparisons": []}
    for directory in (path for group in a.candidate for path in group):
        candidate = load_run(directory)
        report["comparisons"].append({"candidate": {k: candidate[k] for k in ("directory", "input_files")},
                                      **compare(control, candidate)})
    report["limitations"] = LIMITATIONS
    a.output.parent.mkdir(parents=True, exist_ok=True)
    partial = a.output.with_name(a.output.name + ".partial")
    partial.write_text(json.dumps(report, indent=2, allow_nan=False) + "\n")
    partial.replace(a.output)                                                # a reader never sees half a report
    print(json.dumps({"output": str(a.output), "throughput_ratios": [c["throughput_ratio"] for c in report["comparisons"]]}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
