"""Compute / communication overlap from saved chrome traces (no GPU needed).

For every rank and device of the given traces (``train_bench --profile`` writes them) the tool
classifies each device activity as communication -- NCCL kernels and this framework's own
collective kernels (``grad_reduce_kernel`` and its ``bucket_ready_kernel``, ``norm_exchange_kernel``, ``gather_cast_kernel``,
``adamw_shard_push_kernel``) -- or compute
(every other kernel, copies and fills), and sweeps the interval boundaries once to get, in
microseconds: time with only compute running, only communication running (the *exposed*
communication), both, and idle time inside the traced span.  For NCCL kernels the logical
payload is taken from the trace metadata, one entry per (process group, sequence number); channel
kernels of one collective are not counted twice.  The CPU-side order of c10d collective calls is
fingerprinted so that two runs can be checked for the same bucket order.

    python -m warpstate_ai_b200.bench.comm_profile out/profile-rank-*-trace.json --output report.json

Same report fields as the reference's ops/analyze_communication_profile.py:38-182 (different
algorithm: one boundary sweep instead of merged interval lists).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import re
from collections import Counter
from pathlib import Path

ACTIVITY = {"kernel", "gpu_memcpy", "gpu_memset"}
OWN_COLLECTIVES = ("grad_reduce_kernel", "bucket_ready_kernel", "norm_exchange_kernel", "node_barrier_kernel",
                   "gather_cast_kernel", "adamw_shard_push_kernel")
C10D_PREFIX = "c10d::"
DTYPE_BYTES = {"float": 4, "float32": 4, "double": 8, "float64": 8, "half": 2, "float16": 2, "bfloat16": 2,
               "long": 8, "int64": 8, "int": 4, "int32": 4, "short": 2, "int16": 2, "char": 1, "int8": 1,
               "byte": 1, "uint8": 1, "bool": 1}


def is_communication(name: str) -> bool:
    low = name.lower()
    return "nccl" in low or any(k in name for k in OWN_COLLECTIVES)


def sweep(compute, communication) -> dict:
    """One pass over all interval boundaries; overlapping streams are counted once per class."""
    points = []
    for kind, intervals in enumerate((compute, communication)):
        for begin, end in intervals:
            if not (math.isfinite(begin) and math.isfinite(end)):
                raise ValueError("activity intervals must have finite endpoints")
            if end > begin:                       # an activity of no duration occupies nothing and bounds nothing
                points += [(begin, kind, 1), (end, kind, -1)]
    points.sort(key=lambda p: (p[0], -p[2]))  # at equal time open before close: touching intervals merge
    live = [0, 0]
    totals = {"compute_only": 0.0, "communication_only": 0.0, "both": 0.0, "idle": 0.0}
    previous = None
    for time, kind, delta in points:
        if previous is not None and time > previous:
            span = time - previous
            key = ("both" if live[0] and live[1] else "compute_only" if live[0] else
                   "communication_only" if live[1] else "idle")
            totals[key] += span
        live[kind] += delta
        previous = time
    return totals


def nccl_payload(kernels) -> dict:
    calls, missing = {}, 0
    for event in sorted(kernels, key=lambda e: e["ts"]):
        args = event.get("args", {})
        seq = args.get("Seq")
        if args.get("Process Group Name") is None or not args.get("Collective name") or not str(seq).isdigit():
            missing += 1
            continue
        key = (str(args["Process Group Name"]), str(seq))
        count = args.get("In msg nelems")
        width = DTYPE_BYTES.get(str(args.get("dtype", "")).lower())
        size = count * width if isinstance(count, int) and count >= 0 and width else None
        row = {"process_group": key[0], "sequence": key[1], "collective": args["Collective name"],
               "dtype": args.get("dtype"), "input_elements": count, "input_payload_bytes": size}
        seen = calls.get(key)
        if seen is None:
            calls[key] = {**row, "kernel_count": 1, "metadata_consistent": True}
        else:
            seen["kernel_count"] += 1
            if any(seen[k] != v for k, v in row.items()):
                seen["metadata_consistent"] = False
                seen["input_payload_bytes"] = None
    rows = list(calls.values())
    known = sum(r["input_payload_bytes"] or 0 for r in rows)
    complete = not missing and all(r["metadata_consistent"] and r["input_payload_bytes"] is not None for r in rows)
    return {"nccl_kernel_count": len(kernels), "collective_call_count": None if missing else len(rows),
            "known_collective_call_count": len(rows), "kernels_missing_collective_identity": missing,
            "logical_input_payload_bytes": known if complete else None, "known_logical_input_payload_bytes": known,
            "collectives": rows}


def cpu_collective_fingerprint(events) -> dict:
    calls = sorted((e for e in events if e.get("ph") == "X" and e.get("cat") == "cpu_op"
                    and str(e.get("name", "")).startswith(C10D_PREFIX)), key=lambda e: e["ts"])
    sequence = [{"operator": e["name"], "input_dims": e.get("args", {}).get("Input Dims"),
                 "input_types": e.get("args", {}).get("Input type")} for e in calls]
    text = json.dumps(sequence, sort_keys=True, separators=(",", ":"))
    return {"call_count": len(sequence), "sequence": sequence,
            "sha256": hashlib.sha256(text.encode()).hexdigest() if sequence else None}


def summarize_trace(trace: dict) -> dict:
    events = trace.get("traceEvents", [])
    devices, annotations = {}, 0
    for e in events:
        if e.get("ph") != "X":
            continue
        if e.get("cat") == "gpu_user_annotation":
            annotations += 1
        if e.get("cat") not in ACTIVITY:
            continue
        begin, dur = e.get("ts"), e.get("dur")
        if not isinstance(begin, (int, float)) or not isinstance(dur, (int, float)) or dur < 0:
            raise ValueError("device activities need numeric timestamps and non-negative durations")
        device = str(e.get("args", {}).get("device", e.get("pid", "unknown")))
        d = devices.setdefault(device, {"compute": [], "communication": [], "nccl": [], "own": Counter()})
        name = e.get("name", "")
        if e.get("cat") == "kernel" and is_communication(name):
            d["communication"].append((begin, begin + dur))
            if "nccl" in name.lower():
                d["nccl"].append(e)
            else:
                d["own"][name.split("(")[0]] += 1
        else:
            d["compute"].append((begin, begin + dur))
    rows = []
    for device, d in sorted(devices.items()):
        t = sweep(d["compute"], d["communication"])
        comm = t["communication_only"] + t["both"]
        everything = [(b, e) for b, e in d["compute"] + d["communication"] if e > b]      # an empty activity spans nothing
        span = (max(e for _, e in everything) - min(b for b, _ in everything)) if everything else 0.0
        rows.append({"device": device, "activity_span_us": span,
                     "active_union_us": t["compute_only"] + t["communication_only"] + t["both"],
                     "idle_within_activity_span_us": t["idle"],
                     "noncommunication_union_us": t["compute_only"] + t["both"], "communication_union_us": comm,
                     "compute_only_us": t["compute_only"], "compute_communication_overlap_us": t["both"],
                     "communication_only_us": t["communication_only"],
                     "communication_overlap_fraction": t["both"] / comm if comm else None,
                     "summed_noncommunication_us": sum(e - b for b, e in d["compute"]),
                     "summed_communication_us": sum(e - b for b, e in d["communication"]),
                     "nccl_kernel_names": dict(Counter(e["name"] for e in d["nccl"])),
                     "own_collective_kernels": dict(d["own"]), **nccl_payload(d["nccl"])})
    return {"rank": trace.get("distributedInfo", {}).get("rank"), "distributed_info": trace.get("distributedInfo"),
            "devices": rows, "excluded_gpu_annotation_ranges": annotations,
            "cpu_collective_fingerprint": cpu_collective_fingerprint(events)}


LIMITATIONS = [
    "Budgets are per rank and device; never add ranks or devices into a wall-time estimate.",
    "Compute is every non-collective kernel, copy and fill.",
    "Communication-only time is exposed time, not a delay that is guaranteed removable.",
    "Payload bytes are logical collective inputs of NCCL calls; the in-kernel collectives carry no metadata "
    "in a trace (their bytes follow from the bucket layout).",
    "Spans exclude untraced start-up and tail; profiling adds overhead.",
]


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("traces", nargs="+", type=Path)
    p.add_argument("--output", required=True, type=Path)
    a = p.parse_args(argv)
    if a.output.suffix != ".json":
        p.error("--output must be a .json file")
    if a.output.exists():
        p.error("output already exists; choose a new report path")
    report = {"format": "warpstate-communication-profile-v1",
              "analyzer_sha256": hashlib.sha256(Path(__file__).read_bytes()).hexdigest(), "ranks": [],
              "limitations": LIMITATIONS}
    for path in a.traces:
        payload = path.read_bytes()
        summary = summarize_trace(json.loads(payload))
        if summary["rank"] is None:
            match = re.search(r"profile-rank-(\d+)", path.name)
            if match:
                summary["rank"] = int(match.group(1))
        report["ranks"].append({"trace": str(path), "trace_sha256": hashlib.sha256(payload).hexdigest(), **summary})
    a.output.parent.mkdir(parents=True, exist_ok=True)
    partial = a.output.with_name(a.output.name + ".partial")
    with partial.open("x") as f:
        f.write(json.dumps(report, indent=2, allow_nan=False) + "\n")
    partial.replace(a.output)
    print(json.dumps({"output": str(a.output), "traces": len(report["ranks"])}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
