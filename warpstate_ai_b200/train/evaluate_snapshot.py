"""Evaluate a sealed post-training snapshot on the complete pinned SFT hold-out.

The snapshot (``model.pt`` + ``snapshot.json`` + ``tokenizer.model`` in one directory) is verified
against its recorded hash, the prepared data directory against its manifest (format, completion,
tokenizer and renderer identity, per-file checksum, exact re-encoding of every conversation), and
the assistant-token mean loss is computed over every hold-out conversation with the same
evaluation routine the SFT trainer uses.  The report is written once (never overwritten) and
records the identities of everything that went into the number.

    python -m warpstate_ai_b200.train.evaluate_snapshot --snapshot dir/model.pt --data-dir data --output eval.json

Reference: ops/evaluate_sft_snapshot.py:23-110 (CUDA-only there; this one also runs on CPU so
that the tool itself is testable).
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import time
from dataclasses import dataclass
from pathlib import Path

import torch

from ..data import sft as D
from ..utils.io import digest, utc_timestamp

REPORT_FORMAT = "warpstate-sft-snapshot-evaluation-v1"
SUMMARY_KEYS = ("evaluated_samples", "assistant_target_tokens", "val_loss", "val_perplexity", "evaluation_seconds")


@dataclass
class _Evaluator:
    """The two attributes `train.sft.evaluate` reads from a trainer."""
    model: torch.nn.Module
    device: torch.device


def _write_once(path: Path, report: dict) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("x") as out:
        out.write(json.dumps(report, indent=2, allow_nan=False, default=str) + "\n")


def run(snapshot: Path, data_dir: Path, output: Path, device: torch.device, micro_batch: int = 4) -> dict:
    from ..serve.snapshots import SnapshotStore
    from .sft import evaluate
    snapshot, data_dir, output = (Path(p).resolve() for p in (snapshot, data_dir, output))
    if output.exists() or any(output.is_relative_to(place) for place in (snapshot.parent, data_dir)):
        raise ValueError(f"{output}: write the new report to a fresh file outside the snapshot and data directories")
    clock = time.perf_counter
    began = clock()
    store = SnapshotStore(snapshot.parent.parent, snapshot.with_name("tokenizer.model"))
    model, tokenizer, metadata = store.load(snapshot, str(device))
    max_length = json.loads((data_dir / "manifest.json").read_text())["max_length"]
    _, holdout, manifest, data_hash = D.load_data(data_dir, tokenizer, metadata["tokenizer_sha256"], max_length)
    print(f"Validated {len(holdout):,} SFT holdout conversations; evaluating on {device}", flush=True)
    on_gpu = device.type == "cuda"
    if on_gpu:
        torch.cuda.reset_peak_memory_stats(device)
    settings = {"sequence_length": max_length, "micro_batch": micro_batch, "eval_batches": 32}
    pad = tokenizer.pad_id() if tokenizer.pad_id() >= 0 else tokenizer.eos_id()
    measured_from = clock()
    loss, tokens = evaluate(_Evaluator(model, device), holdout, settings, pad, full=True)
    if on_gpu:
        torch.cuda.synchronize(device)
    finished = clock()
    report = {
        "format": REPORT_FORMAT, "timestamp_utc": utc_timestamp(), "snapshot": str(snapshot),
        "snapshot_sha256": digest(snapshot), "snapshot_metadata": metadata, "data_sha256": data_hash,
        "holdout_sha256": manifest["outputs"]["sft_val.jsonl"]["sha256"], "renderer_sha256": D.renderer_sha256(),
        "full_holdout": True, "evaluated_samples": len(holdout), "assistant_target_tokens": tokens, "val_loss": loss,
        "val_perplexity": math.exp(loss), "objective": "assistant-token-mean", "settings": settings,
        "execution": {"device": str(device), "device_name": torch.cuda.get_device_name(device) if on_gpu else "cpu",
                      "torch_version": torch.__version__, "compute_dtype": "bfloat16" if on_gpu else "float32",
                      "parameter_dtype": "float32"},
        "evaluation_seconds": finished - measured_from, "total_seconds": finished - began,
        "peak_allocated_bytes": torch.cuda.max_memory_allocated(device) if on_gpu else None}
    _write_once(output, report)
    return report


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--snapshot", type=Path, required=True, help="model.pt of a sealed export")
    parser.add_argument("--data-dir", type=Path, required=True, help="prepared post-training data")
    parser.add_argument("--output", type=Path, required=True, help="report file (must not exist)")
    parser.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    parser.add_argument("--micro-batch", type=int, default=4)
    args = parser.parse_args(argv)
    device = torch.device(args.device)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    report = run(args.snapshot, args.data_dir, args.output, device, args.micro_batch)
    print(json.dumps({key: report[key] for key in SUMMARY_KEYS}), flush=True)
    print(f"Report: {args.output}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
