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
from pathlib import Path
from types import SimpleNamespace

import torch

from ..data import sft as D
from ..utils.io import digest, utc_timestamp


def run(snapshot: Path, data_dir: Path, output: Path, device: torch.device, micro_batch: int = 4) -> dict:
    from ..serve.chat import load_model
    from .sft import evaluate
    snapshot, data_dir, output = snapshot.resolve(), data_dir.resolve(), output.resolve()
    if output.exists() or output.is_relative_to(snapshot.parent) or output.is_relative_to(data_dir):
        raise ValueError("Select a new report outside the snapshot and dataset directories")
    started = time.perf_counter()
    tokenizer = snapshot.with_name("tokenizer.model")
    model, sp, metadata = load_model(snapshot, tokenizer, device=str(device))
    manifest = json.loads((data_dir / "manifest.json").read_text())
    _, records, manifest, data_hash = D.load_data(data_dir, sp, metadata["tokenizer_sha256"], manifest["max_length"])
    print(f"Validated {len(records):,} SFT holdout conversations; evaluating on {device}", flush=True)
    settings = dict(sequence_length=manifest["max_length"], micro_batch=micro_batch, eval_batches=32)
    pad_id = sp.pad_id() if sp.pad_id() >= 0 else sp.eos_id()
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    evaluation_started = time.perf_counter()
    loss, targets = evaluate(SimpleNamespace(model=model, device=device), records, settings, pad_id, full=True)
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    report = dict(
        format="warpstate-sft-snapshot-evaluation-v1", timestamp_utc=utc_timestamp(), snapshot=str(snapshot),
        snapshot_sha256=digest(snapshot), snapshot_metadata=metadata, data_sha256=data_hash,
        holdout_sha256=manifest["outputs"]["sft_val.jsonl"]["sha256"], renderer_sha256=D.renderer_sha256(),
        full_holdout=True, evaluated_samples=len(records), assistant_target_tokens=targets, val_loss=loss,
        val_perplexity=math.exp(loss), objective="assistant-token-mean", settings=settings,
        execution=dict(device=str(device),
                       device_name=torch.cuda.get_device_name(device) if device.type == "cuda" else "cpu",
                       torch_version=torch.__version__, compute_dtype="bfloat16" if device.type == "cuda" else "float32",
                       parameter_dtype="float32"),
        evaluation_seconds=time.perf_counter() - evaluation_started, total_seconds=time.perf_counter() - started,
        peak_allocated_bytes=torch.cuda.max_memory_allocated(device) if device.type == "cuda" else None)
    output.parent.mkdir(parents=True, exist_ok=True)
    with output.open("x") as stream:
        json.dump(report, stream, indent=2, allow_nan=False, default=str)
        stream.write("\n")
    return report


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--snapshot", type=Path, required=True)
    p.add_argument("--data-dir", type=Path, required=True)
    p.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    p.add_argument("--micro-batch", type=int, default=4)
    p.add_argument("--output", type=Path, required=True)
    a = p.parse_args(argv)
    device = torch.device(a.device)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    report = run(a.snapshot, a.data_dir, a.output, device, a.micro_batch)
    print(json.dumps({k: report[k] for k in ("evaluated_samples", "assistant_target_tokens", "val_loss",
                                             "val_perplexity", "evaluation_seconds")}) + f"\nReport: {a.output}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
