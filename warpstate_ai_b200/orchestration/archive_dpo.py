"""Seal a completed DPO run as a read-only archive, and make a sealed chat copy of it.

The archive is self-describing: it holds the complete training state (``checkpoint.pt``: FP32
model, Adam moments, per-rank RNG), a tensor-exact inference export (``model.pt`` +
``snapshot.json``, ``stage='dpo'``), the tokenizer, the plan and the run's own reports
(settings / evaluation / completion / metrics), the data manifest, the frozen-reference cache
(manifest and both score arrays) and a provenance record.  ``verify`` re-derives every
cross-reference from the preserved files alone -- expected counters from the data manifest and
plan, signatures, ancestry, Adam step counts and dtypes, reference identity, array shapes --
so an archive can be checked years later without the run directory (reference
ops/archive_dpo.py:42-287, ops/prepare_dpo_chat.py).

    python -m warpstate_ai_b200.orchestration.archive_dpo --config plan.json [--verify-only]
    python -m warpstate_ai_b200.orchestration.archive_dpo --chat-copy DEST --archive DIR
"""
from __future__ import annotations

import argparse
import json
import math
import os
import stat
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

from ..ckpt.formats import export_chat_snapshot
from ..train.dpo import DEFAULTS, identity_digest
from ..utils.io import digest, utc_timestamp
from . import archive as A

REPORTS = ("settings.json", "evaluation.json", "completion.json", "metrics.jsonl")
FILES = ("checkpoint.pt", "model.pt", "snapshot.json", "tokenizer.model", "plan.json", *REPORTS, "data-manifest.json",
         "reference-manifest.json", "reference-train.npy", "reference-val.npy", "PROVENANCE.json", "ARCHIVE.md")
CHAT_FILES = ("model.pt", "snapshot.json", "tokenizer.model", "ARCHIVE.md")


def read_json(path):
    return json.loads(Path(path).read_text())


def expected_counters(plan: dict, data: dict) -> dict:
    settings = DEFAULTS | plan["training"]
    world = plan["handoff"]["processes"]
    train = data["outputs"]["dpo_train.jsonl"]
    if settings["max_steps"] is not None:
        raise ValueError("Archive requires a completed whole DPO run, without a plan step cap")
    steps = math.ceil(train["rows"] / (settings["micro_batch"] * settings["grad_accum"] * world)) * settings["epochs"]
    return dict(step=steps, total_steps=steps, sample_cursor=train["rows"] * settings["epochs"],
                tokens_seen=(train["tokens"] - 2 * train["rows"]) * settings["epochs"],
                response_tokens_seen=train["supervised_tokens"] * settings["epochs"], val_step=steps)


def validate_state(checkpoint, evaluation, completion, settings_report, data, reference, plan) -> dict:
    """Consistency of a finished DPO run, judged from its preserved records only."""
    settings = DEFAULTS | plan["training"]
    world = plan["handoff"]["processes"]
    val = data["outputs"]["dpo_val.jsonl"]
    train = data["outputs"]["dpo_train.jsonl"]
    want = expected_counters(plan, data)
    if (checkpoint.get("format") != "warpstate-dpo-v1" or checkpoint.get("completed") is not True
            or any(checkpoint.get(k) != v for k, v in want.items())
            or not math.isfinite(checkpoint.get("val_loss", float("nan")))):
        raise ValueError("DPO checkpoint is not the fully completed, finally evaluated state")
    sig = checkpoint["signature"]
    if (sig.get("plan") != plan or sig.get("settings") != settings or sig.get("world_size") != world
            or settings_report.get("signature") != sig or settings_report.get("total_steps") != want["step"]
            or settings_report.get("train_rows") != train["rows"] or settings_report.get("val_rows") != val["rows"]):
        raise ValueError("DPO checkpoint/settings signatures or dataset counts differ")
    if (data.get("format") != "warpstate-posttrain-data-v1" or data.get("complete") is not True
            or data.get("tokenizer_sha256") != sig["tokenizer_sha256"]
            or data.get("max_length") != settings["sequence_length"]):
        raise ValueError("DPO data provenance differs from its signature")
    origin = checkpoint["origin"]
    parent = plan.get("sft")
    if origin.get("stage") != "sft" or origin.get("weights_sha256") != sig["base_sha256"]:
        raise ValueError("DPO did not start from a sealed SFT export")
    if parent is not None and (origin.get("step") != parent["step"] or origin.get("tokens_seen") != parent["tokens_seen"]):
        raise ValueError("DPO SFT ancestry differs from the authorized plan")
    states = checkpoint.get("optimizer", {}).get("state")
    rng = checkpoint.get("rng_by_rank", [])
    if not states or len(rng) != world or any("torch" not in r for r in rng):
        raise ValueError("DPO optimizer or per-rank RNG state is missing")
    for entry in states.values():
        if float(entry["step"]) != want["step"]:
            raise ValueError("DPO Adam step differs from the final checkpoint")
        if entry["exp_avg"].dtype != torch.float32 or entry["exp_avg_sq"].dtype != torch.float32:
            raise ValueError("DPO Adam state must retain its original FP32 tensors")
    if not checkpoint.get("model"):
        raise ValueError("DPO model tensors are missing")
    for name, tensor in checkpoint["model"].items():
        if tensor.is_floating_point() and tensor.dtype != torch.float32:
            raise ValueError(f"DPO model tensor is not original FP32: {name}")
    counters = ("step", "total_steps", "sample_cursor", "tokens_seen", "response_tokens_seen", "val_loss")
    if (completion.get("format") != "warpstate-dpo-completion-v1" or completion.get("completed") is not True
            or completion.get("paused_for_evaluation") is not True
            or any(completion.get(k) != checkpoint[k] for k in counters)
            or completion.get("reference_sha256") != sig["reference_sha256"]):
        raise ValueError("DPO completion report differs from its checkpoint")
    scores = ("val_loss", "reward_margin", "reward_accuracy", "chosen_nll")
    if (evaluation.get("stage") != "dpo" or evaluation.get("step") != want["step"] or evaluation.get("full_holdout") is not True
            or evaluation.get("evaluated_samples") != val["rows"]
            or evaluation.get("available_validation_samples") != val["rows"]
            or evaluation.get("objective") != settings["objective"]
            or any(evaluation.get(k) != checkpoint["validation"].get(k) for k in (*scores, "evaluated_samples"))
            or any(evaluation.get(k) != sig[k] for k in ("base_sha256", "data_sha256", "tokenizer_sha256", "reference_sha256"))
            or not all(math.isfinite(evaluation.get(k, float("nan"))) for k in scores)):
        raise ValueError("DPO final full-holdout evaluation differs from its checkpoint")
    if not 0 <= evaluation["reward_accuracy"] <= 1 or evaluation["chosen_nll"] < 0:
        raise ValueError("DPO evaluation contains impossible accuracy/NLL")
    ident = reference.get("identity", {})
    if (reference.get("format") != "warpstate-dpo-reference-v1" or reference.get("complete") is not True
            or reference.get("identity_sha256") != identity_digest(ident) or ident.get("weights_sha256") != sig["base_sha256"]
            or ident.get("data_sha256") != sig["data_sha256"] or ident.get("tokenizer_sha256") != sig["tokenizer_sha256"]
            or ident.get("world_size") != world
            or any(v != settings.get(k) for k, v in ident.get("settings", {}).items())):
        raise ValueError("DPO fixed-reference identity differs from its final checkpoint")
    return want


def verify_dpo_archive(folder, *, expected_checkpoint_hash: str | None = None):
    """Full verification of a sealed DPO archive.  Returns (snapshot metadata, checksum entries)."""
    folder = Path(folder)
    if folder.is_symlink() or not folder.is_dir():
        raise ValueError(f"Archive is not a regular directory: {folder}")
    entries = A.read_checksums(folder, FILES)
    if stat.S_IMODE(folder.stat().st_mode) & 0o222 or {p.name for p in folder.iterdir()} != set(FILES) | {"SHA256SUMS"}:
        raise ValueError("DPO archive directory is not sealed or contains unexpected files")
    for name in (*FILES, "SHA256SUMS"):
        path = folder / name
        if path.is_symlink() or not path.is_file() or stat.S_IMODE(path.stat().st_mode) & 0o222:
            raise ValueError(f"Archive file missing, not regular or writable: {name}")
        if name in entries and digest(path) != entries[name]:
            raise ValueError(f"Archive checksum mismatch: {name}")
    if expected_checkpoint_hash and entries["checkpoint.pt"] != expected_checkpoint_hash:
        raise ValueError("Archived DPO state differs from the source checkpoint")
    checkpoint = torch.load(folder / "checkpoint.pt", map_location="cpu", weights_only=False, mmap=True)
    plan, data, reference = (read_json(folder / n) for n in ("plan.json", "data-manifest.json", "reference-manifest.json"))
    validate_state(checkpoint, read_json(folder / "evaluation.json"), read_json(folder / "completion.json"),
                   read_json(folder / "settings.json"), data, reference, plan)
    sig = checkpoint["signature"]
    if (entries["data-manifest.json"] != sig["data_sha256"] or entries["reference-manifest.json"] != sig["reference_sha256"]
            or entries["tokenizer.model"] != sig["tokenizer_sha256"]):
        raise ValueError("Archived data/reference/tokenizer hashes differ from checkpoint signatures")
    for split in ("train", "val"):
        info = reference["files"][f"{split}.npy"]
        rows = data["outputs"][f"dpo_{split}.jsonl"]["rows"]
        values = np.load(folder / f"reference-{split}.npy", allow_pickle=False, mmap_mode="r")
        if (entries[f"reference-{split}.npy"] != info["sha256"] or info["rows"] != rows or values.shape != (rows, 2)
                or values.dtype != np.float64 or not np.isfinite(values).all() or not (values <= 0).all()):
            raise ValueError("Archived fixed-reference score array differs")
    metadata = read_json(folder / "snapshot.json")
    if (metadata.get("format") != "warpstate-chat-v1" or metadata.get("stage") != "dpo"
            or any(metadata.get(k) != checkpoint[k] for k in ("step", "tokens_seen", "val_loss"))
            or metadata.get("tokenizer_sha256") != entries["tokenizer.model"]
            or metadata.get("snapshot_sha256") != entries["model.pt"]
            or metadata.get("snapshot_bytes") != (folder / "model.pt").stat().st_size
            or metadata.get("source", {}).get("sha256") != entries["checkpoint.pt"]):
        raise ValueError("DPO model export metadata differs from the full archive")
    exported = torch.load(folder / "model.pt", map_location="cpu", weights_only=False, mmap=True)
    if exported.get("inference_only") is not True or exported.get("config") != checkpoint["config"]:
        raise ValueError("DPO exported model is not an inference snapshot of this run")
    A.tensors_equal(checkpoint["model"], exported["model"])
    return metadata, entries


NOTE = """# KEEP: completed DPO run

Created: {created}
DPO step: {step} (validation loss {val_loss})
Source checkpoint: {source}
Source SHA-256: {sha}

`checkpoint.pt` is the complete training state (FP32 model, Adam moments, per-rank RNG);
`model.pt` is a tensor-exact inference export.  Every file is listed in `SHA256SUMS`.
Do not modify; copy to continue training or to chat.
"""


def archive_dpo(run_dir, data_dir, cache_dir, tokenizer, plan_path, destination, revision: str = "") -> dict:
    """Build and publish the sealed archive of a finished DPO run.  The caller holds the locks that
    exclude training; nothing under ``run_dir`` is modified.  Idempotent."""
    run_dir, data_dir, cache_dir, tokenizer, destination = map(Path, (run_dir, data_dir, cache_dir, tokenizer, destination))
    source = run_dir / "latest.pt"
    if source.is_symlink():
        raise ValueError("The checkpoint must not be a symlink")
    if destination.exists() or destination.is_symlink():
        return verify_dpo_archive(destination, expected_checkpoint_hash=digest(source))[0]
    before = source.stat()
    checkpoint = torch.load(source, map_location="cpu", weights_only=False, mmap=True)
    plan = read_json(plan_path)
    validate_state(checkpoint, read_json(run_dir / "evaluation.json"), read_json(run_dir / "completion.json"),
                   read_json(run_dir / "settings.json"), read_json(data_dir / "manifest.json"),
                   read_json(cache_dir / "manifest.json"), plan)
    full_hash = digest(source)
    destination.parent.mkdir(parents=True, exist_ok=True)
    staging = Path(tempfile.mkdtemp(prefix=".dpo-final-", dir=destination.parent))
    export_chat_snapshot(checkpoint, staging, tokenizer, {"path": str(source), "sha256": full_hash}, stage="dpo")
    A.copy_regular(source, staging / "checkpoint.pt")
    A.copy_regular(tokenizer, staging / "tokenizer.model")
    A.copy_regular(Path(plan_path), staging / "plan.json")
    for name in REPORTS:
        A.copy_regular(run_dir / name, staging / name)
    A.copy_regular(data_dir / "manifest.json", staging / "data-manifest.json")
    A.copy_regular(cache_dir / "manifest.json", staging / "reference-manifest.json")
    for split in ("train", "val"):
        A.copy_regular(cache_dir / f"{split}.npy", staging / f"reference-{split}.npy")
    A.write_new(staging / "PROVENANCE.json", json.dumps(dict(
        created_utc=utc_timestamp(), revision=revision, source=str(source), source_sha256=full_hash,
        torch_version=torch.__version__, python=sys.version.split()[0], signature=checkpoint["signature"]),
        indent=2, default=str) + "\n")
    A.write_new(staging / "ARCHIVE.md", NOTE.format(created=utc_timestamp(), step=checkpoint["step"],
                                                    val_loss=checkpoint["val_loss"], source=source, sha=full_hash))
    after = source.stat()
    if (before.st_ino, before.st_size, before.st_mtime_ns) != (after.st_ino, after.st_size, after.st_mtime_ns):
        raise RuntimeError("Checkpoint changed while it was being archived")
    A.seal(staging, FILES)
    metadata, _ = verify_dpo_archive(staging, expected_checkpoint_hash=full_hash)
    A.publish_directory(staging, destination)
    return metadata


def chat_copy(archive, destination) -> Path:
    """Verified, sealed, physically independent copy of the archive's inference files."""
    archive, destination = Path(archive), Path(destination)
    metadata, entries = verify_dpo_archive(archive)
    if not destination.exists():
        destination.parent.mkdir(parents=True, exist_ok=True)
        staging = Path(tempfile.mkdtemp(prefix=".chat-", dir=destination.parent))
        for name in CHAT_FILES:
            A.copy_regular(archive / name, staging / name)
        A.seal(staging, CHAT_FILES)
        A.publish_directory(staging, destination)
    copied = A.read_checksums(destination, CHAT_FILES)
    for name in CHAT_FILES:
        if copied[name] != entries[name] or digest(destination / name) != entries[name]:
            raise ValueError(f"Chat copy differs from its archive: {name}")
        a, b = (archive / name).stat(), (destination / name).stat()
        if (a.st_dev, a.st_ino) == (b.st_dev, b.st_ino):
            raise ValueError(f"Chat copy must not hardlink its archive: {name}")
    return destination / "model.pt"


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--config", type=Path, help="DPO plan (with a handoff section naming work/data directories)")
    p.add_argument("--destination", type=Path)
    p.add_argument("--archive", type=Path)
    p.add_argument("--chat-copy", type=Path)
    p.add_argument("--verify-only", action="store_true")
    p.add_argument("--revision", default="")
    a = p.parse_args(argv)
    if a.chat_copy is not None:
        model = chat_copy(a.archive, a.chat_copy)
        print(json.dumps({"snapshot": str(model), "archive": str(a.archive), "independent_copy": True}, indent=2))
        return 0
    workspace = Path(os.environ.get("WARPSTATE_WORKSPACE", "/workspace/WarpState"))
    plan = read_json(a.config)
    handoff = plan["handoff"]
    work = workspace / handoff["work_dir"]
    destination = a.destination or (workspace / handoff.get("final_archive_dir", f"{handoff['work_dir']}-final-archive"))
    if a.verify_only:
        metadata, _ = verify_dpo_archive(destination)
    else:
        from ..utils.io import process_lock
        with process_lock(work / "control/launcher.lock"), process_lock(workspace / "pipeline.lock", shared=True):
            metadata = archive_dpo(work / "run", workspace / handoff["data_dir"], work / "reference-cache",
                                   workspace / handoff["tokenizer"], a.config, destination, a.revision)
    print(json.dumps({"archive": str(destination), "step": metadata["step"], "model_sha256": metadata["snapshot_sha256"]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
