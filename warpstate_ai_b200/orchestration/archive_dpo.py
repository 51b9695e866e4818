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
from ..utils.io import digest, process_lock, utc_timestamp
from ..utils.rules import Rule, enforce, finite, fp32_tensors, matches
from . import archive as A

REPORTS = ("settings.json", "evaluation.json", "completion.json", "metrics.jsonl")
# What the hand-off guardian recorded about this run (`orchestration/handoff.py`), under the run's work directory.
GUARDIAN_RECORDS = {"dpo-execution.json": "control/execution.json", "dpo-handoff.json": "control/handoff.json",
                    "gpu-preflight.json": "preflight/report.json"}
# archive file name <- where it comes from: (root, leaf) with root one of run / work / data / cache / tokenizer / plan
COPIED = {"checkpoint.pt": ("run", "latest.pt"), "tokenizer.model": ("tokenizer", ""), "plan.json": ("plan", ""),
          **{name: ("run", name) for name in REPORTS}, **{name: ("work", leaf) for name, leaf in GUARDIAN_RECORDS.items()},
          "data-manifest.json": ("data", "manifest.json"), "reference-manifest.json": ("cache", "manifest.json"),
          "reference-train.npy": ("cache", "train.npy"), "reference-val.npy": ("cache", "val.npy")}
# the reference's archive layout (reference ops/archive_dpo.py:35-39)
FILES = ("checkpoint.pt", "model.pt", "snapshot.json", "tokenizer.model", "plan.json", *REPORTS, *GUARDIAN_RECORDS,
         "data-manifest.json", "reference-manifest.json", "reference-train.npy", "reference-val.npy", "PROVENANCE.json",
         "ARCHIVE.md")
NO_GUARDIAN = {"recorded": False, "reason": "this run was not started by a hand-off guardian; nothing was recorded here"}
CHAT_FILES = ("model.pt", "snapshot.json", "tokenizer.model", "ARCHIVE.md")
SCORES = ("val_loss", "reward_margin", "reward_accuracy", "chosen_nll")
IDENTITIES = ("base_sha256", "data_sha256", "tokenizer_sha256", "reference_sha256")


def read_json(path):
    with open(path, encoding="utf-8") as handle:
        return json.load(handle)


def load_tensors(path):
    return torch.load(path, map_location="cpu", weights_only=False, mmap=True)


def expected_counters(plan: dict, data: dict) -> dict:
    """Where a whole run over the prepared pairs must end, from the plan and the data manifest alone."""
    settings, ranks = DEFAULTS | plan["training"], plan["handoff"]["processes"]
    if settings["max_steps"] is not None:
        raise ValueError("Archive requires a completed whole DPO run, without a plan step cap")
    pairs, epochs = data["outputs"]["dpo_train.jsonl"], settings["epochs"]
    per_update = settings["micro_batch"] * settings["grad_accum"] * ranks
    updates = epochs * -(-pairs["rows"] // per_update)
    return {"step": updates, "total_steps": updates, "val_step": updates, "sample_cursor": epochs * pairs["rows"],
            "tokens_seen": epochs * (pairs["tokens"] - 2 * pairs["rows"]),       # each branch loses its shifted token
            "response_tokens_seen": epochs * pairs["supervised_tokens"]}


def validate_state(checkpoint, evaluation, completion, settings_report, data, reference, plan) -> dict:
    """Consistency of a finished DPO run, judged from its preserved records only.  Returns the expected counters."""
    settings, ranks = DEFAULTS | plan["training"], plan["handoff"]["processes"]
    train_rows, val_rows = (data["outputs"][f"dpo_{split}.jsonl"]["rows"] for split in ("train", "val"))
    want = expected_counters(plan, data)
    signature = checkpoint.get("signature") or {}
    origin, ancestor = checkpoint.get("origin") or {}, plan.get("sft")
    moments = (checkpoint.get("optimizer") or {}).get("state") or {}
    identity = reference.get("identity") or {}
    enforce([
        Rule("DPO checkpoint is not the fully completed, finally evaluated state",
             lambda: matches(checkpoint, {"format": "warpstate-dpo-v1", "completed": True, **want}) and finite(checkpoint["val_loss"])),
        Rule("DPO checkpoint/settings signatures or dataset counts differ",
             lambda: matches(signature, {"plan": plan, "settings": settings, "world_size": ranks})
             and matches(settings_report, {"signature": signature, "total_steps": want["step"], "train_rows": train_rows,
                                           "val_rows": val_rows})),
        Rule("DPO data provenance differs from its signature",
             lambda: matches(data, {"format": "warpstate-posttrain-data-v1", "complete": True,
                                    "tokenizer_sha256": signature["tokenizer_sha256"],
                                    "max_length": settings["sequence_length"]})),
        Rule("DPO did not start from a sealed SFT export",
             lambda: matches(origin, {"stage": "sft", "weights_sha256": signature["base_sha256"]})),
        Rule("DPO SFT ancestry differs from the authorized plan",
             lambda: ancestor is None or matches(origin, {"step": ancestor["step"], "tokens_seen": ancestor["tokens_seen"]})),
        Rule("DPO optimizer or per-rank RNG state is missing",
             lambda: len(moments) > 0 and len(checkpoint["rng_by_rank"]) == ranks
             and all("torch" in stream for stream in checkpoint["rng_by_rank"])),
        Rule("DPO Adam step differs from the final checkpoint",
             lambda: all(float(entry["step"]) == want["step"] for entry in moments.values())),
        Rule("DPO Adam state must retain its original FP32 tensors",
             lambda: all(entry[key].dtype == torch.float32 for entry in moments.values() for key in ("exp_avg", "exp_avg_sq"))),
        Rule("DPO model tensors are missing", lambda: len(checkpoint["model"]) > 0),
        *fp32_tensors(checkpoint.get("model") or {}, "DPO model tensor is not original FP32: {name}"),
        Rule("DPO completion report differs from its checkpoint",
             lambda: matches(completion, {"format": "warpstate-dpo-completion-v1", "completed": True, "paused_for_evaluation": True,
                                          "reference_sha256": signature["reference_sha256"],
                                          **{key: checkpoint[key] for key in ("step", "total_steps", "sample_cursor", "tokens_seen",
                                                                              "response_tokens_seen", "val_loss")}})),
        Rule("DPO final full-holdout evaluation differs from its checkpoint",
             lambda: matches(evaluation, {"stage": "dpo", "step": want["step"], "full_holdout": True, "evaluated_samples": val_rows,
                                          "available_validation_samples": val_rows, "objective": settings["objective"],
                                          **{key: signature[key] for key in IDENTITIES},
                                          **{key: checkpoint["validation"].get(key) for key in (*SCORES, "evaluated_samples")}})
             and all(finite(evaluation[key]) for key in SCORES)),
        Rule("DPO evaluation contains impossible accuracy/NLL",
             lambda: 0 <= evaluation["reward_accuracy"] <= 1 and evaluation["chosen_nll"] >= 0),
        Rule("DPO fixed-reference identity differs from its final checkpoint",
             lambda: matches(reference, {"format": "warpstate-dpo-reference-v1", "complete": True,
                                         "identity_sha256": identity_digest(identity)})
             and matches(identity, {"weights_sha256": signature["base_sha256"], "data_sha256": signature["data_sha256"],
                                    "tokenizer_sha256": signature["tokenizer_sha256"], "world_size": ranks})
             and matches(settings, identity.get("settings", {}))),
    ])
    return want


def _plain_read_only_file(path: Path) -> bool:
    mode = path.lstat().st_mode if path.exists() or path.is_symlink() else 0
    return stat.S_ISREG(mode) and not stat.S_IMODE(mode) & 0o222


def verify_dpo_archive(folder, *, expected_checkpoint_hash: str | None = None):
    """Full verification of a sealed DPO archive.  Returns (snapshot metadata, checksum entries)."""
    folder = Path(folder)
    if folder.is_symlink() or not folder.is_dir():
        raise ValueError(f"Archive is not a regular directory: {folder}")
    entries = A.read_checksums(folder, FILES)
    members = (*FILES, "SHA256SUMS")
    enforce([Rule("DPO archive directory is not sealed or contains unexpected files",
                  lambda: not stat.S_IMODE(folder.stat().st_mode) & 0o222 and sorted(p.name for p in folder.iterdir()) == sorted(members)),
             *(Rule(f"Archive file missing, not regular or writable: {name}", lambda name=name: _plain_read_only_file(folder / name))
               for name in members),
             *(Rule(f"Archive checksum mismatch: {name}", lambda name=name: digest(folder / name) == entries[name]) for name in FILES),
             Rule("Archived DPO state differs from the source checkpoint",
                  lambda: not expected_checkpoint_hash or entries["checkpoint.pt"] == expected_checkpoint_hash)])
    checkpoint = load_tensors(folder / "checkpoint.pt")
    records = {name: read_json(folder / f"{name}.json") for name in ("plan", "data-manifest", "reference-manifest", "evaluation",
                                                                      "completion", "settings", "snapshot")}
    data, reference, metadata = records["data-manifest"], records["reference-manifest"], records["snapshot"]
    validate_state(checkpoint, records["evaluation"], records["completion"], records["settings"], data, reference, records["plan"])
    signature = checkpoint["signature"]

    def scores_intact(split: str) -> bool:
        listed, rows = reference["files"][f"{split}.npy"], data["outputs"][f"dpo_{split}.jsonl"]["rows"]
        values = np.load(folder / f"reference-{split}.npy", allow_pickle=False, mmap_mode="r")
        return (listed["sha256"] == entries[f"reference-{split}.npy"] and listed["rows"] == rows
                and (values.shape, values.dtype) == ((rows, 2), np.float64)
                and bool(np.isfinite(values).all()) and bool((values <= 0).all()))      # log-probabilities

    exported = load_tensors(folder / "model.pt")
    enforce([Rule("Archived data/reference/tokenizer hashes differ from checkpoint signatures",
                  lambda: (entries["data-manifest.json"], entries["reference-manifest.json"], entries["tokenizer.model"])
                  == (signature["data_sha256"], signature["reference_sha256"], signature["tokenizer_sha256"])),
             *(Rule("Archived fixed-reference score array differs", lambda split=split: scores_intact(split)) for split in ("train", "val")),
             Rule("DPO model export metadata differs from the full archive",
                  lambda: matches(metadata, {"format": "warpstate-chat-v1", "stage": "dpo", "tokenizer_sha256": entries["tokenizer.model"],
                                             "snapshot_sha256": entries["model.pt"],
                                             "snapshot_bytes": (folder / "model.pt").stat().st_size,
                                             **{key: checkpoint[key] for key in ("step", "tokens_seen", "val_loss")}})
                  and metadata["source"]["sha256"] == entries["checkpoint.pt"]),
             Rule("DPO exported model is not an inference snapshot of this run",
                  lambda: exported["inference_only"] is True and exported["config"] == checkpoint["config"])])
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
    roots = {"run": Path(run_dir), "work": Path(run_dir).parent, "data": Path(data_dir), "cache": Path(cache_dir),
             "tokenizer": Path(tokenizer), "plan": Path(plan_path)}
    destination, source = Path(destination), Path(run_dir) / "latest.pt"
    if source.is_symlink():
        raise ValueError("The checkpoint must not be a symlink")
    if destination.exists() or destination.is_symlink():
        return verify_dpo_archive(destination, expected_checkpoint_hash=digest(source))[0]

    def fingerprint():
        seen = source.stat()
        return seen.st_ino, seen.st_size, seen.st_mtime_ns

    first_seen = fingerprint()
    checkpoint = load_tensors(source)
    validate_state(checkpoint, *(read_json(roots["run"] / f"{name}.json") for name in ("evaluation", "completion", "settings")),
                   read_json(roots["data"] / "manifest.json"), read_json(roots["cache"] / "manifest.json"), read_json(plan_path))
    whole = digest(source)
    destination.parent.mkdir(parents=True, exist_ok=True)
    staging = Path(tempfile.mkdtemp(prefix=".dpo-final-", dir=destination.parent))
    export_chat_snapshot(checkpoint, staging, roots["tokenizer"], {"path": str(source), "sha256": whole}, stage="dpo")
    for name, (root, leaf) in COPIED.items():
        origin = roots[root] / leaf if leaf else roots[root]
        if name in GUARDIAN_RECORDS and not origin.exists():
            A.write_new(staging / name, json.dumps(NO_GUARDIAN, indent=2) + "\n")     # same layout, and it says so
        else:
            A.copy_regular(origin, staging / name)
    provenance = {"created_utc": utc_timestamp(), "revision": revision, "source": str(source), "source_sha256": whole,
                  "torch_version": torch.__version__, "python": sys.version.split()[0], "signature": checkpoint["signature"]}
    A.write_new(staging / "PROVENANCE.json", json.dumps(provenance, indent=2, default=str) + "\n")
    A.write_new(staging / "ARCHIVE.md", NOTE.format(created=provenance["created_utc"], step=checkpoint["step"],
                                                    val_loss=checkpoint["val_loss"], source=source, sha=whole))
    if fingerprint() != first_seen:
        raise RuntimeError("Checkpoint changed while it was being archived")
    A.seal(staging, FILES)
    metadata, _ = verify_dpo_archive(staging, expected_checkpoint_hash=whole)
    A.publish_directory(staging, destination)
    return metadata


def chat_copy(archive, destination) -> Path:
    """Verified, sealed, physically independent copy of the archive's inference files."""
    archive, destination = Path(archive), Path(destination)
    _, entries = verify_dpo_archive(archive)
    if not destination.exists():
        destination.parent.mkdir(parents=True, exist_ok=True)
        staging = Path(tempfile.mkdtemp(prefix=".chat-", dir=destination.parent))
        for name in CHAT_FILES:
            A.copy_regular(archive / name, staging / name)
        A.seal(staging, CHAT_FILES)
        A.publish_directory(staging, destination)
    listed = A.read_checksums(destination, CHAT_FILES)

    def separate_file(name: str) -> bool:
        original, copy = (archive / name).stat(), (destination / name).stat()
        return (original.st_dev, original.st_ino) != (copy.st_dev, copy.st_ino)

    enforce([*(Rule(f"Chat copy differs from its archive: {name}",
                    lambda name=name: listed[name] == entries[name] == digest(destination / name)) for name in CHAT_FILES),
             *(Rule(f"Chat copy must not hardlink its archive: {name}", lambda name=name: separate_file(name)) for name in CHAT_FILES)])
    return destination / "model.pt"


def guardian_done(root: Path, section: dict, work: Path, program: str) -> None:
    """Where a guardian ran the job (the plan names its supervisor socket), archive only what it has finished with: the
    program exited cleanly and its journal reached ``complete`` (reference ops/archive_dpo.py:273-276)."""
    if "supervisor_socket" not in section:
        return
    from .handoff import clean_exit, process_status
    enforce([Rule("DPO guardian must have exited successfully before archival",
                  lambda: clean_exit(process_status(root / section["supervisor_socket"], program))),
             Rule("DPO guardian has not completed its final integrity checks",
                  lambda: (work / "control/handoff.json").is_file()
                  and read_json(work / "control/handoff.json")["phase"] == "complete")])


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--config", type=Path, help="DPO plan (its handoff section names the work and data directories)")
    parser.add_argument("--destination", type=Path, help="archive directory (default: <work_dir>-final-archive)")
    parser.add_argument("--archive", type=Path, help="with --chat-copy: the sealed archive to copy from")
    parser.add_argument("--chat-copy", type=Path, help="make a sealed chat copy here instead of archiving")
    parser.add_argument("--verify-only", action="store_true")
    parser.add_argument("--revision", default="")
    parser.add_argument("--program", default="warpstate-dpo",
                        help="supervisor program of the DPO guardian: where the plan names a supervisor socket, the archive is "
                             "made only after that program has exited cleanly and recorded phase 'complete'")
    options = parser.parse_args(argv)
    if options.chat_copy is not None:
        model = chat_copy(options.archive, options.chat_copy)
        print(json.dumps({"snapshot": str(model), "archive": str(options.archive), "independent_copy": True}, indent=2))
        return 0
    from .launcher import workspace_root
    root, section = workspace_root(), read_json(options.config)["handoff"]
    work = root / section["work_dir"]
    destination = options.destination or root / section.get("final_archive_dir", section["work_dir"] + "-final-archive")
    if options.verify_only:
        metadata, _ = verify_dpo_archive(destination)
    else:
        with process_lock(work / "control/launcher.lock"), process_lock(root / "pipeline.lock", shared=True):
            guardian_done(root, section, work, options.program)
            metadata = archive_dpo(work / "run", root / section["data_dir"], work / "reference-cache", root / section["tokenizer"],
                                   options.config, destination, options.revision)
    print(json.dumps({"archive": str(destination), "step": metadata["step"], "model_sha256": metadata["snapshot_sha256"]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
