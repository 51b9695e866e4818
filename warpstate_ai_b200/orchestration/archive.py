"""Sealed, verifiable model archives and independent copies of them.

An archive is a directory with ``model.pt`` (a ``warpstate-chat-v1`` export), its ``snapshot.json``, the exact
``tokenizer.model``, a human note ``ARCHIVE.md`` and ``SHA256SUMS``.  The properties that matter (the
reference's hand-off scripts establish them, reference ops/posttrain_handoff.py:61-283, ops/archive_dpo.py):

* a partial archive never appears under its final name -- it is assembled in a staging directory and
  published with ``renameat2(RENAME_NOREPLACE)``, which also refuses to replace an existing archive;
* everything in it is read-only, and `verify` re-checks structure, permissions, every hash and that the
  metadata names the expected training boundary (step, tokens seen, tokenizer);
* what a later stage trains from is a *physical* copy (never a hard link), so no training run can alter
  the archive.

The archive of a finished SFT run holds more (`SFT_ARCHIVE_FILES`, reference ops/dpo_handoff.py:34-37): the
byte-identical final checkpoint with its optimizer and RNG state, the run's reports and the guardian's records; the
DPO stage copies only `INIT_FILES` out of it.

`SealedDirectory` is one such directory with its list of files; the module functions are its verbs under the names
the hand-off code uses.
"""
from __future__ import annotations

import ctypes
import json
import os
import shutil
import stat
import tempfile
from pathlib import Path

import torch

from ..utils.io import digest, fsync_dir, utc_timestamp

ARCHIVE_FILES = ("model.pt", "snapshot.json", "tokenizer.model", "ARCHIVE.md")
# A finished SFT run is archived whole (reference ops/dpo_handoff.py:34-37): the byte-identical checkpoint with its
# optimizer and RNG state, the model-only export, the run's reports and what the guardian recorded about it.
SFT_ARCHIVE_FILES = ("checkpoint.pt", "model.pt", "snapshot.json", "tokenizer.model", "settings.json", "evaluation.json",
                     "completion.json", "metrics.jsonl", "sft-execution.json", "sft-handoff.json", "PROVENANCE.json",
                     "ARCHIVE.md")
# What a later stage needs of an archive to start from it.
INIT_FILES = ("model.pt", "snapshot.json", "tokenizer.model")
SUMS = "SHA256SUMS"


def publish_directory(staging, destination) -> None:
    """Rename ``staging`` to ``destination`` atomically; fails (OSError) when the destination exists."""
    rename = ctypes.CDLL(None, use_errno=True).renameat2
    rename.restype = ctypes.c_int
    rename.argtypes = (ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint)
    here, no_replace = -100, 1            # AT_FDCWD, RENAME_NOREPLACE
    if rename(here, os.fsencode(staging), here, os.fsencode(destination), no_replace) != 0:
        number = ctypes.get_errno()
        raise OSError(number, os.strerror(number), str(destination))
    fsync_dir(Path(destination).parent)


def _regular(path: Path) -> bool:
    return path.is_file() and not path.is_symlink()


def copy_regular(source: Path, destination: Path) -> None:
    """Byte copy into a new read-only file; symlinks and existing targets are refused."""
    if not _regular(source):
        raise ValueError(f"{source} is not a regular file")
    with source.open("rb") as src, destination.open("xb") as dst:
        shutil.copyfileobj(src, dst, length=8 << 20)
        dst.flush()
        os.fsync(dst.fileno())
    os.chmod(destination, 0o444)


def write_new(path: Path, text: str) -> None:
    with path.open("x") as out:
        out.write(text)
        out.flush()
        os.fsync(out.fileno())


def _identity(st) -> tuple:
    return st.st_dev, st.st_ino, st.st_size, st.st_mtime_ns


class SealedDirectory:
    def __init__(self, folder, files=ARCHIVE_FILES):
        self.folder, self.files = Path(folder), tuple(files)

    def path(self, name: str) -> Path:
        return self.folder / name

    # ------------------------------------------------------------------ sealing
    def seal(self) -> None:
        """Write ``SHA256SUMS`` over the archive's files and make everything read-only."""
        lines = [f"{digest(self.path(name))}  {name}\n" for name in self.files]
        write_new(self.path(SUMS), "".join(lines))
        for name in (*self.files, SUMS):
            os.chmod(self.path(name), 0o444)
        os.chmod(self.folder, 0o555)
        fsync_dir(self.folder)

    def checksums(self) -> dict:
        """``{file name: recorded SHA-256}``; raises unless exactly the archive's files are listed once."""
        listing = self.path(SUMS)
        if not _regular(listing):
            raise ValueError(f"{self.folder} has no {SUMS}")
        recorded: dict[str, str] = {}
        for line in listing.read_text().splitlines():
            value, _, name = line.partition("  ")
            if name not in self.files or name in recorded:
                raise ValueError(f"{SUMS} lists an unexpected or repeated file: {name!r}")
            recorded[name] = value
        if len(recorded) != len(self.files):
            raise ValueError(f"{SUMS} does not list every file of the archive")
        return recorded

    # ------------------------------------------------------------------ verification
    def verify(self, boundary: dict, expected_model_hash: str | None = None, sealed: bool = True) -> dict:
        """Structure, permissions, hashes, and metadata against ``boundary`` (step, tokens_seen,
        tokenizer_sha256).  Returns the snapshot metadata."""
        if self.folder.is_symlink() or not self.folder.is_dir():
            raise ValueError(f"{self.folder} is not a plain directory")
        recorded = self.checksums()
        for name in (*self.files, SUMS):
            item = self.path(name)
            if not _regular(item):
                raise ValueError(f"archive file {name} is missing or not a regular file")
            if sealed and stat.S_IMODE(item.stat().st_mode) & 0o222:
                raise ValueError(f"archive file {name} is writable: the archive was not sealed")
            if name != SUMS and digest(item) != recorded[name]:
                raise ValueError(f"checksum mismatch: {name}")
        metadata = json.loads(self.path("snapshot.json").read_text())
        wanted = {"format": "warpstate-chat-v1", "step": boundary["step"], "tokens_seen": boundary["tokens_seen"],
                  "tokenizer_sha256": boundary["tokenizer_sha256"]}
        if any(metadata.get(key) != value for key, value in wanted.items()):
            raise ValueError(f"{self.folder} was not made at the requested boundary (step, tokens or tokenizer differ)")
        consistent = (metadata.get("snapshot_sha256") == recorded["model.pt"]
                      and metadata.get("snapshot_bytes") == self.path("model.pt").stat().st_size
                      and digest(self.path("tokenizer.model")) == boundary["tokenizer_sha256"])
        if not consistent:
            raise ValueError("the archive's metadata does not describe its model file and tokenizer")
        if expected_model_hash is not None and recorded["model.pt"] != expected_model_hash:
            raise ValueError("the archive is not the one recorded earlier (its model hash changed)")
        return metadata

    # ------------------------------------------------------------------ copies
    def copy_to(self, destination, boundary: dict, model_hash: str, only=None) -> Path:
        """A verified physical copy at ``destination`` (created if absent); returns the copy's ``model.pt``.
        ``only`` names the files to take (a sealed directory of its own, with its own checksum list); by default the
        whole archive is copied, checksum list included."""
        destination = Path(destination)
        self.verify(boundary, model_hash)
        kept = self.files if only is None else tuple(only)
        names = (*kept, SUMS) if only is None else kept
        if not destination.exists() and not destination.is_symlink():
            destination.parent.mkdir(parents=True, exist_ok=True)
            staging = SealedDirectory(tempfile.mkdtemp(prefix=".initialization-", dir=destination.parent), kept)
            for name in names:
                copy_regular(self.path(name), staging.path(name))
            if only is not None:
                staging.seal()
            staging.verify(boundary, model_hash)
            fsync_dir(staging.folder)
            publish_directory(staging.folder, destination)
        copy = SealedDirectory(destination, kept)
        copy.verify(boundary, model_hash)
        for name in names:
            mine, theirs = self.path(name).stat(), copy.path(name).stat()
            if (mine.st_dev, mine.st_ino) == (theirs.st_dev, theirs.st_ino):
                raise ValueError(f"{name} in {destination} is a hard link into the archive, not a copy")
        return copy.path("model.pt")


# ----------------------------------------------------------------------------------- functional forms
def seal(folder: Path, files=ARCHIVE_FILES) -> None:
    SealedDirectory(folder, files).seal()


def read_checksums(folder: Path, files=ARCHIVE_FILES) -> dict:
    return SealedDirectory(folder, files).checksums()


def verify_archive(folder, boundary: dict, expected_model_hash: str | None = None, *, sealed: bool = True,
                   files=ARCHIVE_FILES) -> dict:
    return SealedDirectory(folder, files).verify(boundary, expected_model_hash, sealed)


def independent_copy(archive, destination, boundary: dict, model_hash: str, *, files=ARCHIVE_FILES, only=None) -> Path:
    return SealedDirectory(archive, files).copy_to(destination, boundary, model_hash, only)


def tensors_equal(original: dict, exported: dict) -> None:
    """Raises unless the two state dicts hold the same names, dtypes, shapes and bits."""
    if set(original) != set(exported):
        raise ValueError("the export's parameter names differ from the checkpoint's")
    for name, tensor in original.items():
        twin = exported[name]
        if (tensor.dtype, tensor.shape) != (twin.dtype, twin.shape) or not torch.equal(tensor, twin):
            raise ValueError(f"the export changed tensor {name}")


def _load(path):
    return torch.load(path, map_location="cpu", weights_only=False, mmap=True)


def archive_training_checkpoint(source, tokenizer, destination, boundary: dict, note: str, validate) -> dict:
    """Seal the model of a training checkpoint into an archive at ``destination``.

    ``validate(checkpoint)`` checks the boundary (exact step, final validation present, FP32 weights,
    tokenizer identity).  When the archive already exists it is verified, tensor by tensor, instead."""
    from ..serve.snapshots import SnapshotStore
    source, tokenizer, destination = Path(source), Path(tokenizer), Path(destination)
    if source.is_symlink():
        raise ValueError(f"{source} is a symlink; archive the checkpoint file itself")
    seen_first = _identity(source.stat())
    checkpoint = _load(source)
    validate(checkpoint)
    if destination.exists() or destination.is_symlink():
        metadata = SealedDirectory(destination).verify(boundary)
        tensors_equal(checkpoint["model"], _load(destination / "model.pt")["model"])
        return metadata
    destination.parent.mkdir(parents=True, exist_ok=True)
    workbench = Path(tempfile.mkdtemp(prefix=".archive-", dir=destination.parent))
    export = SnapshotStore(workbench, tokenizer).export(source)
    staging = SealedDirectory(export.parent)
    tensors_equal(checkpoint["model"], _load(export)["model"])
    source_hash = digest(source)
    if _identity(source.stat()) != seen_first:
        raise RuntimeError(f"{source} changed while it was being archived")
    copy_regular(tokenizer, staging.path("tokenizer.model"))
    write_new(staging.path("ARCHIVE.md"), note.format(
        created=utc_timestamp(), step=boundary["step"], tokens=boundary["tokens_seen"], source=source,
        source_sha256=source_hash, val_loss=checkpoint.get("val_loss")))
    staging.seal()
    metadata = staging.verify(boundary)
    publish_directory(staging.folder, destination)
    workbench.rmdir()
    return metadata
