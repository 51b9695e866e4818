"""Sealed, verifiable model archives and independent copies.

An archive directory holds ``model.pt`` (a ``warpstate-chat-v1`` export), its ``snapshot.json``,
the exact ``tokenizer.model``, a human note ``ARCHIVE.md`` and ``SHA256SUMS``; every file is
read-only, the directory is published with ``renameat2(RENAME_NOREPLACE)`` so that a partial
archive never appears under its final name, and copies are physical byte copies (never
hardlinks), so that training that starts from a copy cannot touch the archive (reference
ops/posttrain_handoff.py:61-283, ops/archive_dpo.py).
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
RENAME_NOREPLACE = 1
AT_FDCWD = -100


def publish_directory(staging, destination) -> None:
    """Atomic rename that fails if ``destination`` exists."""
    libc = ctypes.CDLL(None, use_errno=True)
    fn = libc.renameat2
    fn.argtypes = (ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint)
    fn.restype = ctypes.c_int
    if fn(AT_FDCWD, os.fsencode(staging), AT_FDCWD, os.fsencode(destination), RENAME_NOREPLACE):
        code = ctypes.get_errno()
        raise OSError(code, os.strerror(code), str(destination))
    fsync_dir(Path(destination).parent)


def copy_regular(source: Path, destination: Path) -> None:
    """Byte copy into a new read-only file; refuses symlinks and existing targets."""
    if source.is_symlink() or not source.is_file():
        raise ValueError(f"Expected regular source file: {source}")
    with source.open("rb") as reader, destination.open("xb") as writer:
        shutil.copyfileobj(reader, writer, length=8 << 20)
        writer.flush()
        os.fsync(writer.fileno())
    os.chmod(destination, 0o444)


def write_new(path: Path, text: str) -> None:
    with path.open("x") as stream:
        stream.write(text)
        stream.flush()
        os.fsync(stream.fileno())


def seal(folder: Path, files=ARCHIVE_FILES) -> None:
    write_new(folder / "SHA256SUMS", "".join(f"{digest(folder / name)}  {name}\n" for name in files))
    for name in (*files, "SHA256SUMS"):
        os.chmod(folder / name, 0o444)
    os.chmod(folder, 0o555)
    fsync_dir(folder)


def read_checksums(folder: Path, files=ARCHIVE_FILES) -> dict:
    path = folder / "SHA256SUMS"
    if path.is_symlink() or not path.is_file():
        raise ValueError("Archive checksum manifest is missing")
    entries = {}
    for line in path.read_text().splitlines():
        value, name = line.split("  ", 1)
        if name not in files or name in entries:
            raise ValueError("Unexpected or duplicate archive checksum entry")
        entries[name] = value
    if set(entries) != set(files):
        raise ValueError("Archive checksum manifest is incomplete")
    return entries


def verify_archive(folder, boundary: dict, expected_model_hash: str | None = None, *, sealed: bool = True,
                   files=ARCHIVE_FILES) -> dict:
    """Checks structure, permissions, hashes and that the metadata matches the requested
    (step, tokens_seen, tokenizer) boundary.  Returns the snapshot metadata."""
    folder = Path(folder)
    if folder.is_symlink() or not folder.is_dir():
        raise ValueError(f"Archive is not a regular directory: {folder}")
    entries = read_checksums(folder, files)
    for name in (*files, "SHA256SUMS"):
        path = folder / name
        if path.is_symlink() or not path.is_file():
            raise ValueError(f"Archive file missing or not regular: {name}")
        if sealed and stat.S_IMODE(path.stat().st_mode) & 0o222:
            raise ValueError(f"Archive is not sealed read-only: {name}")
        if name in entries and digest(path) != entries[name]:
            raise ValueError(f"Archive checksum mismatch: {name}")
    metadata = json.loads((folder / "snapshot.json").read_text())
    if (metadata.get("format") != "warpstate-chat-v1" or metadata.get("step") != boundary["step"]
            or metadata.get("tokens_seen") != boundary["tokens_seen"]
            or metadata.get("tokenizer_sha256") != boundary["tokenizer_sha256"]):
        raise ValueError("Archive metadata does not match the requested boundary")
    if (metadata.get("snapshot_sha256") != entries["model.pt"]
            or digest(folder / "tokenizer.model") != boundary["tokenizer_sha256"]
            or metadata.get("snapshot_bytes") != (folder / "model.pt").stat().st_size):
        raise ValueError("Archive model/tokenizer metadata mismatch")
    if expected_model_hash and entries["model.pt"] != expected_model_hash:
        raise ValueError("Existing archive differs from its recorded immutable identity")
    return metadata


def tensors_equal(original: dict, exported: dict) -> None:
    if original.keys() != exported.keys():
        raise ValueError("Archive model parameter names differ from the raw checkpoint")
    for name, value in original.items():
        other = exported[name]
        if value.dtype != other.dtype or value.shape != other.shape or not torch.equal(value, other):
            raise ValueError(f"Archive changed a raw model tensor: {name}")


def archive_training_checkpoint(source, tokenizer, destination, boundary: dict, note: str, validate) -> dict:
    """Export the model of a training checkpoint into a sealed archive directory.

    ``validate(checkpoint)`` checks the boundary (exact step, final validation present, FP32
    weights, tokenizer identity).  Idempotent: an existing archive is verified instead."""
    from ..serve.chat import capture_latest
    source, tokenizer, destination = Path(source), Path(tokenizer), Path(destination)
    if source.is_symlink():
        raise ValueError("The checkpoint must not be a symlink")
    before = source.stat()
    checkpoint = torch.load(source, map_location="cpu", weights_only=False, mmap=True)
    validate(checkpoint)
    if destination.exists() or destination.is_symlink():
        metadata = verify_archive(destination, boundary)
        exported = torch.load(destination / "model.pt", map_location="cpu", weights_only=False, mmap=True)
        tensors_equal(checkpoint["model"], exported["model"])
        return metadata
    destination.parent.mkdir(parents=True, exist_ok=True)
    staging_root = Path(tempfile.mkdtemp(prefix=".archive-", dir=destination.parent))
    exported_path = capture_latest(source, tokenizer, staging_root)
    staging = exported_path.parent
    exported = torch.load(exported_path, map_location="cpu", weights_only=False, mmap=True)
    tensors_equal(checkpoint["model"], exported["model"])
    full_hash = digest(source)
    after = source.stat()
    if (before.st_dev, before.st_ino, before.st_size, before.st_mtime_ns) != (
            after.st_dev, after.st_ino, after.st_size, after.st_mtime_ns):
        raise RuntimeError("Checkpoint changed while it was being archived")
    copy_regular(tokenizer, staging / "tokenizer.model")
    write_new(staging / "ARCHIVE.md", note.format(created=utc_timestamp(), step=boundary["step"],
                                                  tokens=boundary["tokens_seen"], source=source,
                                                  source_sha256=full_hash,
                                                  val_loss=checkpoint.get("val_loss")))
    seal(staging)
    metadata = verify_archive(staging, boundary)
    publish_directory(staging, destination)
    staging_root.rmdir()
    return metadata


def independent_copy(archive, destination, boundary: dict, model_hash: str) -> Path:
    """A verified physical copy of an archive (the initialisation a training stage reads)."""
    archive, destination = Path(archive), Path(destination)
    verify_archive(archive, boundary, model_hash)
    if not destination.exists() and not destination.is_symlink():
        destination.parent.mkdir(parents=True, exist_ok=True)
        staging = Path(tempfile.mkdtemp(prefix=".initialization-", dir=destination.parent))
        for name in (*ARCHIVE_FILES, "SHA256SUMS"):
            copy_regular(archive / name, staging / name)
        verify_archive(staging, boundary, model_hash)
        fsync_dir(staging)
        publish_directory(staging, destination)
    verify_archive(destination, boundary, model_hash)
    for name in (*ARCHIVE_FILES, "SHA256SUMS"):
        a, b = (archive / name).stat(), (destination / name).stat()
        if (a.st_dev, a.st_ino) == (b.st_dev, b.st_ino):
            raise ValueError(f"Initialization must not hardlink its archive: {name}")
    return destination / "model.pt"
