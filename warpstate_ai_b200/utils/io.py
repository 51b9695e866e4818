"""Small host-side utilities shared by the entry points: hashing, atomic file publication,
advisory process locks (flock), JSON-lines logging.

Lock semantics follow the reference pipeline (run_40b.py:211-224, posttrain.py main): the
pretraining job holds ``pipeline.lock`` exclusively, post-training ranks hold it shared, and a
lock lives as long as the file descriptor -- including in child processes that inherited it -- so
an orphaned worker keeps the next job from starting.
"""
from __future__ import annotations

import contextlib
import fcntl
import hashlib
import json
import os
import time
from pathlib import Path


def digest(path, block: int = 1 << 20) -> str:
    h = hashlib.sha256()
    with Path(path).open("rb") as f:
        while True:
            chunk = f.read(block)
            if not chunk:
                break
            h.update(chunk)
    return h.hexdigest()


def digest_bytes(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def fsync_dir(path: Path) -> None:
    fd = os.open(path, os.O_RDONLY | os.O_DIRECTORY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def atomic_write(path, writer) -> None:
    """``writer(file)`` into a temporary sibling, fsync, rename over ``path``."""
    path = Path(path)
    temporary = path.with_suffix(path.suffix + ".tmp")
    try:
        with temporary.open("wb") as f:
            writer(f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(temporary, path)
        fsync_dir(path.parent)
    except BaseException:
        temporary.unlink(missing_ok=True)
        raise


def atomic_json(path, payload, indent: int | None = 2) -> None:
    atomic_write(path, lambda f: f.write(json.dumps(payload, indent=indent, sort_keys=False).encode("utf-8")))


def append_jsonl(path, record: dict) -> None:
    with Path(path).open("a", encoding="utf-8") as f:
        f.write(json.dumps(record) + "\n")


class LockHeld(RuntimeError):
    pass


@contextlib.contextmanager
def process_lock(path, shared: bool = False, blocking: bool = False):
    """Advisory lock on ``path`` for the life of the context (or of any inheriting child)."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("a+b") as f:
        mode = fcntl.LOCK_SH if shared else fcntl.LOCK_EX
        if not blocking:
            mode |= fcntl.LOCK_NB
        try:
            fcntl.flock(f, mode)
        except BlockingIOError as error:
            raise LockHeld(f"{path} is locked by another process") from error
        # No explicit unlock: closing this descriptor drops the lock only when no other process
        # still holds the same open file description (an inherited descriptor keeps it).
        yield f


def utc_timestamp() -> str:
    return time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
