"""Endpoint agent of the artifact transfer tool: stdlib only, self-contained.

The text of this file is what the transfer client executes at the far end of an SSH connection
(``python3 -c <this file> <action> ...``), so it imports nothing from the package.  Actions:

    manifest  PATH CHUNK                     -> {"manifest": {...}, "identity": [...]}
    identity  PATH IDENTITY_JSON             -> {"identity": [...]}   (fails if the file changed)
    read      PATH IDENTITY_JSON OFF LEN     -> raw bytes on stdout
    prepare   DEST SHA   (manifest on stdin) -> {"complete": bool, "completed": [chunk indices]}
    write     DEST SHA INDEX (bytes on stdin)-> {"index": i, "sha256": ..., "bytes": n}
    finalize  DEST SHA                       -> {"complete": true, ...}

A receiver keeps three sidecars next to DEST: ``.uploading`` (sparse file of the final size),
``.upload-state.json`` (the manifest the partial file belongs to) and ``.upload-chunks/`` (one
receipt per verified chunk).  ``prepare`` re-hashes every receipted chunk and drops receipts that
no longer match; ``finalize`` hashes the whole file and publishes it with
``renameat2(RENAME_NOREPLACE)``, so a destination is never replaced.  Paths must lie below
``$WARPSTATE_WORKSPACE`` (default ``/workspace/WarpState``) with no symlink on the way
(reference ops/transfer_artifacts.py:43-366).
"""
import ctypes
import fcntl
import hashlib
import json
import os
import stat
import sys
import uuid
from pathlib import Path

BLOCK = 1 << 20


def root() -> Path:
    return Path(os.environ.get("WARPSTATE_WORKSPACE", "/workspace/WarpState")).resolve()


def confined(value) -> Path:
    """Absolute path below the workspace root with no symlink in any component."""
    path = Path(os.path.abspath(value))
    base = root()
    if path == base or not path.is_relative_to(base):
        raise ValueError(f"Path must be below {base}: {path}")
    current = base
    for part in path.relative_to(base).parts:
        current = current / part
        if current.is_symlink():
            raise ValueError(f"Symlink is not allowed: {current}")
    return path


def open_regular(path, flags, mode=0o600) -> int:
    fd = os.open(confined(path), flags | os.O_NOFOLLOW, mode)
    if not stat.S_ISREG(os.fstat(fd).st_mode):
        os.close(fd)
        raise ValueError(f"Not a regular file: {path}")
    return fd


def sync_dir(path) -> None:
    fd = os.open(path, os.O_DIRECTORY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def write_json(path: Path, value) -> None:
    temporary = confined(f"{path}.{uuid.uuid4().hex}.tmp")
    fd = open_regular(temporary, os.O_WRONLY | os.O_CREAT | os.O_EXCL)
    try:
        with os.fdopen(fd, "w") as stream:
            stream.write(json.dumps(value, sort_keys=True) + "\n")
            stream.flush()
            os.fsync(stream.fileno())
        os.replace(temporary, path)
        sync_dir(path.parent)
    finally:
        if temporary.exists():
            temporary.unlink()


def read_json(path):
    with os.fdopen(open_regular(path, os.O_RDONLY), "r") as stream:
        return json.load(stream)


def sha_range(path, offset=0, count=None) -> str:
    h = hashlib.sha256()
    with os.fdopen(open_regular(path, os.O_RDONLY), "rb") as stream:
        stream.seek(offset)
        while count is None or count > 0:
            data = stream.read(BLOCK if count is None else min(BLOCK, count))
            if not data:
                if count:
                    raise ValueError("Unexpected end of file during verification")
                break
            h.update(data)
            if count is not None:
                count -= len(data)
    return h.hexdigest()


def file_identity(info) -> list:
    if not stat.S_ISREG(info.st_mode):
        raise ValueError("Source is not a regular file")
    return [info.st_dev, info.st_ino, info.st_size, info.st_mtime_ns, info.st_ctime_ns]


def chunk_manifest(stream, chunk_size: int) -> dict:
    whole, chunks, size = hashlib.sha256(), [], 0
    while True:
        part, used = hashlib.sha256(), 0
        while used < chunk_size:
            data = stream.read(min(BLOCK, chunk_size - used))
            if not data:
                break
            whole.update(data)
            part.update(data)
            used += len(data)
        if not used:
            break
        chunks.append(part.hexdigest())
        size += used
    return {"version": 1, "size": size, "sha256": whole.hexdigest(), "chunk_size": chunk_size, "chunk_sha256": chunks}


# ------------------------------------------------------------------------------------ source side
def source_action(action: str, argv: list) -> None:
    path = confined(argv[0])
    with os.fdopen(os.open(path, os.O_RDONLY | os.O_NOFOLLOW), "rb") as stream:
        before = file_identity(os.fstat(stream.fileno()))

        def unchanged():
            if file_identity(os.fstat(stream.fileno())) != before or file_identity(os.stat(path, follow_symlinks=False)) != before:
                raise ValueError("Source changed during transfer")

        if action == "manifest":
            chunk = int(argv[1])
            if chunk < 1:
                raise ValueError("Chunk size must be positive")
            manifest = chunk_manifest(stream, chunk)
            unchanged()
            print(json.dumps({"manifest": manifest, "identity": before}))
            return
        if before != json.loads(argv[1]):
            raise ValueError("Source changed during transfer")
        if action == "identity":
            unchanged()
            print(json.dumps({"identity": before}))
            return
        offset, remaining = int(argv[2]), int(argv[3])
        if offset < 0 or remaining < 0 or offset + remaining > before[2]:
            raise ValueError("Invalid source chunk range")
        stream.seek(offset)
        while remaining:
            data = stream.read(min(BLOCK, remaining))
            if not data:
                raise ValueError("Source ended early")
            sys.stdout.buffer.write(data)
            remaining -= len(data)
        sys.stdout.buffer.flush()
        unchanged()


# ---------------------------------------------------------------------------------- receiver side
def chunk_extent(state: dict, index: int):
    offset = index * state["chunk_size"]
    return offset, min(state["chunk_size"], state["size"] - offset)


def receiver_action(action: str, argv: list) -> None:
    target, expected = confined(argv[0]), argv[1]
    target.parent.mkdir(parents=True, exist_ok=True)
    confined(target.parent)
    partial = confined(f"{target}.uploading")
    state_path = confined(f"{target}.upload-state.json")
    receipts = confined(f"{target}.upload-chunks")
    lock = open_regular(f"{target}.upload.lock", os.O_RDWR | os.O_CREAT)
    fcntl.flock(lock, fcntl.LOCK_SH if action == "write" else fcntl.LOCK_EX)

    def already_published(size: int) -> bool:
        if not target.exists():
            return False
        if target.stat().st_size != size or sha_range(target) != expected:
            raise ValueError(f"Existing destination differs; refusing overwrite: {target}")
        return True

    if action == "prepare":
        incoming = json.load(sys.stdin)
        if incoming["sha256"] != expected:
            raise ValueError("Source identity mismatch")
        if already_published(incoming["size"]):
            print(json.dumps({"complete": True, "sha256": expected}))
            return
        if state_path.exists():
            state = read_json(state_path)
            if state != incoming:
                raise ValueError("Partial upload belongs to a different source or chunk size")
        else:
            if partial.exists() or receipts.exists():
                raise ValueError("Unclaimed upload sidecar exists; refusing to replace it")
            write_json(state_path, incoming)  # identity first: an interruption here can resume
            state = incoming
        if not partial.exists():
            fd = open_regular(partial, os.O_WRONLY | os.O_CREAT | os.O_EXCL)
            try:
                os.ftruncate(fd, state["size"])
                os.fsync(fd)
            finally:
                os.close(fd)
        if partial.stat().st_size != state["size"]:
            raise ValueError("Partial upload has an unexpected size")
        receipts.mkdir(exist_ok=True)
        done = []
        for index, want in enumerate(state["chunk_sha256"]):
            receipt = confined(receipts / f"{index:08d}.json")
            if not receipt.exists():
                continue
            offset, length = chunk_extent(state, index)
            try:
                good = read_json(receipt) == {"sha256": want, "size": length} and sha_range(partial, offset, length) == want
            except (ValueError, OSError):
                good = False
            if good:
                done.append(index)
            else:
                receipt.unlink()
        sync_dir(receipts)
        print(json.dumps({"complete": False, "completed": done}))
        return

    state = read_json(state_path)
    if state["sha256"] != expected:
        raise ValueError("Upload source identity mismatch")
    if action == "write":
        index = int(argv[2])
        if not 0 <= index < len(state["chunk_sha256"]):
            raise ValueError("Invalid chunk index")
        offset, length = chunk_extent(state, index)
        h = hashlib.sha256()
        fd = open_regular(partial, os.O_WRONLY)
        try:
            remaining, position = length, offset
            while remaining:
                data = sys.stdin.buffer.read(min(BLOCK, remaining))
                if not data:
                    raise ValueError("Upload stream ended early")
                h.update(data)
                view = memoryview(data)
                while view:
                    wrote = os.pwrite(fd, view, position)
                    if wrote <= 0:
                        raise OSError("pwrite made no progress")
                    view = view[wrote:]
                    position += wrote
                remaining -= len(data)
            if sys.stdin.buffer.read(1):
                raise ValueError("Upload stream exceeded its chunk length")
            if h.hexdigest() != state["chunk_sha256"][index]:
                raise ValueError("Chunk SHA256 mismatch")
            os.fsync(fd)
        finally:
            os.close(fd)
        write_json(confined(receipts / f"{index:08d}.json"), {"sha256": h.hexdigest(), "size": length})
        print(json.dumps({"index": index, "sha256": h.hexdigest(), "bytes": length}))
        return
    if action != "finalize":
        raise ValueError("Unknown receiver action")
    if already_published(state["size"]):
        print(json.dumps({"complete": True, "sha256": expected, "bytes": state["size"]}))
        return
    for index, want in enumerate(state["chunk_sha256"]):
        _, length = chunk_extent(state, index)
        receipt = confined(receipts / f"{index:08d}.json")
        if not receipt.exists() or read_json(receipt) != {"sha256": want, "size": length}:
            raise ValueError(f"Missing or invalid receipt for chunk {index}")
    if partial.stat().st_size != state["size"] or sha_range(partial) != expected:
        raise ValueError("Full destination SHA256 mismatch; partial upload retained")
    libc = ctypes.CDLL(None, use_errno=True)
    libc.renameat2.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint]
    libc.renameat2.restype = ctypes.c_int
    if libc.renameat2(-100, os.fsencode(partial), -100, os.fsencode(target), 1):
        code = ctypes.get_errno()
        raise OSError(code, os.strerror(code), str(target))
    sync_dir(target.parent)
    print(json.dumps({"complete": True, "sha256": expected, "bytes": state["size"]}))


def agent_main(argv: list) -> None:
    action = argv[0]
    if action in ("manifest", "identity", "read"):
        source_action(action, argv[1:])
    elif action in ("prepare", "write", "finalize"):
        receiver_action(action, argv[1:])
    else:
        raise ValueError(f"Unknown action {action}")


if __name__ == "__main__":
    agent_main(sys.argv[1:])
