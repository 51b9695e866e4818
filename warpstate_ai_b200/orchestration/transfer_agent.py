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


# ------------------------------------------------------------------------------------ confinement and file helpers
def root() -> Path:
    return Path(os.environ.get("WARPSTATE_WORKSPACE", "/workspace/WarpState")).resolve()


def confined(value) -> Path:
    """``value`` as an absolute path strictly below the workspace root, with no symlink on the way down."""
    base, path = root(), Path(os.path.abspath(value))
    if base not in path.parents:
        raise ValueError(f"{path} is not below {base}")
    for ancestor in [path, *path.parents]:
        if ancestor == base:
            break
        if ancestor.is_symlink():
            raise ValueError(f"{ancestor} is a symlink; transfers follow none")
    return path


def open_regular(path, flags, mode=0o600) -> int:
    fd = os.open(confined(path), flags | os.O_NOFOLLOW, mode)
    if stat.S_ISREG(os.fstat(fd).st_mode):
        return fd
    os.close(fd)
    raise ValueError(f"{path} is not a regular file")


def sync_dir(path) -> None:
    fd = os.open(path, os.O_DIRECTORY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def write_json(path: Path, value) -> None:
    """Replace ``path`` with ``value`` (sorted keys) through a uniquely named sibling."""
    sibling = confined(f"{path}.{uuid.uuid4().hex}.tmp")
    try:
        with os.fdopen(open_regular(sibling, os.O_WRONLY | os.O_CREAT | os.O_EXCL), "w") as out:
            out.write(json.dumps(value, sort_keys=True) + "\n")
            out.flush()
            os.fsync(out.fileno())
        os.replace(sibling, path)
        sync_dir(path.parent)
    finally:
        if sibling.exists():
            sibling.unlink()


def read_json(path):
    with os.fdopen(open_regular(path, os.O_RDONLY), "r") as source:
        return json.load(source)


def blocks(stream, count=None, exact=True):
    """``count`` bytes of ``stream`` (all of it when None) in pieces of at most BLOCK bytes.  With ``exact`` an
    early end of the stream is an error, otherwise the pieces simply stop."""
    left = count
    while left is None or left > 0:
        piece = stream.read(BLOCK if left is None else min(BLOCK, left))
        if not piece:
            if left and exact:
                raise ValueError("the file ended before the expected number of bytes")
            return
        yield piece
        if left is not None:
            left -= len(piece)


def sha_range(path, offset=0, count=None) -> str:
    digest = hashlib.sha256()
    with os.fdopen(open_regular(path, os.O_RDONLY), "rb") as stream:
        stream.seek(offset)
        for piece in blocks(stream, count):
            digest.update(piece)
    return digest.hexdigest()


def file_identity(info) -> list:
    if not stat.S_ISREG(info.st_mode):
        raise ValueError("the source is not a regular file")
    return [info.st_dev, info.st_ino, info.st_size, info.st_mtime_ns, info.st_ctime_ns]


def chunk_manifest(stream, chunk_size: int) -> dict:
    """Size, whole-file SHA-256 and one SHA-256 per ``chunk_size`` bytes of ``stream``."""
    whole, per_chunk, size = hashlib.sha256(), [], 0
    while True:
        one, got = hashlib.sha256(), 0
        for piece in blocks(stream, chunk_size, exact=False):
            one.update(piece)
            whole.update(piece)
            got += len(piece)
        if got == 0:
            break
        per_chunk.append(one.hexdigest())
        size += got
        if got < chunk_size:
            break
    return {"version": 1, "size": size, "sha256": whole.hexdigest(), "chunk_size": chunk_size, "chunk_sha256": per_chunk}


# ------------------------------------------------------------------------------------ source side
class SourceFile:
    """The file being sent, held open; every action ends by checking that it is still the same file."""

    def __init__(self, path):
        self.path = confined(path)
        self.stream = os.fdopen(os.open(self.path, os.O_RDONLY | os.O_NOFOLLOW), "rb")
        self.identity = file_identity(os.fstat(self.stream.fileno()))

    def require_unchanged(self) -> None:
        now = (file_identity(os.fstat(self.stream.fileno())), file_identity(os.stat(self.path, follow_symlinks=False)))
        if now != (self.identity, self.identity):
            raise ValueError("the source file changed during the transfer")

    def require_identity(self, expected) -> None:
        if self.identity != expected:
            raise ValueError("the source file changed during the transfer")

    def manifest(self, chunk_size: int) -> dict:
        if chunk_size < 1:
            raise ValueError("the chunk size must be at least one byte")
        described = chunk_manifest(self.stream, chunk_size)
        self.require_unchanged()
        return {"manifest": described, "identity": self.identity}

    def send(self, offset: int, length: int, out) -> None:
        if offset < 0 or length < 0 or offset + length > self.identity[2]:
            raise ValueError("the requested range lies outside the source file")
        self.stream.seek(offset)
        for piece in blocks(self.stream, length):
            out.write(piece)
        out.flush()
        self.require_unchanged()


def source_action(action: str, argv: list) -> None:
    source = SourceFile(argv[0])
    with source.stream:
        if action == "manifest":
            print(json.dumps(source.manifest(int(argv[1]))))
            return
        source.require_identity(json.loads(argv[1]))
        if action == "identity":
            source.require_unchanged()
            print(json.dumps({"identity": source.identity}))
        else:
            source.send(int(argv[2]), int(argv[3]), sys.stdout.buffer)


# ---------------------------------------------------------------------------------- receiver side
def chunk_extent(state: dict, index: int):
    offset = index * state["chunk_size"]
    return offset, min(state["chunk_size"], state["size"] - offset)


def publish_noreplace(source: Path, target: Path) -> None:
    rename = ctypes.CDLL(None, use_errno=True).renameat2
    rename.restype = ctypes.c_int
    rename.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint]
    if rename(-100, os.fsencode(source), -100, os.fsencode(target), 1) != 0:      # AT_FDCWD, RENAME_NOREPLACE
        number = ctypes.get_errno()
        raise OSError(number, os.strerror(number), str(target))
    sync_dir(target.parent)


class Upload:
    """Receiver state of one destination file: the partial file, its manifest and the chunk receipts."""

    def __init__(self, target, expected_sha: str, exclusive: bool):
        self.target, self.expected = confined(target), expected_sha
        self.target.parent.mkdir(parents=True, exist_ok=True)
        confined(self.target.parent)
        self.partial = confined(f"{self.target}.uploading")
        self.state_path = confined(f"{self.target}.upload-state.json")
        self.receipts = confined(f"{self.target}.upload-chunks")
        self.lock = open_regular(f"{self.target}.upload.lock", os.O_RDWR | os.O_CREAT)
        fcntl.flock(self.lock, fcntl.LOCK_EX if exclusive else fcntl.LOCK_SH)   # chunk writers share, the rest exclude
        self.state = None

    def receipt(self, index: int) -> Path:
        return confined(self.receipts / f"{index:08d}.json")

    def published(self, size: int) -> bool:
        """True when the destination already holds exactly this file; raises when it holds another."""
        if not self.target.exists():
            return False
        if self.target.stat().st_size == size and sha_range(self.target) == self.expected:
            return True
        raise ValueError(f"{self.target} exists with other contents; it is never overwritten")

    def load_state(self) -> None:
        self.state = read_json(self.state_path)
        if self.state["sha256"] != self.expected:
            raise ValueError("the partial upload belongs to another source file")

    # ---- prepare
    def prepare(self, incoming: dict) -> dict:
        if incoming["sha256"] != self.expected:
            raise ValueError("the manifest does not describe the announced source file")
        if self.published(incoming["size"]):
            return {"complete": True, "sha256": self.expected}
        if self.state_path.exists():
            if read_json(self.state_path) != incoming:
                raise ValueError("a partial upload of another source or chunk size is in the way")
        elif self.partial.exists() or self.receipts.exists():
            raise ValueError("upload sidecars without a manifest are in the way; not touching them")
        else:
            write_json(self.state_path, incoming)     # the manifest comes first: any later interruption can resume
        self.state = incoming
        if not self.partial.exists():
            fd = open_regular(self.partial, os.O_WRONLY | os.O_CREAT | os.O_EXCL)
            try:
                os.ftruncate(fd, incoming["size"])
                os.fsync(fd)
            finally:
                os.close(fd)
        if self.partial.stat().st_size != incoming["size"]:
            raise ValueError("the partial file does not have the size its manifest states")
        self.receipts.mkdir(exist_ok=True)
        kept = [index for index in range(len(incoming["chunk_sha256"])) if self._receipt_holds(index)]
        sync_dir(self.receipts)
        return {"complete": False, "completed": kept}

    def _receipt_holds(self, index: int) -> bool:
        """Re-hash a receipted chunk; a receipt that no longer matches is dropped."""
        note = self.receipt(index)
        if not note.exists():
            return False
        offset, length = chunk_extent(self.state, index)
        want = self.state["chunk_sha256"][index]
        try:
            good = read_json(note) == {"sha256": want, "size": length} and sha_range(self.partial, offset, length) == want
        except (OSError, ValueError):
            good = False
        if not good:
            note.unlink()
        return good

    # ---- write
    def write(self, index: int, incoming) -> dict:
        self.load_state()
        if not 0 <= index < len(self.state["chunk_sha256"]):
            raise ValueError("no such chunk")
        offset, length = chunk_extent(self.state, index)
        digest = hashlib.sha256()
        fd = open_regular(self.partial, os.O_WRONLY)
        try:
            at = offset
            for piece in blocks(incoming, length):
                digest.update(piece)
                rest = memoryview(piece)
                while rest:
                    done = os.pwrite(fd, rest, at)
                    if done <= 0:
                        raise OSError("pwrite wrote nothing")
                    rest, at = rest[done:], at + done
            if incoming.read(1):
                raise ValueError("more bytes arrived than the chunk holds")
            if digest.hexdigest() != self.state["chunk_sha256"][index]:
                raise ValueError("chunk SHA256 mismatch")
            os.fsync(fd)
        finally:
            os.close(fd)
        write_json(self.receipt(index), {"sha256": digest.hexdigest(), "size": length})
        return {"index": index, "sha256": digest.hexdigest(), "bytes": length}

    # ---- finalize
    def finalize(self) -> dict:
        self.load_state()
        outcome = {"complete": True, "sha256": self.expected, "bytes": self.state["size"]}
        if self.published(self.state["size"]):
            return outcome
        for index, want in enumerate(self.state["chunk_sha256"]):
            note = self.receipt(index)
            if not note.exists() or read_json(note) != {"sha256": want, "size": chunk_extent(self.state, index)[1]}:
                raise ValueError(f"chunk {index} has no valid receipt")
        if self.partial.stat().st_size != self.state["size"] or sha_range(self.partial) != self.expected:
            raise ValueError("the assembled file does not hash to the source's SHA256; the partial upload is kept")
        publish_noreplace(self.partial, self.target)
        return outcome


def receiver_action(action: str, argv: list) -> None:
    upload = Upload(argv[0], argv[1], exclusive=action != "write")
    if action == "prepare":
        result = upload.prepare(json.load(sys.stdin))
    elif action == "write":
        result = upload.write(int(argv[2]), sys.stdin.buffer)
    elif action == "finalize":
        result = upload.finalize()
    else:
        raise ValueError(f"unknown receiver action {action}")
    print(json.dumps(result))


def agent_main(argv: list) -> None:
    action = argv[0]
    if action in ("manifest", "identity", "read"):
        source_action(action, argv[1:])
    elif action in ("prepare", "write", "finalize"):
        receiver_action(action, argv[1:])
    else:
        raise ValueError(f"unknown action {action}")


if __name__ == "__main__":
    agent_main(sys.argv[1:])
