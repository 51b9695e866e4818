"""Sealed inference snapshots: export from a training checkpoint, verification, loading.

What the reference guarantees and this module keeps (reference chat.py:37-151): a training
checkpoint (``warpstate-server-v1``) is never served directly.  The trainer publishes ``latest.pt``
by rename, so a reader that holds the file open keeps one complete version; the exporter pins the
file by descriptor, copies only the model into a read-only ``warpstate-chat-v1`` file, checks that
the pinned file did not change meanwhile, and writes a ``snapshot.json`` seal (SHA-256 and size of
the export plus provenance).  Loading re-checks the seal, the tokenizer hash and a strict
meta-device state-dict load.

Structure here: `PinnedFile` owns the descriptor and the "did it change" question,
`SnapshotSeal` is the sidecar as a typed record, `SnapshotStore` is a directory of exports.
"""
from __future__ import annotations

import gc
import json
import os
import stat
import tempfile
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch

from ..ckpt.formats import CHAT_FORMAT, SERVER_FORMAT
from ..config import WarpStateConfig
from ..models.warpstate import WarpStateLM
from ..utils.io import digest, fsync_dir, utc_timestamp

SEAL_NAME = "snapshot.json"
WEIGHTS_NAME = "model.pt"


class PinnedFile:
    """A regular file held open read-only; the descriptor keeps one version of a file that its
    writer replaces by rename."""

    def __init__(self, path: Path):
        self.path = Path(path)
        if self.path.suffix != ".pt" or self.path.is_symlink():
            raise ValueError(f"{self.path}: need a finished, regular .pt checkpoint (no link, no temporary file)")
        self.fd = os.open(self.path, os.O_RDONLY | os.O_NOFOLLOW)
        self.first = os.fstat(self.fd)
        if not stat.S_ISREG(self.first.st_mode):
            os.close(self.fd)
            raise ValueError(f"{self.path}: not a regular file")

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        os.close(self.fd)

    @staticmethod
    def _identity(st) -> tuple:
        return st.st_dev, st.st_ino, st.st_size, st.st_mtime_ns

    def unchanged(self) -> bool:
        return self._identity(os.fstat(self.fd)) == self._identity(self.first)

    def load(self):
        return torch.load(f"/proc/self/fd/{self.fd}", map_location="cpu", weights_only=False, mmap=True)

    def provenance(self) -> dict:
        st = self.first
        return {"path": str(self.path.resolve()), "device": st.st_dev, "inode": st.st_ino, "size": st.st_size,
                "mtime_ns": st.st_mtime_ns}


@dataclass
class SnapshotSeal:
    """Contents of ``snapshot.json`` (and, minus the last two fields, the metadata stored inside the export)."""
    format: str
    inference_only: bool
    config: dict
    step: int
    tokens_seen: int
    val_loss: float | None
    tokenizer_sha256: str
    captured_at_utc: str
    source: dict
    extra: dict = field(default_factory=dict)      # stage / origin of post-training exports
    snapshot_sha256: str | None = None
    snapshot_bytes: int | None = None

    def embedded(self) -> dict:
        record = asdict(self)
        record.update(record.pop("extra"))
        record.pop("snapshot_sha256")
        record.pop("snapshot_bytes")
        return record

    def sidecar(self) -> dict:
        record = self.embedded()
        record["snapshot_sha256"], record["snapshot_bytes"] = self.snapshot_sha256, self.snapshot_bytes
        return record


def _write_once(path: Path, write) -> None:
    """Create ``path`` (must not exist), write, flush to disk."""
    with path.open("xb") as stream:
        write(stream)
        stream.flush()
        os.fsync(stream.fileno())


class SnapshotStore:
    """A directory holding one sub-directory per export (``step-<n>-<random>/model.pt`` + seal)."""

    def __init__(self, root, tokenizer):
        self.root, self.tokenizer = Path(root), Path(tokenizer)

    # ------------------------------------------------------------------ export
    def export(self, checkpoint_path) -> Path:
        tokenizer_hash = digest(self.tokenizer)
        with PinnedFile(Path(checkpoint_path)) as pinned:
            checkpoint = pinned.load()
            kind = checkpoint.get("format")
            if kind == CHAT_FORMAT:
                raise ValueError(f"{pinned.path} is already an inference export but its {SEAL_NAME} is missing; "
                                 "put the seal back next to it or export again from a training checkpoint")
            if kind != SERVER_FORMAT:
                raise ValueError(f"{pinned.path}: expected a {SERVER_FORMAT} training checkpoint, found {kind!r}")
            trained_with = checkpoint["signature"]["data"]["signature"]["tokenizer_sha256"]
            if trained_with != tokenizer_hash:
                raise ValueError("the tokenizer file is not the one this checkpoint was trained with (SHA256 differs)")
            seal = SnapshotSeal(format=CHAT_FORMAT, inference_only=True, config=checkpoint["config"],
                                step=checkpoint["step"], tokens_seen=checkpoint["tokens_seen"],
                                val_loss=checkpoint.get("val_loss"), tokenizer_sha256=tokenizer_hash,
                                captured_at_utc=utc_timestamp(), source=pinned.provenance())
            self.root.mkdir(parents=True, exist_ok=True)
            folder = Path(tempfile.mkdtemp(prefix=f"step-{seal.step}-", dir=self.root))
            print(f"Exporting step {seal.step:,} ({seal.tokens_seen:,} tokens): model weights only ...", flush=True)
            staging, final = folder / (WEIGHTS_NAME + ".tmp"), folder / WEIGHTS_NAME
            _write_once(staging, lambda stream: torch.save({**seal.embedded(), "model": checkpoint["model"]}, stream))
            if not pinned.unchanged():
                raise RuntimeError("the checkpoint changed while it was being exported; nothing was published")
            os.chmod(staging, 0o444)
            os.replace(staging, final)
            seal.snapshot_sha256, seal.snapshot_bytes = digest(final), final.stat().st_size
            _write_once(folder / SEAL_NAME,
                        lambda stream: stream.write((json.dumps(seal.sidecar(), indent=2) + "\n").encode()))
            fsync_dir(folder)
            return final

    def resolve(self, path) -> Path:
        """An existing export is used as it is; anything else is treated as a training checkpoint."""
        path = Path(path)
        if not path.is_file():
            raise ValueError(f"{path}: no such checkpoint file")
        return path if path.with_name(SEAL_NAME).exists() else self.export(path)

    # ------------------------------------------------------------------ load
    def load(self, snapshot, device: str = "cpu"):
        """-> (model in eval mode on ``device``, SentencePiece processor, metadata without weights)."""
        import sentencepiece as spm
        snapshot = Path(snapshot)
        seal_path = snapshot.with_name(SEAL_NAME)
        if not seal_path.exists():
            raise ValueError(f"{seal_path} is missing: pass a training checkpoint with --checkpoint to export it, "
                             "or restore the seal written at export time")
        seal = json.loads(seal_path.read_text())
        recorded = seal.get("snapshot_sha256") if isinstance(seal, dict) else None
        if not isinstance(recorded, str):
            raise ValueError(f"{seal_path} is not a snapshot seal")
        if recorded != digest(snapshot):
            raise ValueError("snapshot SHA256 does not match its seal")
        payload = torch.load(snapshot, map_location="cpu", weights_only=False, mmap=True)
        if payload.get("format") != CHAT_FORMAT or payload.get("inference_only") is not True:
            raise ValueError("not an inference export (a live training checkpoint must be exported first)")
        if payload["tokenizer_sha256"] != digest(self.tokenizer):
            raise ValueError("tokenizer SHA256 does not match the snapshot")
        config = WarpStateConfig(**payload["config"])
        processor = spm.SentencePieceProcessor(model_file=str(self.tokenizer))
        if processor.vocab_size() != config.vocab_size:
            raise ValueError("tokenizer and model disagree on the vocabulary size")
        with torch.device("meta"):
            model = WarpStateLM(config)
        model.load_state_dict(payload["model"], strict=True, assign=True)
        model.eval().requires_grad_(False)
        if {p.dtype for p in model.parameters()} != {torch.float32}:
            raise ValueError("an export keeps the FP32 master parameters; found another dtype")
        metadata = {key: value for key, value in payload.items() if key != "model"}
        model = model.to(device)
        del payload
        gc.collect()
        return model, processor, metadata
