"""Model configuration (same fields, defaults and JSON form as the reference's
warpstate/config.py:12-46, so checkpoints that store ``vars(cfg)`` load unchanged)."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, fields
from pathlib import Path


@dataclass
class WarpStateConfig:
    vocab_size: int = 32768
    d_model: int = 1280
    n_heads: int = 20
    n_cores: int = 4
    logical_depth: int = 16
    ffn_hidden: int = 4480
    chunk_size: int = 128
    dropout: float = 0.0
    rms_eps: float = 1e-5
    gradient_checkpointing: bool = True
    parallel_memory: bool = False
    loss_chunk_size: int = 128

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def validate(self) -> None:
        if self.d_model % self.n_heads != 0:
            raise AssertionError("d_model must be divisible by n_heads")
        if self.logical_depth < self.n_cores:
            raise AssertionError("logical_depth must be at least n_cores")
        if self.chunk_size <= 0 or self.n_cores <= 0 or self.loss_chunk_size <= 0:
            raise AssertionError("chunk_size, n_cores and loss_chunk_size must be positive")
        if self.head_dim % 2 != 0:
            raise AssertionError("head_dim must be even (rotary pairs)")

    @classmethod
    def from_dict(cls, data: dict) -> "WarpStateConfig":
        known = {f.name for f in fields(cls)}
        unknown = set(data) - known
        if unknown:
            raise TypeError(f"unknown WarpStateConfig fields: {sorted(unknown)}")
        cfg = cls(**data)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str | Path) -> "WarpStateConfig":
        return cls.from_dict(json.loads(Path(path).read_text(encoding="utf-8")))

    def to_json(self, path: str | Path) -> None:
        Path(path).write_text(json.dumps(asdict(self), indent=2), encoding="utf-8")

    def to_dict(self) -> dict:
        return asdict(self)


def warpstate_2b() -> WarpStateConfig:
    """The 2,005,111,424-parameter production configuration (256 tensors)."""
    return WarpStateConfig(vocab_size=32768, d_model=2048, n_heads=32, n_cores=28, logical_depth=28,
                           ffn_hidden=7168, chunk_size=128, dropout=0.0, rms_eps=1e-5,
                           gradient_checkpointing=True, parallel_memory=True, loss_chunk_size=128)


def warpstate_smoke() -> WarpStateConfig:
    """Tiny CPU smoke configuration: 2 shared cores x 2 depth passes each."""
    return WarpStateConfig(vocab_size=32768, d_model=256, n_heads=4, n_cores=2, logical_depth=4,
                           ffn_hidden=688, chunk_size=128, dropout=0.0, rms_eps=1e-5,
                           gradient_checkpointing=False, parallel_memory=True, loss_chunk_size=128)
