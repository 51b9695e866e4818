"""Chunk attention + matrix-memory kernels (front-end; kernels live in csrc/attention_*.cu)."""
from __future__ import annotations

import torch


def kernels_ready(core) -> bool:
    return False
