"""Fused LM-head cross-entropy kernels (front-end)."""
from __future__ import annotations

import torch


def kernels_ready(hidden: torch.Tensor, weight: torch.Tensor) -> bool:
    return False
