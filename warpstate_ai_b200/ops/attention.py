"""Chunk attention + matrix-memory kernels (front-end of csrc/attention_fwd.cu, attention_bwd.cu).

Supported geometry: chunk_size 128, head_dim 64, sequence length a multiple of 128 (the
production model).  Other geometries use the plain-PyTorch composite in `reference.py`.
"""
from __future__ import annotations

import torch

from . import _ext
from .gemm import error_flag

_rope_cache: dict = {}
BACKWARD_READY = True
MAX_CHUNKS = 256


def rope_table(device: torch.device, pair_major: bool = False) -> torch.Tensor:
    """(cos, sin) per in-chunk position and rotary pair: float32 [128, 32, 2], or with
    ``pair_major`` [32, 128, 2] (what the chunk kernels read: one thread per position)."""
    if pair_major:
        key = (device.type, device.index, "pair-major")
        table = _rope_cache.get(key)
        if table is None:
            table = rope_table(device).transpose(0, 1).contiguous()
            _rope_cache[key] = table
        return table
    key = (device.type, device.index)
    table = _rope_cache.get(key)
    if table is None:
        pos = torch.arange(128, device=device, dtype=torch.float32)
        inv = 1.0 / (10000 ** (torch.arange(0, 64, 2, device=device, dtype=torch.float32) / 64))
        ang = torch.outer(pos, inv)
        table = torch.stack((ang.cos(), ang.sin()), dim=-1).contiguous()
        _rope_cache[key] = table
    return table


def geometry_ok(core) -> bool:
    return core.chunk == 128 and core.hd == 64 and core.cfg.dropout == 0.0


def kernels_ready(core) -> bool:
    return BACKWARD_READY and geometry_ok(core) and _ext.available()


def _logits(core):
    return (core.fast_decay_logit.detach().float().contiguous(),
            core.slow_decay_logit.detach().float().contiguous(),
            core.memory_mix_logit.detach().float().contiguous())


def forward_only(qkvgu: torch.Tensor, core, batch: int, seq: int, want_final: bool = False):
    """y [M,d] (and optionally the final fast/slow states) with the CUDA kernels."""
    _ext.require()
    ops = torch.ops.ws_b200
    rope = rope_table(qkvgu.device, pair_major=True)
    flag = error_flag(qkvgu.device)
    writes = ops.chunk_writes(qkvgu, rope, batch, seq, core.h, flag)
    fl = core.fast_decay_logit.detach().float().contiguous()
    sl = core.slow_decay_logit.detach().float().contiguous()
    ml = core.memory_mix_logit.detach().float().contiguous()
    states, ff, fs = ops.memory_scan(writes, fl, sl, ml, True, want_final, None, None)
    y = ops.attn_fwd(qkvgu, states, rope, batch, seq, core.h, flag)
    return y, writes, states, (ff, fs)


def forward(qkvgu: torch.Tensor, core, batch: int, seq: int):
    y, writes, states, _ = forward_only(qkvgu, core, batch, seq)
    return y, (writes, states)


def backward(dy, qkvgu, saved, core, batch: int, seq: int):
    """-> (dqkvgu [M,5d] BF16, d fast_decay_logit, d slow_decay_logit, d memory_mix_logit)."""
    if seq // 128 > MAX_CHUNKS:
        raise ValueError(f"the memory-scan backward kernel handles at most {MAX_CHUNKS} chunks per sequence")
    writes, states = saved
    fl, sl, ml = _logits(core)
    dqkvgu, partials = torch.ops.ws_b200.attn_bwd(qkvgu, dy.contiguous(), states, writes, rope_table(qkvgu.device, pair_major=True),
                                                  fl, sl, ml, batch, seq, core.h, error_flag(qkvgu.device))
    g = partials.view(batch, core.h, 16, 3).sum(dim=(0, 2))  # [H, 3] gradients w.r.t. the sigmoids
    df, ds, mix = torch.sigmoid(fl), torch.sigmoid(sl), torch.sigmoid(ml)
    return (dqkvgu, g[:, 0] * df * (1 - df), g[:, 1] * ds * (1 - ds), g[:, 2] * mix * (1 - mix))
