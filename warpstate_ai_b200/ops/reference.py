"""Plain-PyTorch definitions of every fused op.

These functions are (a) the CPU / non-CUDA execution path of the model and (b) the oracles
the CUDA kernels are tested against.  The math follows the reference model
(warpstate/model.py:15-60 for norm/rope/SwiGLU, :114-207 for the core).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- norm / rope / swiglu
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """FP32 statistics; result in the input dtype (warpstate/model.py:22-28)."""
    dtype = x.dtype
    x32 = x.float()
    x32 = x32 * torch.rsqrt(x32.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x32.to(dtype) * weight.to(dtype)


def rope_tables(length: int, dim: int, device, dtype=torch.float32):
    """cos/sin ``[length, dim]`` with each frequency repeated for an interleaved pair."""
    pos = torch.arange(length, device=device, dtype=torch.float32)
    inv = 1.0 / (10000 ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    ang = torch.repeat_interleave(torch.outer(pos, inv), 2, dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def rotate_pairs(x: torch.Tensor) -> torch.Tensor:
    """(x0, x1, x2, x3, ...) -> (-x1, x0, -x3, x2, ...)."""
    even = x[..., 0::2]
    odd = x[..., 1::2]
    return torch.stack((-odd, even), dim=-1).flatten(-2)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x [..., C, Dh]`` rotated by position inside the chunk (tables ``[C, Dh]``)."""
    return x * cos + rotate_pairs(x) * sin


def swiglu(packed: torch.Tensor) -> torch.Tensor:
    """``packed = (up | gate)``: first half is `up`, second half is `gate`."""
    up, gate = packed.chunk(2, dim=-1)
    return F.silu(gate) * up


# --------------------------------------------------------------------------- memory scan helpers
def decay_weights(logit: torch.Tensor, n_chunks: int) -> torch.Tensor:
    """``W[h,i,j] = (1-d_h) d_h^(i-j-1)`` for ``j < i`` else 0, FP32 (warpstate/model.py:162-167)."""
    index = torch.arange(n_chunks, device=logit.device)
    lag = index[:, None] - index[None, :] - 1
    mask = lag >= 0
    decay = logit.float().sigmoid()[:, None, None]
    return (1 - decay) * decay.pow(lag.clamp_min(0)[None]) * mask


def chunk_writes(k_roped: torch.Tensor, u: torch.Tensor, chunk: int) -> torch.Tensor:
    """``tanh(K)^T tanh(U) / C`` per chunk: ``[B,N,H,C,Dh] -> [B,N,H,Dh,Dh]``."""
    return (torch.tanh(k_roped).transpose(-2, -1) @ torch.tanh(u)) / chunk


def prefix_states(writes: torch.Tensor, logit: torch.Tensor) -> torch.Tensor:
    """State seen by chunk ``i`` = decayed sum of the writes of chunks ``< i`` (matrix form)."""
    b, n, h, dh, _ = writes.shape
    weights = decay_weights(logit, n)
    values = writes.permute(0, 2, 1, 3, 4).flatten(-2)
    result = torch.matmul(weights.to(values.dtype), values)
    return result.view(b, h, n, dh, dh).transpose(1, 2)


# --------------------------------------------------------------------------- the core's middle
def attention_memory(qkvgu: torch.Tensor, fast_logit: torch.Tensor, slow_logit: torch.Tensor,
                     mix_logit: torch.Tensor, n_heads: int, chunk: int, parallel_memory: bool,
                     cos: torch.Tensor, sin: torch.Tensor, dropout_p: float = 0.0,
                     return_state: bool = False):
    """Everything between ``in_proj`` and ``out_proj``.

    ``qkvgu [B,T,5d]`` holds Q,K,V,gate,U in that order.  Returns ``y [B,T,d]`` =
    ``sigmoid(g) * local + (1 - sigmoid(g)) * memory`` where `local` is causal attention inside
    each 128-token chunk and `memory` reads the fast/slow states built from *earlier* chunks.
    With ``return_state`` also returns the (fast, slow) states after the last chunk.
    """
    b, t, d5 = qkvgu.shape
    d = d5 // 5
    hd = d // n_heads
    if t % chunk != 0:
        raise ValueError(f"sequence length {t} must be divisible by chunk_size={chunk}")
    n = t // chunk
    q, k, v, g, u = qkvgu.chunk(5, dim=-1)

    def chunked(y):  # [B,T,d] -> [B,N,H,C,Dh]
        return y.reshape(b, n, chunk, n_heads, hd).permute(0, 1, 3, 2, 4).contiguous()

    q, k, v, g, u = chunked(q), chunked(k), chunked(v), chunked(g), chunked(u)
    cos = cos.to(q.dtype).view(1, 1, 1, chunk, hd)
    sin = sin.to(q.dtype).view(1, 1, 1, chunk, hd)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)

    local = F.scaled_dot_product_attention(
        q.reshape(b * n, n_heads, chunk, hd), k.reshape(b * n, n_heads, chunk, hd),
        v.reshape(b * n, n_heads, chunk, hd), dropout_p=dropout_p, is_causal=True,
    ).view(b, n, n_heads, chunk, hd)

    fast_decay = torch.sigmoid(fast_logit).to(q.dtype).view(1, n_heads, 1, 1)
    slow_decay = torch.sigmoid(slow_logit).to(q.dtype).view(1, n_heads, 1, 1)
    mix = torch.sigmoid(mix_logit).to(q.dtype).view(1, n_heads, 1, 1)
    scale = 1.0 / math.sqrt(hd)

    final_state = None
    if parallel_memory:
        writes = chunk_writes(k, u, chunk)
        mix5 = mix.unsqueeze(1)
        state = mix5 * prefix_states(writes, fast_logit) + (1 - mix5) * prefix_states(writes, slow_logit)
        memory = (q @ state) / math.sqrt(hd)
        gate = torch.sigmoid(g)
        y = gate * local + (1 - gate) * memory
        if return_state:
            fast = torch.zeros((b, n_heads, hd, hd), device=q.device, dtype=q.dtype)
            slow = torch.zeros_like(fast)
            for i in range(n):
                fast = fast_decay * fast + (1.0 - fast_decay) * writes[:, i]
                slow = slow_decay * slow + (1.0 - slow_decay) * writes[:, i]
            final_state = (fast, slow)
    else:
        fast = torch.zeros((b, n_heads, hd, hd), device=q.device, dtype=q.dtype)
        slow = torch.zeros_like(fast)
        outs = []
        for i in range(n):
            qi = q[:, i]
            gi = torch.sigmoid(g[:, i])
            read_fast = torch.matmul(qi, fast) / math.sqrt(hd)
            read_slow = torch.matmul(qi, slow) / math.sqrt(hd)
            memory = mix * read_fast + (1.0 - mix) * read_slow
            outs.append(gi * local[:, i] + (1.0 - gi) * memory)
            write = torch.matmul(torch.tanh(k[:, i]).transpose(-2, -1), torch.tanh(u[:, i])) / float(chunk)
            fast = fast_decay * fast + (1.0 - fast_decay) * write
            slow = slow_decay * slow + (1.0 - slow_decay) * write
        y = torch.stack(outs, dim=1)
        final_state = (fast, slow)
    del scale
    y = y.permute(0, 1, 3, 2, 4).contiguous().view(b, t, d)
    if return_state:
        return y, final_state
    return y


# --------------------------------------------------------------------------- LM head
def lm_head_loss_sum(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                     ignore_index: int = -100) -> torch.Tensor:
    """Sum over valid rows of the cross-entropy of ``hidden @ weight.T`` (FP32 softmax)."""
    return F.cross_entropy(F.linear(hidden, weight).float(), labels, ignore_index=ignore_index, reduction="sum")


def lm_head_token_logps(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                        ignore_index: int = -100) -> torch.Tensor:
    """Per-row log-probability of the label (0 where the label is ignored), FP32."""
    return -F.cross_entropy(F.linear(hidden, weight).float(), labels, ignore_index=ignore_index, reduction="none")
