"""The model's arithmetic in plain PyTorch, one small function per operation.

Two roles: the execution path on anything that is not a CUDA device with the kernel library, and the statement of
each operation that the CUDA kernels are tested against.  What is computed is fixed by the architecture (reference
warpstate/model.py:15-60 for norm, rotary pairs and SwiGLU; :114-207 for the block's middle; :222-274 for the decode
recurrence); how it is written here is this package's own: tensors keep named axes

    b batch   n chunk   h head   c position in the chunk   x, y head-feature axes   t = n * c

the two memory modes differ only in how the per-chunk states are accumulated (`states_seen`), and the decode step is
the same arithmetic on one position (`decode_position`).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

IGNORE = -100


# ------------------------------------------------------------------------------------------- element-wise pieces
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Root-mean-square normalisation with FP32 statistics; rounded to the input dtype before the learned scale."""
    wide = x.to(torch.float32)
    inverse_rms = torch.rsqrt(torch.mean(wide * wide, dim=-1, keepdim=True) + eps)
    return (wide * inverse_rms).to(x.dtype) * weight.to(x.dtype)


def rope_tables(length: int, dim: int, device, dtype=torch.float32):
    """``(cos, sin)`` of shape ``[length, dim]``; feature pair ``(2i, 2i + 1)`` turns at ``10000 ** (-2i / dim)``
    radians per position, so each frequency appears twice in a row."""
    frequency = torch.pow(10000.0, -torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim)
    position = torch.arange(length, device=device, dtype=torch.float32)
    angle = (position[:, None] * frequency[None, :]).repeat_interleave(2, dim=1)
    return torch.cos(angle).to(dtype), torch.sin(angle).to(dtype)


def rotate_pairs(x: torch.Tensor) -> torch.Tensor:
    """Quarter turn of every feature pair: ``(a, b) -> (-b, a)``."""
    pairs = x.unflatten(-1, (-1, 2))
    return torch.stack((-pairs[..., 1], pairs[..., 0]), dim=-1).flatten(-2)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate ``x [..., c, x]`` by the angle of its position inside the chunk (tables broadcast against ``x``)."""
    return cos * x + sin * rotate_pairs(x)


def swiglu(packed: torch.Tensor) -> torch.Tensor:
    """``packed`` holds ``up`` in its first half and ``gate`` in its second: ``up * silu(gate)``."""
    half = packed.shape[-1] // 2
    return packed[..., :half] * F.silu(packed[..., half:])


# ------------------------------------------------------------------------------------------- matrix memory
def chunk_writes(k_roped: torch.Tensor, u: torch.Tensor, chunk: int) -> torch.Tensor:
    """What a chunk adds to the memory: ``mean over c of tanh(k)[c, x] * tanh(u)[c, y]`` -> ``[..., x, y]``."""
    return torch.einsum("...cx,...cy->...xy", torch.tanh(k_roped), torch.tanh(u)) / chunk


def decay_weights(logit: torch.Tensor, n_chunks: int, rows: int | None = None) -> torch.Tensor:
    """``W[h, i, j]``: weight of chunk ``j``'s write in the state after ``i`` chunks, ``(1 - d) d^(i - 1 - j)`` for
    ``j < i`` and zero otherwise, with ``d = sigmoid(logit[h])``; FP32.  Row ``i < n`` is what chunk ``i`` reads;
    ``rows = n + 1`` adds the state left behind by the last chunk."""
    rows = n_chunks if rows is None else rows
    keep = torch.sigmoid(logit.to(torch.float32))[:, None, None]
    age = (torch.arange(rows, device=logit.device)[:, None] - 1 - torch.arange(n_chunks, device=logit.device)[None, :])
    return torch.where(age >= 0, (1.0 - keep) * torch.pow(keep, age.clamp(min=0)), torch.zeros((), device=logit.device))


def states_seen(writes: torch.Tensor, logit: torch.Tensor, parallel: bool):
    """-> (state read by every chunk ``[b, n, h, x, y]``, state after the last chunk ``[b, h, x, y]``).

    ``parallel`` evaluates the recurrence ``S <- d S + (1 - d) write`` for all chunks at once as a lower-triangular
    weighting of the writes; otherwise it is run chunk after chunk.  Same numbers up to the order of additions."""
    chunks = writes.shape[1]
    if parallel:
        weights = decay_weights(logit, chunks, rows=chunks + 1).to(writes.dtype)
        every = torch.einsum("hij,bjhxy->bihxy", weights, writes)
        return every[:, :chunks], every[:, chunks]
    keep = torch.sigmoid(logit).to(writes.dtype)[None, :, None, None]
    state = torch.zeros_like(writes[:, 0])
    seen = []
    for index in range(chunks):
        seen.append(state)
        state = keep * state + (1.0 - keep) * writes[:, index]
    return torch.stack(seen, dim=1), state


def split_heads(qkvgu: torch.Tensor, n_heads: int, chunk: int):
    """``[b, t, 5 * h * x]`` (Q | K | V | gate | U) -> five tensors ``[b, n, h, c, x]``."""
    batch, length, packed = qkvgu.shape
    if length % chunk:
        raise ValueError(f"sequence length {length} must be divisible by chunk_size={chunk}")
    features = packed // (5 * n_heads)
    parts = qkvgu.reshape(batch, length // chunk, chunk, 5, n_heads, features).permute(3, 0, 1, 4, 2, 5)
    return tuple(part.contiguous() for part in parts)


def attention_memory(qkvgu: torch.Tensor, fast_logit: torch.Tensor, slow_logit: torch.Tensor,
                     mix_logit: torch.Tensor, n_heads: int, chunk: int, parallel_memory: bool,
                     cos: torch.Tensor, sin: torch.Tensor, dropout_p: float = 0.0,
                     return_state: bool = False):
    """The block between its input and output projections: ``[b, t, 5d] -> [b, t, d]``.

    Every position attends causally inside its own chunk (rotary angles restart with the chunk) and reads a matrix
    memory that holds only *earlier* chunks: two decayed sums of the chunks' writes, a fast and a slow one, blended
    per head; a learned gate mixes the two results per feature.  With ``return_state`` the (fast, slow) memories
    after the last chunk are returned as well (where a decode continues from)."""
    q, k, v, gate, u = split_heads(qkvgu, n_heads, chunk)
    features = q.shape[-1]
    cos, sin = cos.to(q.dtype), sin.to(q.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    # chunks are independent sequences for the attention: fold them into the batch (four dimensions, so that the
    # library may pick any of its kernels)
    local = F.scaled_dot_product_attention(q.flatten(0, 1), k.flatten(0, 1), v.flatten(0, 1), dropout_p=dropout_p,
                                           is_causal=True).unflatten(0, q.shape[:2])

    writes = chunk_writes(k, u, chunk)
    fast_seen, fast_last = states_seen(writes, fast_logit, parallel_memory)
    slow_seen, slow_last = states_seen(writes, slow_logit, parallel_memory)
    mix = torch.sigmoid(mix_logit).to(q.dtype)[None, None, :, None, None]
    blended = mix * fast_seen + (1.0 - mix) * slow_seen
    memory = torch.einsum("bnhcx,bnhxy->bnhcy", q, blended) / math.sqrt(features)

    open_gate = torch.sigmoid(gate)
    y = open_gate * local + (1.0 - open_gate) * memory
    y = y.transpose(2, 3).reshape(qkvgu.shape[0], qkvgu.shape[1], n_heads * features)
    return (y, (fast_last, slow_last)) if return_state else y


def decode_position(q, k, v, gate, u, keys, values, pending, fast, slow, position: int, chunk: int,
                    fast_logit, slow_logit, mix_logit):
    """One new position of every sequence, the recurrence that `attention_memory` evaluates chunk-wise.

    ``q .. u [b, h, 1, x]`` are the position's projections (not yet rotated); ``keys / values [b, h, chunk, x]`` hold
    the chunk so far, ``pending [b, h, x, y]`` its unnormalised write, ``fast / slow`` the memories of the earlier
    chunks.  All five are updated in place; at the last position of a chunk the write is folded into the memories and
    the chunk's buffers are cleared.  -> (output ``[b, h, 1, x]``, position inside the chunk of the next call)."""
    features = q.shape[-1]
    cos, sin = rope_tables(position + 1, features, q.device, q.dtype)
    q, k = apply_rope(q, cos[position], sin[position]), apply_rope(k, cos[position], sin[position])
    keys[:, :, position] = k[:, :, 0]
    values[:, :, position] = v[:, :, 0]
    filled = position + 1
    scores = torch.einsum("bhqx,bhkx->bhqk", q, keys[:, :, :filled]) / math.sqrt(features)
    local = torch.einsum("bhqk,bhkx->bhqx", torch.softmax(scores, dim=-1), values[:, :, :filled])

    per_head = lambda logit: torch.sigmoid(logit).to(q.dtype)[None, :, None, None]
    mix = per_head(mix_logit)
    memory = torch.einsum("bhqx,bhxy->bhqy", q, mix * fast + (1.0 - mix) * slow) / math.sqrt(features)
    open_gate = torch.sigmoid(gate)
    out = open_gate * local + (1.0 - open_gate) * memory

    pending += chunk_writes(k, u, 1)
    if filled < chunk:
        return out, filled
    write = pending / chunk
    for state, logit in ((fast, fast_logit), (slow, slow_logit)):
        keep = per_head(logit)
        state.copy_(keep * state + (1.0 - keep) * write)
    for buffer in (keys, values, pending):
        buffer.zero_()
    return out, 0


# ------------------------------------------------------------------------------------------- tied output head
def lm_head_loss_sum(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                     ignore_index: int = IGNORE) -> torch.Tensor:
    """Cross-entropy of ``hidden @ weight.T`` against ``labels``, summed over the rows that have a label; the
    soft-max runs in FP32."""
    logits = torch.matmul(hidden, weight.t()).to(torch.float32)
    return F.cross_entropy(logits, labels, ignore_index=ignore_index, reduction="sum")


def lm_head_token_logps(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                        ignore_index: int = IGNORE) -> torch.Tensor:
    """FP32 log-probability of each row's label; 0 where the label is ``ignore_index``."""
    logits = torch.matmul(hidden, weight.t()).to(torch.float32)
    picked = torch.log_softmax(logits, dim=-1).gather(1, labels.clamp(min=0)[:, None])[:, 0]
    return torch.where(labels == ignore_index, torch.zeros_like(picked), picked)
