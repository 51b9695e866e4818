"""WarpState language model.

Public surface and state-dict keys match the reference (warpstate/model.py:15-358):
``WarpStateLM(cfg)``, ``forward(input_ids, targets=None, *, return_logits=True)``,
``num_parameters()``, ``init_generation_cache(B, device, dtype)``, ``step(ids[B,1], caches)``;
keys ``depth_scale, depth_bias, embed.weight, cores.{i}.{fast_decay_logit, slow_decay_logit,
memory_mix_logit, norm1.weight, in_proj.weight, out_proj.weight, norm2.weight,
ffn.up_gate.weight, ffn.down.weight}, final_norm.weight``.

Two execution paths share these modules:

* the plain-PyTorch path (any device, any dtype) is the definition of the model and the oracle
  for tests; it is what runs on CPU;
* the fused sm_100a path (`ops.fused`) runs when the input is on a CUDA device, the kernel
  library is loaded and BF16 autocast is active: one autograd node per core whose forward and
  backward are sequences of hand-written kernels (tcgen05 GEMMs with fused epilogues, chunk
  attention + memory, RMSNorm, LM-head cross-entropy).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..config import WarpStateConfig
from ..ops import reference as R


def _fused_active(x: torch.Tensor) -> bool:
    if not x.is_cuda:
        return False
    from ..ops import fused
    return fused.active(x)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps
        self.use_fused = False  # kept for API parity; the CUDA path is selected by `fused.active`

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return R.rmsnorm(x, self.weight, self.eps)


# Re-exported helper names of the reference module.
rotate_half = R.rotate_pairs


def rope_cos_sin(length: int, dim: int, device: torch.device, dtype: torch.dtype):
    return R.rope_tables(length, dim, device, dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    return R.apply_rope(x, cos.view(1, 1, 1, *cos.shape), sin.view(1, 1, 1, *sin.shape))


class SwiGLU(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.up_gate = nn.Linear(dim, hidden * 2, bias=False)
        self.down = nn.Linear(hidden, dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(R.swiglu(self.up_gate(x)))


@dataclass
class LayerCache:
    """Decode state of one logical depth: two matrix memories per head, the current chunk's
    keys/values, and the running (unnormalised) write of the current chunk."""
    fast_state: torch.Tensor
    slow_state: torch.Tensor
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    write_accum: torch.Tensor
    chunk_len: int = 0


class WarpStateCore(nn.Module):
    """One block: norm -> fused Q/K/V/gate/U projection -> (chunk-local causal attention,
    fast/slow matrix-memory read) -> gated blend -> out projection -> SwiGLU FFN."""

    def __init__(self, cfg: WarpStateConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.d_model
        self.h = cfg.n_heads
        self.hd = cfg.head_dim
        self.chunk = cfg.chunk_size
        self.norm1 = RMSNorm(d, cfg.rms_eps)
        self.in_proj = nn.Linear(d, 5 * d, bias=False)
        self.out_proj = nn.Linear(d, d, bias=False)
        self.norm2 = RMSNorm(d, cfg.rms_eps)
        self.ffn = SwiGLU(d, cfg.ffn_hidden)
        self.fast_decay_logit = nn.Parameter(torch.full((self.h,), math.log(0.90 / 0.10)))
        self.slow_decay_logit = nn.Parameter(torch.full((self.h,), math.log(0.99 / 0.01)))
        self.memory_mix_logit = nn.Parameter(torch.zeros(self.h))
        # Real tables even when the module is built on the meta device (they are not in the state
        # dict, so a meta-constructed model could never fill them in).
        table_device = torch.device("cpu") if torch.get_default_device().type == "meta" else None
        cos, sin = R.rope_tables(self.chunk, self.hd, table_device, torch.float32)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    # ------------------------------------------------------------------ training / prefill
    def forward(self, x: torch.Tensor, depth_scale: torch.Tensor | None = None,
                depth_bias: torch.Tensor | None = None) -> torch.Tensor:
        """``x [B,T,d]``.  When ``depth_scale/bias`` are given the depth modulation
        ``x*(1+scale)+bias`` is applied first (the fused path folds it into its first kernel)."""
        if x.shape[1] % self.chunk != 0:
            raise ValueError(f"sequence length {x.shape[1]} must be divisible by chunk_size={self.chunk}")
        # cores whose projections were replaced by row-sharded layers (parallel/sharded_model.py) take the
        # module-by-module path: their weights are not whole tensors that the fused layer kernels could read
        if _fused_active(x) and not getattr(self, "sharded_linears", False):
            from ..ops import fused
            return fused.core_forward(self, x, depth_scale, depth_bias)
        if depth_scale is not None:
            x = x * (1.0 + depth_scale) + depth_bias
        return self._forward_torch(x)

    def _forward_torch(self, x: torch.Tensor) -> torch.Tensor:
        z = self.norm1(x)
        y = R.attention_memory(
            self.in_proj(z), self.fast_decay_logit, self.slow_decay_logit, self.memory_mix_logit,
            self.h, self.chunk, self.cfg.parallel_memory, self.rope_cos, self.rope_sin,
            dropout_p=self.cfg.dropout if self.training else 0.0)
        x = x + self.out_proj(y)
        return x + self.ffn(self.norm2(x))

    def forward_with_state(self, x: torch.Tensor):
        """Prefill helper: like ``forward`` on whole chunks, and also returns the (fast, slow)
        states after the last chunk (plain-PyTorch path; the CUDA prefill lives in serve/)."""
        z = self.norm1(x)
        y, state = R.attention_memory(
            self.in_proj(z), self.fast_decay_logit, self.slow_decay_logit, self.memory_mix_logit,
            self.h, self.chunk, self.cfg.parallel_memory, self.rope_cos, self.rope_sin,
            return_state=True)
        x = x + self.out_proj(y)
        return x + self.ffn(self.norm2(x)), state

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def init_cache(self, batch_size: int, device: torch.device, dtype: torch.dtype) -> LayerCache:
        state = (batch_size, self.h, self.hd, self.hd)
        kv = (batch_size, self.h, self.chunk, self.hd)
        z = lambda shape: torch.zeros(shape, device=device, dtype=dtype)
        return LayerCache(z(state), z(state), z(kv), z(kv), z(state), 0)

    @torch.no_grad()
    def step(self, x: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        """One token (``x [B,1,d]``) with the sequential recurrence (warpstate/model.py:222-274)."""
        assert x.shape[1] == 1
        b = x.shape[0]
        z = self.norm1(x)
        q, k, v, g, u = (t.view(b, 1, self.h, self.hd).permute(0, 2, 1, 3)
                         for t in self.in_proj(z).chunk(5, dim=-1))
        pos = cache.chunk_len
        cos, sin = R.rope_tables(pos + 1, self.hd, x.device, q.dtype)
        c = cos[pos:pos + 1].view(1, 1, 1, self.hd)
        s = sin[pos:pos + 1].view(1, 1, 1, self.hd)
        q = q * c + R.rotate_pairs(q) * s
        k = k * c + R.rotate_pairs(k) * s
        cache.k_cache[:, :, pos:pos + 1].copy_(k)
        cache.v_cache[:, :, pos:pos + 1].copy_(v)
        local = F.scaled_dot_product_attention(q, cache.k_cache[:, :, :pos + 1], cache.v_cache[:, :, :pos + 1],
                                               is_causal=False, dropout_p=0.0)
        shape = (1, self.h, 1, 1)
        fast_decay = torch.sigmoid(self.fast_decay_logit).to(q.dtype).view(shape)
        slow_decay = torch.sigmoid(self.slow_decay_logit).to(q.dtype).view(shape)
        mix = torch.sigmoid(self.memory_mix_logit).to(q.dtype).view(shape)
        read_fast = torch.matmul(q, cache.fast_state) / math.sqrt(self.hd)
        read_slow = torch.matmul(q, cache.slow_state) / math.sqrt(self.hd)
        memory = mix * read_fast + (1.0 - mix) * read_slow
        gate = torch.sigmoid(g)
        y = gate * local + (1.0 - gate) * memory
        cache.write_accum.add_(torch.matmul(torch.tanh(k).transpose(-2, -1), torch.tanh(u)))
        y = y.permute(0, 2, 1, 3).contiguous().view(b, 1, self.cfg.d_model)
        x = x + self.out_proj(y)
        x = x + self.ffn(self.norm2(x))
        if pos + 1 == self.chunk:
            write = cache.write_accum / float(self.chunk)
            cache.fast_state.mul_(fast_decay).add_(write * (1.0 - fast_decay))
            cache.slow_state.mul_(slow_decay).add_(write * (1.0 - slow_decay))
            cache.k_cache.zero_()
            cache.v_cache.zero_()
            cache.write_accum.zero_()
            cache.chunk_len = 0
        else:
            cache.chunk_len = pos + 1
        return x


class WarpStateLM(nn.Module):
    def __init__(self, cfg: WarpStateConfig):
        super().__init__()
        cfg.validate()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.cores = nn.ModuleList([WarpStateCore(cfg) for _ in range(cfg.n_cores)])
        self.depth_scale = nn.Parameter(torch.zeros(cfg.logical_depth, cfg.d_model))
        self.depth_bias = nn.Parameter(torch.zeros(cfg.logical_depth, cfg.d_model))
        self.final_norm = RMSNorm(cfg.d_model, cfg.rms_eps)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """normal(0, 0.02) for matrices and the embedding; residual-writing projections are
        scaled by 1/sqrt(2*logical_depth) (warpstate/model.py:291-304)."""
        for module in self.modules():
            if isinstance(module, (nn.Linear, nn.Embedding)):
                nn.init.normal_(module.weight, mean=0.0, std=0.02)
        scale = 1.0 / math.sqrt(2.0 * self.cfg.logical_depth)
        for core in self.cores:
            nn.init.normal_(core.out_proj.weight, mean=0.0, std=0.02 * scale)
            nn.init.normal_(core.ffn.down.weight, mean=0.0, std=0.02 * scale)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    # ------------------------------------------------------------------ trunk
    def hidden_states(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Embedding, all logical depths and the final norm: ``[B,T] -> [B,T,d]``."""
        if _fused_active(self.embed.weight) and input_ids.is_cuda and not getattr(self, "sharded_linears", False):
            from ..ops import fused
            return fused.trunk_forward(self, input_ids)
        x = self.embed(input_ids)
        for depth in range(self.cfg.logical_depth):
            core = self.cores[depth % self.cfg.n_cores]
            x = x * (1.0 + self.depth_scale[depth]) + self.depth_bias[depth]
            if self.training and self.cfg.gradient_checkpointing and torch.is_grad_enabled():
                x = checkpoint(core, x, use_reentrant=False)
            else:
                x = core(x)
        return self.final_norm(x)

    def forward(self, input_ids: torch.Tensor, targets: torch.Tensor | None = None, *,
                return_logits: bool = True):
        x = self.hidden_states(input_ids)
        if targets is not None and not return_logits:
            return None, self.loss_from_hidden(x, targets)
        logits = self.logits_from_hidden(x)
        if targets is None:
            return logits
        loss = F.cross_entropy(logits.reshape(-1, logits.size(-1)), targets.reshape(-1))
        return logits, loss

    def logits_from_hidden(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.embed.weight)  # tied head

    def loss_from_hidden(self, x: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Mean cross-entropy over labels != -100 without keeping ``[tokens, vocab]`` logits.
        A rank whose labels are all masked gets a finite 0 (sum / max(count, 1))."""
        hidden = x.reshape(-1, x.size(-1))
        labels = targets.reshape(-1)
        count = labels.ne(-100).sum().clamp_min(1)
        if _fused_active(hidden):
            from ..ops import fused
            return fused.lm_head_loss(hidden, self.embed.weight, labels) / count
        rows = int(getattr(self, "loss_chunk_size", self.cfg.loss_chunk_size))
        total = x.new_zeros((), dtype=torch.float32)
        recompute = self.training and torch.is_grad_enabled()
        for start in range(0, labels.numel(), rows):
            h, y = hidden[start:start + rows], labels[start:start + rows]
            if recompute:
                total = total + checkpoint(R.lm_head_loss_sum, h, self.embed.weight, y, use_reentrant=False)
            else:
                total = total + R.lm_head_loss_sum(h, self.embed.weight, y)
        return total / count

    def sequence_logps(self, input_ids: torch.Tensor, targets: torch.Tensor, head_chunk_size: int = 256) -> torch.Tensor:
        """Per-sequence sum of label log-probabilities over positions whose target is not -100
        (FP32, ``[B]``), without keeping ``[B, T, vocab]`` logits: the scoring head of DPO
        (reference dpo.py:130-163)."""
        x = self.hidden_states(input_ids)
        b, t, d = x.shape
        if _fused_active(x):
            from ..ops import lmhead
            hidden = x.reshape(b * t, d)
            if hidden.dtype != torch.bfloat16:
                hidden = hidden.to(torch.bfloat16)
            if lmhead.kernels_ready(hidden, self.embed.weight):
                return lmhead.token_logps(hidden, self.embed.weight, targets.reshape(-1)).view(b, t).sum(dim=1)

        def score(h, weight, labels):
            return R.lm_head_token_logps(h.reshape(-1, h.size(-1)), weight, labels.reshape(-1)).view(labels.shape).sum(dim=1)

        logps = x.new_zeros((b,), dtype=torch.float32)
        for start in range(0, t, head_chunk_size):
            args = (x[:, start:start + head_chunk_size], self.embed.weight, targets[:, start:start + head_chunk_size])
            logps = logps + (checkpoint(score, *args, use_reentrant=False) if torch.is_grad_enabled() else score(*args))
        return logps

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def init_generation_cache(self, batch_size: int, device: torch.device, dtype: torch.dtype) -> List[LayerCache]:
        return [self.cores[depth % self.cfg.n_cores].init_cache(batch_size, device, dtype)
                for depth in range(self.cfg.logical_depth)]

    @torch.no_grad()
    def step(self, input_ids: torch.Tensor, caches: List[LayerCache]) -> torch.Tensor:
        """``input_ids [B,1]`` -> logits ``[B,1,V]``; caches are updated in place."""
        x = self.embed(input_ids)
        for depth in range(self.cfg.logical_depth):
            x = x * (1.0 + self.depth_scale[depth]) + self.depth_bias[depth]
            x = self.cores[depth % self.cfg.n_cores].step(x, caches[depth])
        return F.linear(self.final_norm(x), self.embed.weight)
