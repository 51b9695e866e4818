"""WarpState language model.

The public surface and the state-dict keys are the reference's (warpstate/model.py:15-358), because checkpoints,
the entry points and users of ``warpstate.model`` depend on them: ``WarpStateLM(cfg)``,
``forward(input_ids, targets=None, *, return_logits=True)``, ``num_parameters()``,
``init_generation_cache(B, device, dtype)``, ``step(ids[B,1], caches)``; keys ``depth_scale, depth_bias,
embed.weight, cores.{i}.{fast_decay_logit, slow_decay_logit, memory_mix_logit, norm1.weight, in_proj.weight,
out_proj.weight, norm2.weight, ffn.up_gate.weight, ffn.down.weight}, final_norm.weight``.

The modules here hold parameters and route; the arithmetic lives elsewhere:

* `ops.reference` states every operation in plain PyTorch.  That is the model on a CPU (or on any device without the
  kernel library) and what the CUDA kernels are tested against;
* `ops.fused` is the sm_100a path, taken when the input is on a CUDA device, the kernel library is loaded and BF16
  autocast is active: one autograd node per block whose forward and backward are sequences of hand-written kernels
  (tcgen05 GEMMs with fused epilogues, chunk attention + memory, RMSNorm, LM-head cross-entropy).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..config import WarpStateConfig
from ..ops import reference as R

INIT_STD = 0.02
# One logit per head: the fast memory starts by keeping 0.90 of itself per chunk, the slow one 0.99, and a read
# weighs the two equally.
INITIAL_LOGITS = {"fast_decay_logit": math.log(0.90 / 0.10), "slow_decay_logit": math.log(0.99 / 0.01),
                  "memory_mix_logit": 0.0}


def _kernels_take(x: torch.Tensor, owner: nn.Module) -> bool:
    """The fused path handles ``x`` for ``owner`` (whose projections are whole tensors, not row-sharded layers)."""
    if not x.is_cuda or getattr(owner, "sharded_linears", False):
        return False
    from ..ops import fused
    return fused.active(x)


def _projection(inputs: int, outputs: int) -> nn.Linear:
    return nn.Linear(inputs, outputs, bias=False)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))
        self.use_fused = False      # attribute of the reference's module; the CUDA path is chosen per block, not here

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return R.rmsnorm(x, self.weight, self.eps)


class SwiGLU(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.up_gate = _projection(dim, 2 * hidden)
        self.down = _projection(hidden, dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(R.swiglu(self.up_gate(x)))


# Helper names that ``warpstate.model`` exports.
rotate_half = R.rotate_pairs
rope_cos_sin = R.rope_tables
apply_rope = R.apply_rope


@dataclass
class LayerCache:
    """What one logical depth carries between decode steps: the fast and slow memories of the finished chunks, the
    keys and values of the chunk in progress, its write so far (not yet divided by the chunk length), and how many
    positions of the chunk are filled."""
    fast_state: torch.Tensor
    slow_state: torch.Tensor
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    write_accum: torch.Tensor
    chunk_len: int = 0


class WarpStateCore(nn.Module):
    """One block: ``x + out_proj(mix(in_proj(norm1 x)))`` followed by ``x + ffn(norm2 x)``, where ``mix`` is
    chunk-local causal attention blended with a read of the fast / slow matrix memories (`ops.reference`)."""

    def __init__(self, cfg: WarpStateConfig):
        super().__init__()
        self.cfg = cfg
        self.h, self.hd, self.chunk = cfg.n_heads, cfg.head_dim, cfg.chunk_size
        width = cfg.d_model
        self.norm1 = RMSNorm(width, cfg.rms_eps)
        self.in_proj = _projection(width, 5 * width)         # Q | K | V | gate | U
        self.out_proj = _projection(width, width)
        self.norm2 = RMSNorm(width, cfg.rms_eps)
        self.ffn = SwiGLU(width, cfg.ffn_hidden)
        for name, logit in INITIAL_LOGITS.items():
            self.register_parameter(name, nn.Parameter(torch.full((self.h,), logit)))
        # The rotary tables are not part of the state dict, so a module built on the meta device (as loaders do) could
        # never fill them in afterwards: they are always computed for real.
        on_meta = torch.get_default_device().type == "meta"
        cos, sin = R.rope_tables(self.chunk, self.hd, torch.device("cpu") if on_meta else None, torch.float32)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def _memory_arguments(self):
        return (self.fast_decay_logit, self.slow_decay_logit, self.memory_mix_logit, self.h, self.chunk,
                self.cfg.parallel_memory, self.rope_cos, self.rope_sin)

    def _finish(self, x: torch.Tensor, mixed: torch.Tensor) -> torch.Tensor:
        x = x + self.out_proj(mixed)
        return x + self.ffn(self.norm2(x))

    # ------------------------------------------------------------------ whole chunks (training, prefill)
    def forward(self, x: torch.Tensor, depth_scale: torch.Tensor | None = None,
                depth_bias: torch.Tensor | None = None) -> torch.Tensor:
        """``x [B, T, d]`` with ``T`` a whole number of chunks.  ``depth_scale / depth_bias``, when given, are applied
        first (the fused path folds them into its first kernel)."""
        if x.shape[1] % self.chunk:
            raise ValueError(f"sequence length {x.shape[1]} must be divisible by chunk_size={self.chunk}")
        if _kernels_take(x, self):
            from ..ops import fused
            return fused.core_forward(self, x, depth_scale, depth_bias)
        if depth_scale is not None:
            x = x * (1.0 + depth_scale) + depth_bias
        drop = self.cfg.dropout if self.training else 0.0
        return self._finish(x, R.attention_memory(self.in_proj(self.norm1(x)), *self._memory_arguments(), dropout_p=drop))

    def forward_with_state(self, x: torch.Tensor):
        """`forward` in plain PyTorch that also returns the (fast, slow) memories after the last chunk, for a
        prefill that a decode continues (the CUDA prefill is in `serve.engine`)."""
        mixed, memories = R.attention_memory(self.in_proj(self.norm1(x)), *self._memory_arguments(), return_state=True)
        return self._finish(x, mixed), memories

    # ------------------------------------------------------------------ one position (decode)
    @torch.no_grad()
    def init_cache(self, batch_size: int, device: torch.device, dtype: torch.dtype) -> LayerCache:
        def zeros(*shape):
            return torch.zeros((batch_size, self.h, *shape), device=device, dtype=dtype)
        return LayerCache(fast_state=zeros(self.hd, self.hd), slow_state=zeros(self.hd, self.hd),
                          k_cache=zeros(self.chunk, self.hd), v_cache=zeros(self.chunk, self.hd),
                          write_accum=zeros(self.hd, self.hd), chunk_len=0)

    @torch.no_grad()
    def step(self, x: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        """``x [B, 1, d]``: the next position of every sequence; ``cache`` moves on by one position."""
        if x.shape[1] != 1:
            raise ValueError("the decode step takes exactly one position per sequence")
        batch = x.shape[0]
        packed = self.in_proj(self.norm1(x)).view(batch, 5, self.h, 1, self.hd)
        mixed, cache.chunk_len = R.decode_position(
            *packed.unbind(1), cache.k_cache, cache.v_cache, cache.write_accum, cache.fast_state, cache.slow_state,
            cache.chunk_len, self.chunk, self.fast_decay_logit, self.slow_decay_logit, self.memory_mix_logit)
        return self._finish(x, mixed.transpose(1, 2).reshape(batch, 1, self.h * self.hd))


class WarpStateLM(nn.Module):
    """Token embedding, ``logical_depth`` passes through ``n_cores`` shared blocks (block ``depth % n_cores`` at each
    depth, told apart by a learned per-depth scale and bias), a final norm and a head tied to the embedding."""

    def __init__(self, cfg: WarpStateConfig):
        super().__init__()
        cfg.validate()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.cores = nn.ModuleList(WarpStateCore(cfg) for _ in range(cfg.n_cores))
        self.depth_scale = nn.Parameter(torch.zeros(cfg.logical_depth, cfg.d_model))
        self.depth_bias = nn.Parameter(torch.zeros(cfg.logical_depth, cfg.d_model))
        self.final_norm = RMSNorm(cfg.d_model, cfg.rms_eps)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Every matrix and the embedding from ``normal(0, 0.02)``; the two projections of a block that write into
        the residual stream from a distribution narrower by ``sqrt(2 * logical_depth)``."""
        for module in self.modules():
            if isinstance(module, (nn.Linear, nn.Embedding)):
                nn.init.normal_(module.weight, mean=0.0, std=INIT_STD)
        narrow = INIT_STD / math.sqrt(2.0 * self.cfg.logical_depth)
        for core in self.cores:          # drawn again, after all the others
            for writer in (core.out_proj, core.ffn.down):
                nn.init.normal_(writer.weight, mean=0.0, std=narrow)

    def num_parameters(self) -> int:
        return sum(parameter.numel() for parameter in self.parameters())

    def _depths(self):
        """(depth index, the block that runs at that depth)."""
        return ((depth, self.cores[depth % self.cfg.n_cores]) for depth in range(self.cfg.logical_depth))

    # ------------------------------------------------------------------ trunk
    def hidden_states(self, input_ids: torch.Tensor) -> torch.Tensor:
        """``[B, T]`` token ids -> ``[B, T, d]`` after the final norm."""
        if input_ids.is_cuda and _kernels_take(self.embed.weight, self):
            from ..ops import fused
            return fused.trunk_forward(self, input_ids)
        recompute = self.training and self.cfg.gradient_checkpointing and torch.is_grad_enabled()
        x = self.embed(input_ids)
        for depth, core in self._depths():
            x = x * (1.0 + self.depth_scale[depth]) + self.depth_bias[depth]
            x = checkpoint(core, x, use_reentrant=False) if recompute else core(x)
        return self.final_norm(x)

    def logits_from_hidden(self, x: torch.Tensor) -> torch.Tensor:
        return torch.matmul(x, self.embed.weight.t())       # the head is the embedding, transposed

    def forward(self, input_ids: torch.Tensor, targets: torch.Tensor | None = None, *,
                return_logits: bool = True):
        """Three answers, as in the reference: logits when there are no ``targets``; ``(logits, mean loss)`` with
        targets; ``(None, mean loss over targets != -100)`` with ``return_logits=False``, which never builds the
        ``[tokens, vocabulary]`` matrix."""
        x = self.hidden_states(input_ids)
        if targets is None:
            return self.logits_from_hidden(x)
        if not return_logits:
            return None, self.loss_from_hidden(x, targets)
        logits = self.logits_from_hidden(x)
        return logits, nn.functional.cross_entropy(logits.flatten(0, -2), targets.flatten())

    def loss_from_hidden(self, x: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Mean cross-entropy over the labels that are not -100, a block of rows at a time.  Where every label is
        masked (a rank without supervised tokens) the result is a finite 0: sum / max(count, 1)."""
        rows, labels = x.flatten(0, -2), targets.flatten()
        counted = (labels != R.IGNORE).sum().clamp(min=1)
        if _kernels_take(rows, None):
            from ..ops import fused
            return fused.lm_head_loss(rows, self.embed.weight, labels) / counted
        block = int(getattr(self, "loss_chunk_size", self.cfg.loss_chunk_size))
        recompute = self.training and torch.is_grad_enabled()      # keep the hidden rows, not the logits, for backward
        total = torch.zeros((), dtype=torch.float32, device=x.device)
        for begin in range(0, labels.numel(), block):
            piece = (rows[begin:begin + block], self.embed.weight, labels[begin:begin + block])
            total = total + (checkpoint(R.lm_head_loss_sum, *piece, use_reentrant=False) if recompute
                             else R.lm_head_loss_sum(*piece))
        return total / counted

    def sequence_logps(self, input_ids: torch.Tensor, targets: torch.Tensor, head_chunk_size: int = 256) -> torch.Tensor:
        """``[B]`` FP32: for each sequence, the sum of the log-probabilities of its targets (positions whose target is
        -100 add nothing).  The scoring head of DPO (reference dpo.py:130-163); ``[B, T, vocabulary]`` is never held."""
        x = self.hidden_states(input_ids)
        batch, length, width = x.shape
        if _kernels_take(x, None):
            from ..ops import lmhead
            rows = x.reshape(batch * length, width).to(torch.bfloat16)
            if lmhead.kernels_ready(rows, self.embed.weight):
                return lmhead.token_logps(rows, self.embed.weight, targets.reshape(-1)).view(batch, length).sum(dim=1)

        def span_score(hidden, weight, labels):
            flat = R.lm_head_token_logps(hidden.flatten(0, 1), weight, labels.flatten())
            return flat.view(labels.shape).sum(dim=1)

        scores = torch.zeros(batch, dtype=torch.float32, device=x.device)
        for begin in range(0, length, head_chunk_size):
            span = slice(begin, begin + head_chunk_size)
            piece = (x[:, span], self.embed.weight, targets[:, span])
            scores = scores + (checkpoint(span_score, *piece, use_reentrant=False) if torch.is_grad_enabled()
                               else span_score(*piece))
        return scores

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def init_generation_cache(self, batch_size: int, device: torch.device, dtype: torch.dtype) -> List[LayerCache]:
        """One cache per logical depth: blocks are shared between depths, their decode state is not."""
        return [core.init_cache(batch_size, device, dtype) for _, core in self._depths()]

    @torch.no_grad()
    def step(self, input_ids: torch.Tensor, caches: List[LayerCache]) -> torch.Tensor:
        """``input_ids [B, 1]`` -> logits ``[B, 1, V]``; ``caches`` move on by one position."""
        x = self.embed(input_ids)
        for depth, core in self._depths():
            x = core.step(x * (1.0 + self.depth_scale[depth]) + self.depth_bias[depth], caches[depth])
        return self.logits_from_hidden(self.final_norm(x))
