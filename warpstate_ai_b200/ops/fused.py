"""Fused sm_100a execution of the WarpState trunk.

One autograd node per core (`CoreFn`): its forward and backward are explicit sequences of the
kernels in csrc/ -- tcgen05 GEMMs with fused epilogues, RMSNorm (with the depth modulation
folded in), chunk attention + matrix-memory kernels -- so there is no per-op autograd graph,
no separate residual adds, SwiGLU passes, gradient casts or weight-gradient accumulations.

What the reference runs as separate library / Inductor kernels and where it went
(warpstate/model.py:114-178 is the math being executed):

* norm1 + depth modulation          -> rmsnorm_fwd (one pass, emits BF16 activations + rstd)
* in_proj                            -> gemm (BF16 epilogue)
* chunkify, RoPE, SDPA, tanh writes, decay scan, memory read, gate blend
                                     -> attention kernels (ops/attention.py)
* out_proj + residual                -> gemm (residual epilogue, FP32 stream)
* norm2                              -> rmsnorm_fwd
* up_gate + SwiGLU                   -> gemm (paired SwiGLU epilogue)
* down + residual                    -> gemm (residual epilogue)
* backward: dX GEMMs (MN-major weight reads, SwiGLU-backward epilogue), dW GEMMs that
  accumulate in FP32 straight into the parameter's gradient buffer, rmsnorm_bwd that also
  adds the residual-stream gradient and emits the BF16 copy the next GEMM needs.

Weight gradients: when a parameter carries ``main_grad`` (set by `optim.ParamArena`) the dW GEMM
accumulates into it and autograd sees no gradient for that parameter; otherwise a fresh FP32
gradient is returned to autograd.
"""
from __future__ import annotations

import contextlib
import os

import torch
import torch.nn.functional as F

from . import _ext
from . import gemm as G
from . import reference as R

_enabled = os.environ.get("WARPSTATE_DISABLE_KERNELS", "0") != "1"


def active(x: torch.Tensor) -> bool:
    """Fused path is used for CUDA tensors under BF16 autocast when the library is present."""
    if not (_enabled and x.is_cuda):
        return False
    if not torch.is_autocast_enabled("cuda") or torch.get_autocast_dtype("cuda") != torch.bfloat16:
        return False
    return _ext.available()


@contextlib.contextmanager
def disabled():
    """Run the plain-PyTorch path (oracle) even on a CUDA device."""
    global _enabled
    old = _enabled
    _enabled = False
    try:
        yield
    finally:
        _enabled = old


def _ops():
    return torch.ops.ws_b200


_core_grad_hook = None


def set_core_grad_hook(fn) -> None:
    """``fn(core)`` is called when a core's weight gradients are final for this backward pass
    (used by the gradient synchroniser to start reducing that core's bucket early)."""
    global _core_grad_hook
    _core_grad_hook = fn


# --------------------------------------------------------------------------- BF16 weight views
def bf16_weight(p: torch.Tensor) -> torch.Tensor:
    """BF16 copy of an FP32 master weight.

    `optim.ParamArena` keeps a persistent BF16 mirror that the optimizer kernel refreshes
    (``p.bf16_view``); without it the cast is done here and cached until the parameter's
    version counter changes (the reference re-casts every micro-batch under autocast).
    """
    view = getattr(p, "bf16_view", None)
    if view is not None:
        return view
    if p.dtype == torch.bfloat16:
        return p.detach()
    cached = getattr(p, "_ws_cast", None)
    if cached is not None and cached[0] == p._version and cached[1].device == p.device:
        return cached[1]
    w = _ops().cast_bf16(p.detach().contiguous(), None)
    p._ws_cast = (p._version, w)
    return w


def _wgrad_group(items):
    """``items`` = [(dy, x, param), ...] -> list of gradients for autograd (None where the result
    was accumulated into ``param.main_grad``).  All products run as one grouped launch."""
    work, results = [], []
    for dy, x, p in items:
        main = getattr(p, "main_grad", None)
        if main is not None:
            work.append((dy, x, main, True))
            results.append(None)
        else:
            grad = torch.empty(p.shape, dtype=torch.float32, device=p.device)
            work.append((dy, x, grad, False))
            results.append((grad, p.dtype))
    G.grad_weight_accumulate_group(work)
    return [None if r is None else r[0].to(r[1]) for r in results]


# --------------------------------------------------------------------------- attention hook
def _attention_forward(qkvgu: torch.Tensor, core, batch: int, seq: int):
    """qkvgu [M,5d] BF16 -> (y [M,d] BF16, saved-for-backward)."""
    from . import attention
    if attention.kernels_ready(core):
        return attention.forward(qkvgu, core, batch, seq)
    with torch.no_grad():
        y = R.attention_memory(qkvgu.view(batch, seq, -1), core.fast_decay_logit, core.slow_decay_logit,
                               core.memory_mix_logit, core.h, core.chunk, core.cfg.parallel_memory,
                               core.rope_cos, core.rope_sin)
    return y.reshape(batch * seq, -1).contiguous(), None


def _attention_backward(dy: torch.Tensor, qkvgu: torch.Tensor, saved, core, batch: int, seq: int):
    """-> (dqkvgu [M,5d] BF16, d_fast_logit, d_slow_logit, d_mix_logit)."""
    from . import attention
    if attention.kernels_ready(core):
        return attention.backward(dy, qkvgu, saved, core, batch, seq)
    with torch.enable_grad():
        leaf = qkvgu.detach().view(batch, seq, -1).requires_grad_(True)
        logits = [t.detach().requires_grad_(True) for t in
                  (core.fast_decay_logit, core.slow_decay_logit, core.memory_mix_logit)]
        y = R.attention_memory(leaf, logits[0], logits[1], logits[2], core.h, core.chunk,
                               core.cfg.parallel_memory, core.rope_cos, core.rope_sin)
        grads = torch.autograd.grad(y, [leaf] + logits, dy.view(batch, seq, -1))
    return grads[0].reshape(batch * seq, -1).contiguous(), grads[1], grads[2], grads[3]


_SIDE_STREAMS: dict = {}


def _side_stream(device: torch.device):
    """The per-device second stream for small bandwidth-bound kernels that overlap a GEMM
    (``WARPSTATE_SIDE_STREAM=0`` keeps everything on one stream)."""
    if device.type != "cuda" or os.environ.get("WARPSTATE_SIDE_STREAM", "1") == "0":
        return None
    key = device.index if device.index is not None else torch.cuda.current_device()
    stream = _SIDE_STREAMS.get(key)
    if stream is None:
        stream = _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return stream


# --------------------------------------------------------------------------- projection weights
class LocalWeights:
    """BF16 compute copies of a core's four projection weights when they are whole on this rank.
    `parallel.fsdp.CoreWeights` offers the same calls for row-sharded weights (gathers included)."""

    def __init__(self, w_in, w_out, w_ug, w_down):
        self.w = (w_in, w_out, w_ug, w_down)

    def begin_forward(self) -> None:
        pass

    def in_proj(self, z):
        return G.linear(z, bf16_weight(self.w[0]))

    def up_gate(self, z):
        return G.linear_swiglu(z, bf16_weight(self.w[2]))

    def out_w(self):
        return bf16_weight(self.w[1])

    def down_w(self):
        return bf16_weight(self.w[3])

    def end_forward(self) -> None:
        pass

    def begin_backward(self) -> None:
        pass

    def backward_weights(self):
        return tuple(bf16_weight(w) for w in self.w)

    def end_backward(self) -> None:
        pass


def _weights_of(core, params):
    sharded = getattr(core, "ws_weights", None)
    return sharded if sharded is not None else LocalWeights(*params)


# --------------------------------------------------------------------------- one core
def _core_kernels(core, weights, x_in, scale, bias, n1w, n2w, batch, seq, want_output=True):
    """The forward kernel sequence of one core on ``x_in [M, d]`` (FP32 or BF16 residual stream).
    Returns every tensor the backward pass reads, and ``x3`` (None when ``want_output`` is False: the
    recomputation inside a checkpointed backward stops before the down projection)."""
    ops = _ops()
    has_mod = scale is not None
    weights.begin_forward()
    z1, rstd1, xmod = ops.rmsnorm_fwd(x_in, scale, bias, n1w, core.cfg.rms_eps, True)
    qkvgu = weights.in_proj(z1)
    y, attn_saved = _attention_forward(qkvgu, core, batch, seq)
    x2 = G.linear_residual(y, weights.out_w(), xmod)
    z2, rstd2, _ = ops.rmsnorm_fwd(x2, None, None, n2w, core.cfg.rms_eps, False)
    packed, act = weights.up_gate(z2)
    x3 = G.linear_residual(act, weights.down_w(), x2) if want_output else None
    weights.end_forward()
    return (xmod if has_mod else x_in, rstd1, z1, qkvgu, y, x2, rstd2, z2, packed, act, attn_saved), x3


class CoreFn(torch.autograd.Function):
    """One core as one autograd node.  ``checkpoint=True`` keeps only the core's input (and the small
    vectors) for the backward pass and re-runs the forward kernels there -- the fused counterpart of the
    reference's per-core ``torch.utils.checkpoint`` (warpstate/model.py:310-313)."""

    @staticmethod
    def forward(ctx, x, depth_scale, depth_bias, n1w, w_in, w_out, n2w, w_ug, w_down, fast_logit,
                slow_logit, mix_logit, core, notify=True, checkpoint=False):
        batch, seq, d = x.shape
        m = batch * seq
        x_in = x.reshape(m, d)
        if not x_in.is_contiguous():
            x_in = x_in.contiguous()
        has_mod = depth_scale is not None
        scale = depth_scale.detach().float().contiguous() if has_mod else None
        bias = depth_bias.detach().float().contiguous() if has_mod else None
        n1 = n1w.detach().float()
        n2 = n2w.detach().float()
        weights = _weights_of(core, (w_in, w_out, w_ug, w_down))
        saved, x3 = _core_kernels(core, weights, x_in, scale, bias, n1, n2, batch, seq)
        xmod, rstd1, z1, qkvgu, y, x2, rstd2, z2, packed, act, attn_saved = saved
        ctx.core = core
        ctx.notify = notify
        ctx.dims = (batch, seq, d)
        ctx.has_mod = has_mod
        ctx.checkpoint = bool(checkpoint)
        ctx.params = (w_in, w_out, w_ug, w_down)
        dummy = rstd1
        if ctx.checkpoint:
            ctx.attn_saved = None
            ctx.save_for_backward(x_in, scale if has_mod else dummy, bias if has_mod else dummy, n1w, n2w)
        else:
            ctx.attn_saved = attn_saved
            ctx.save_for_backward(x_in if has_mod else xmod, xmod, rstd1, z1, qkvgu, y, x2, rstd2, z2, packed, act,
                                  scale if has_mod else dummy, n1w, n2w)
        return x3.view(batch, seq, d)

    @staticmethod
    def backward(ctx, dx3):
        ops = _ops()
        core = ctx.core
        batch, seq, d = ctx.dims
        m = batch * seq
        w_in, w_out, w_ug, w_down = ctx.params
        weights = _weights_of(core, ctx.params)
        weights.begin_backward()
        if ctx.checkpoint:
            x_in, scale, bias, n1w, n2w = ctx.saved_tensors
            with torch.no_grad():
                saved, _ = _core_kernels(core, weights, x_in, scale if ctx.has_mod else None,
                                         bias if ctx.has_mod else None, n1w.detach().float(), n2w.detach().float(),
                                         batch, seq, want_output=False)
            xmod, rstd1, z1, qkvgu, y, x2, rstd2, z2, packed, act, attn_saved = saved
        else:
            x_in, xmod, rstd1, z1, qkvgu, y, x2, rstd2, z2, packed, act, scale, n1w, n2w = ctx.saved_tensors
            attn_saved = ctx.attn_saved
        bw_in, bw_out, bw_ug, bw_down = weights.backward_weights()
        dx3 = dx3.reshape(m, d)
        if not dx3.is_contiguous():
            dx3 = dx3.contiguous()
        stream_bf16 = dx3.dtype == torch.bfloat16
        # ---- FFN
        dx3b = dx3 if stream_bf16 else ops.cast_bf16(dx3, None)
        dpacked = G.grad_input_swiglu(dx3b, bw_down, packed)
        dz2 = G.grad_input(dpacked, bw_ug)
        dx2, dx2b, g_n2 = ops.rmsnorm_bwd(dz2, x2, rstd2, n2w.detach().float(), dx3, None, not stream_bf16)
        if stream_bf16:
            dx2b = dx2
        del dz2
        # ---- attention / memory
        dy = G.grad_input(dx2b, bw_out)
        dqkvgu, g_fast, g_slow, g_mix = _attention_backward(dy, qkvgu, attn_saved, core, batch, seq)
        del dy
        dz1 = G.grad_input(dqkvgu, bw_in)
        dx_in, _, g_n1 = ops.rmsnorm_bwd(dz1, xmod, rstd1, n1w.detach().float(), dx2, scale if ctx.has_mod else None, False)
        g_scale = g_bias = None
        side = _side_stream(dx_in.device) if ctx.has_mod else None
        if ctx.has_mod:
            # d bias = colsum(d x_mod), d scale = colsum(d x_mod * x_in), with d x_mod = dx_in / (1+scale).
            # Bandwidth-bound and independent of the weight gradients: it runs on a second stream under
            # the grouped dW launch below, whose CTAs leave room for it on every SM.
            if side is not None:
                main = torch.cuda.current_stream(dx_in.device)
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    g_bias, g_scale = ops.colsum2(dx_in, x_in, scale)
                for t in (g_bias, g_scale, dx_in, x_in, scale):
                    t.record_stream(side)
            else:
                g_bias, g_scale = ops.colsum2(dx_in, x_in, scale)
        # ---- the four weight gradients, deferred to one grouped launch (their tiles share waves)
        g_down, g_ug, g_out, g_in = _wgrad_group([(dx3b, act, w_down), (dpacked, z2, w_ug), (dx2b, y, w_out),
                                                  (dqkvgu, z1, w_in)])
        del dpacked, dqkvgu
        weights.end_backward()
        if side is not None:
            torch.cuda.current_stream(dx_in.device).wait_stream(side)
        if ctx.notify and _core_grad_hook is not None:
            _attach_small_grads(core, g_n1, g_n2, g_fast, g_slow, g_mix)
            _core_grad_hook(core)
            g_n1 = g_n2 = g_fast = g_slow = g_mix = None
        return (dx_in.view(batch, seq, d), g_scale, g_bias, g_n1, g_in, g_out, g_n2, g_ug, g_down,
                g_fast, g_slow, g_mix, None, None, None)


def _attach_small_grads(core, g_n1, g_n2, g_fast, g_slow, g_mix) -> None:
    """Add the core's small-parameter gradients to the arena now (instead of letting autograd do
    it after this node returns) so that the whole bucket is final when the hook fires."""
    pairs = ((core.norm1.weight, g_n1), (core.norm2.weight, g_n2), (core.fast_decay_logit, g_fast),
             (core.slow_decay_logit, g_slow), (core.memory_mix_logit, g_mix))
    for p, g in pairs:
        if g is None:
            continue
        main = getattr(p, "main_grad", None)
        if main is None:
            raise RuntimeError("core gradient hook requires parameters bound to a ParamArena")
        main.add_(g.to(main.dtype))


def core_forward(core, x: torch.Tensor, depth_scale=None, depth_bias=None, notify: bool = True,
                 checkpoint: bool = False) -> torch.Tensor:
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    return CoreFn.apply(x, depth_scale, depth_bias, core.norm1.weight, core.in_proj.weight,
                        core.out_proj.weight, core.norm2.weight, core.ffn.up_gate.weight,
                        core.ffn.down.weight, core.fast_decay_logit, core.slow_decay_logit,
                        core.memory_mix_logit, core, notify, checkpoint)


# --------------------------------------------------------------------------- embedding / final norm
class EmbedFn(torch.autograd.Function):
    """Embedding rows into the residual stream: FP32 by default, BF16 when the model runs with a BF16
    residual stream (the reference's ``apply_bf16_residuals``, ops/residual_experiment.py:25-58, which
    casts the embedding and the depth modulation so that every residual add rounds to BF16)."""

    @staticmethod
    def forward(ctx, ids, table, out_bf16=False):
        ctx.save_for_backward(ids)
        ctx.table = table
        out = _ops().embed_fwd(ids.reshape(-1).contiguous(), table.detach(), bool(out_bf16))
        return out.view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dx):
        (ids,) = ctx.saved_tensors
        table = ctx.table
        d = table.shape[1]
        dx = dx.reshape(-1, d).contiguous()
        main = getattr(table, "main_grad", None)
        if main is not None:
            _ops().embed_bwd(dx, ids, main)
            return None, None, None
        grad = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        _ops().embed_bwd(dx, ids, grad)
        return None, grad.to(table.dtype), None


class NormFn(torch.autograd.Function):
    """Standalone RMSNorm (final norm): FP32/BF16 stream in, BF16 activations out."""

    @staticmethod
    def forward(ctx, x, w, eps):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        z, rstd, _ = _ops().rmsnorm_fwd(x2, None, None, w.detach().float(), eps, False)
        ctx.save_for_backward(x2, rstd, w)
        ctx.shape = shape
        return z.view(shape)

    @staticmethod
    def backward(ctx, dz):
        x2, rstd, w = ctx.saved_tensors
        dz = dz.reshape(x2.shape)
        if dz.dtype != torch.bfloat16:
            dz = dz.to(torch.bfloat16)
        dx, _, dw = _ops().rmsnorm_bwd(dz.contiguous(), x2, rstd, w.detach().float(), None, None, False)
        return dx.view(ctx.shape), dw, None


def trunk_forward(model, input_ids: torch.Tensor) -> torch.Tensor:
    """Embedding -> logical depths -> final norm; returns BF16 hidden states ``[B,T,d]``.

    ``model.bf16_residuals`` selects a BF16 residual stream; ``cfg.gradient_checkpointing`` (while training
    with gradients enabled) keeps only each core's input and recomputes the core in its backward."""
    cfg = model.cfg
    x = EmbedFn.apply(input_ids, model.embed.weight, bool(getattr(model, "bf16_residuals", False)))
    checkpoint = bool(cfg.gradient_checkpointing and model.training and torch.is_grad_enabled())
    for depth in range(cfg.logical_depth):
        core = model.cores[depth % cfg.n_cores]
        # the first forward use of a (possibly shared) core is its last use in backward
        x = core_forward(core, x, model.depth_scale[depth], model.depth_bias[depth], notify=depth < cfg.n_cores,
                         checkpoint=checkpoint)
    return NormFn.apply(x, model.final_norm.weight, cfg.rms_eps)


# --------------------------------------------------------------------------- LM head + CE
_LM_ROWS = 8192


class LMHeadLossFn(torch.autograd.Function):
    """Sum over valid rows of CE(hidden @ W.T, labels) without keeping [tokens, vocab] logits.

    Forward and backward walk over row blocks; the backward recomputes the block's logits,
    forms ``softmax - onehot`` in BF16 and feeds the dX / dW GEMMs (dW accumulates in FP32
    into the tied embedding's gradient).  Same contract as the reference's checkpointed and
    full losses (warpstate/model.py:316-334, ops/loss_experiment.py:14-19).
    """

    @staticmethod
    def forward(ctx, hidden, weight, labels):
        hidden = hidden.contiguous()
        wb = bf16_weight(weight)
        total = torch.zeros((), dtype=torch.float32, device=hidden.device)
        lse_all = torch.empty(hidden.shape[0], dtype=torch.float32, device=hidden.device)
        for start in range(0, hidden.shape[0], _LM_ROWS):
            h = hidden[start:start + _LM_ROWS]
            y = labels[start:start + _LM_ROWS]
            logits = G.linear(h, wb).float()
            lse = torch.logsumexp(logits, dim=-1)
            lse_all[start:start + _LM_ROWS] = lse
            valid = y.ne(-100)
            picked = logits.gather(1, y.clamp_min(0).unsqueeze(1)).squeeze(1)
            total = total + ((lse - picked) * valid).sum()
        ctx.save_for_backward(hidden, labels, lse_all)
        ctx.weight = weight
        return total

    @staticmethod
    def backward(ctx, grad_out):
        hidden, labels, lse_all = ctx.saved_tensors
        weight = ctx.weight
        wb = bf16_weight(weight)
        dh = torch.empty_like(hidden)
        main = getattr(weight, "main_grad", None)
        grad_w = main if main is not None else torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        for start in range(0, hidden.shape[0], _LM_ROWS):
            h = hidden[start:start + _LM_ROWS]
            y = labels[start:start + _LM_ROWS]
            logits = G.linear(h, wb).float()
            p = torch.exp(logits - lse_all[start:start + _LM_ROWS].unsqueeze(1))
            valid = y.ne(-100)
            p.scatter_add_(1, y.clamp_min(0).unsqueeze(1), -torch.ones_like(p[:, :1]))
            p.mul_((valid * grad_out).unsqueeze(1))
            dlogits = p.to(torch.bfloat16)
            G.grad_input(dlogits, wb, out=dh[start:start + _LM_ROWS])
            G.grad_weight_accumulate(dlogits, h, grad_w, accumulate=True)
        return dh, (None if main is not None else grad_w.to(weight.dtype)), None


def lm_head_loss(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    if hidden.dtype != torch.bfloat16:
        hidden = hidden.to(torch.bfloat16)
    from . import lmhead
    if lmhead.kernels_ready(hidden, weight):
        return lmhead.loss_sum(hidden, weight, labels)
    return LMHeadLossFn.apply(hidden, weight, labels)


# --------------------------------------------------------------------------- prefill
@torch.no_grad()
def core_prefill(core, x: torch.Tensor, depth_scale, depth_bias):
    """Forward of one core over whole chunks that also returns the fast / slow memory states
    after the last chunk (FP32 ``[B,H,64,64]``): the chunked prefill of the decode engine."""
    from . import attention
    ops = _ops()
    batch, seq, d = x.shape
    x_in = x.reshape(batch * seq, d).contiguous()
    scale = depth_scale.detach().float().contiguous()
    bias = depth_bias.detach().float().contiguous()
    z1, _, xmod = ops.rmsnorm_fwd(x_in, scale, bias, core.norm1.weight.detach().float(), core.cfg.rms_eps, True)
    qkvgu = G.linear(z1, bf16_weight(core.in_proj.weight))
    if attention.geometry_ok(core):
        y, _, _, (fast, slow) = attention.forward_only(qkvgu, core, batch, seq, want_final=True)
    else:
        y, (fast, slow) = R.attention_memory(qkvgu.view(batch, seq, -1), core.fast_decay_logit, core.slow_decay_logit,
                                             core.memory_mix_logit, core.h, core.chunk, core.cfg.parallel_memory,
                                             core.rope_cos, core.rope_sin, return_state=True)
        y = y.reshape(batch * seq, -1).contiguous()
    x2 = G.linear_residual(y, bf16_weight(core.out_proj.weight), xmod)
    z2, _, _ = ops.rmsnorm_fwd(x2, None, None, core.norm2.weight.detach().float(), core.cfg.rms_eps, False)
    _, act = G.linear_swiglu(z2, bf16_weight(core.ffn.up_gate.weight))
    x3 = G.linear_residual(act, bf16_weight(core.ffn.down.weight), x2)
    return x3.view(batch, seq, d), fast, slow
