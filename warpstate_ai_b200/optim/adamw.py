"""AdamW over a `ParamArena`, LR schedules and gradient clipping.

Same update rule, defaults and state-dict layout as the reference's optimizer
(``torch.optim.AdamW(lr, betas=(0.9, 0.95), eps=1e-8, weight_decay, fused=True)`` on all
parameters in one group, reference run_40b.py:534-535; global-norm clip at 1.0 with a
non-finite check, run_40b.py:751), executed as three kernels over the flat arena on CUDA
(`ops/csrc/optim.cu`) and as a handful of vector ops on CPU.  The sharded forms are `parallel.zero.ShardedAdamW`
(moments per bucket slice) and `parallel.fsdp.ShardedParamAdamW` (parameters, gradients and moments per row owner).
"""
from __future__ import annotations

import math

import torch

from .arena import ParamArena


def cosine_lr(step: int, *, lr: float, min_lr: float, warmup_steps: int, total_steps: int) -> float:
    """Linear warm-up ``lr*(step+1)/warm`` then cosine to ``min_lr`` (reference run_40b.py:729-733)."""
    warm = min(warmup_steps, total_steps)
    if step < warm:
        return lr * (step + 1) / warm
    return min_lr + (lr - min_lr) * 0.5 * (1 + math.cos(math.pi * (step - warm) / max(1, total_steps - warm)))


def host_clip_stats(sumsq: torch.Tensor, max_norm: float, status: torch.Tensor | None = None) -> torch.Tensor:
    """``[norm, coef, norm^2, skip, 0, 0, 0, 0]`` from a sum of squares, as the kernels lay it out."""
    sumsq = sumsq.reshape(()).float()
    norm = sumsq.sqrt()
    coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else torch.ones_like(norm)
    bad = ~torch.isfinite(norm)
    if status is not None:
        bad = bad | (status.reshape(-1)[0] != 0)
    zero = torch.zeros_like(norm)
    return torch.stack([norm, torch.where(bad, zero, coef), sumsq, bad.float(), zero, zero, zero, zero])


def host_adamw(p, grad, m, v, lr, b1, b2, eps, weight_decay, step) -> None:
    """torch.optim.AdamW's update on flat tensors (the CPU form of `adamw_kernel`)."""
    p.mul_(1 - lr * weight_decay)
    m.lerp_(grad, 1 - b1)
    v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
    denom = (v.sqrt() / math.sqrt(1 - b2 ** step)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / (1 - b1 ** step))


class ArenaAdamW:
    def __init__(self, arena: ParamArena, lr: float = 1.5e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float | None = 1.0):
        self.arena = arena
        self.lr = lr
        self.betas = betas
        self.eps = eps
        self.weight_decay = weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.lo, self.hi = 0, arena.numel          # the range of the arena this optimizer updates: all of it
        n = self.hi - self.lo
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=arena.device)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=arena.device)
        self.last_stats: torch.Tensor | None = None  # [norm, clip_coef, norm^2] on device

    # ------------------------------------------------------------------ step
    def zero_grad(self, set_to_none: bool = False) -> None:
        self.arena.zero_grad()

    def clip_stats(self, extra_sumsq: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
        """Device statistics of the owned slice (+ ``extra_sumsq``): ``[||g||, clip coefficient, ||g||^2,
        skip, ...]``.  ``skip`` is 1 when the norm is not finite or the communication ``status`` word is
        non-zero; `step` then leaves parameters and moments untouched."""
        g = self.arena.grad[self.lo:self.hi]
        max_norm = self.max_grad_norm if self.max_grad_norm is not None else 0.0
        if g.is_cuda and _kernels():
            return torch.ops.ws_b200.grad_norm_clip(g, float(max_norm), extra_sumsq, status)
        sumsq = g.double().pow(2).sum().float()
        if extra_sumsq is not None:
            sumsq = sumsq + extra_sumsq.reshape(())
        return host_clip_stats(sumsq, max_norm, status)

    @torch.no_grad()
    def step(self, lr: float | None = None, stats: torch.Tensor | None = None) -> torch.Tensor:
        """One update.  Returns the device tensor ``[grad_norm, clip_coef, norm^2, skip, ...]``; callers that
        want the reference's ``error_if_nonfinite`` behaviour check ``stats[0]`` when they read
        the loss (one host sync per step instead of two).  When ``stats[3]`` is set nothing is changed on
        the device and the caller is expected to call `rollback_step()` when it raises."""
        if lr is not None:
            self.lr = lr
        a = self.arena
        if stats is None:
            stats = self.clip_stats()
        self.last_stats = stats
        self.step_count += 1
        b1, b2 = self.betas
        p = a.master[self.lo:self.hi]
        g = a.grad[self.lo:self.hi]
        if p.is_cuda and _kernels():
            pb = a.bf16[self.lo:self.hi] if a.bf16 is not None else None
            torch.ops.ws_b200.adamw_step(p, g, self.exp_avg, self.exp_avg_sq, pb, float(self.lr), b1, b2,
                                         self.eps, self.weight_decay, self.step_count, stats[1:2], 1.0, stats[3:4])
            return stats
        if float(stats[3]) != 0.0:
            return stats
        host_adamw(p, g * stats[1], self.exp_avg, self.exp_avg_sq, self.lr, b1, b2, self.eps, self.weight_decay,
                   self.step_count)
        if a.bf16 is not None:
            a.bf16[self.lo:self.hi].copy_(p)
        return stats

    def rollback_step(self) -> None:
        """Undo the step count of an update that the device skipped (``stats[3]`` set)."""
        self.step_count = max(0, self.step_count - 1)

    # ------------------------------------------------------------------ torch-compatible state
    def state_dict(self) -> dict:
        """Same structure as ``torch.optim.AdamW.state_dict()``: integer keys in
        ``model.parameters()`` order with ``step / exp_avg / exp_avg_sq`` and one param group."""
        a = self.arena
        state = {}
        for index, (name, _p) in enumerate(a.order):
            s = a.by_name[name]
            if self.step_count == 0:
                continue
            state[index] = {
                "step": torch.tensor(float(self.step_count)),
                "exp_avg": self.exp_avg[s.offset:s.offset + s.numel].view(s.shape).clone(),
                "exp_avg_sq": self.exp_avg_sq[s.offset:s.offset + s.numel].view(s.shape).clone(),
            }
        group = {"lr": self.lr, "betas": tuple(self.betas), "eps": self.eps, "weight_decay": self.weight_decay,
                 "amsgrad": False, "maximize": False, "foreach": None, "capturable": False,
                 "differentiable": False, "fused": True, "decoupled_weight_decay": True,
                 "params": list(range(len(a.order)))}
        return {"state": state, "param_groups": [group]}

    def load_state_dict(self, sd: dict) -> None:
        a = self.arena
        group = sd["param_groups"][0]
        self.lr = group.get("lr", self.lr)
        self.betas = tuple(group.get("betas", self.betas))
        self.eps = group.get("eps", self.eps)
        self.weight_decay = group.get("weight_decay", self.weight_decay)
        steps = set()
        self.exp_avg.zero_()
        self.exp_avg_sq.zero_()
        for index, (name, _p) in enumerate(a.order):
            entry = sd["state"].get(index)
            if entry is None:
                continue
            s = a.by_name[name]
            lo, hi = max(s.offset, self.lo), min(s.offset + s.numel, self.hi)
            if lo < hi:
                flat_m = entry["exp_avg"].reshape(-1)
                flat_v = entry["exp_avg_sq"].reshape(-1)
                self.exp_avg[lo - self.lo:hi - self.lo].copy_(flat_m[lo - s.offset:hi - s.offset])
                self.exp_avg_sq[lo - self.lo:hi - self.lo].copy_(flat_v[lo - s.offset:hi - s.offset])
            steps.add(int(float(entry["step"])))
        if len(steps) > 1:
            raise ValueError(f"optimizer state has parameters at different steps: {sorted(steps)}")
        self.step_count = steps.pop() if steps else 0


def _kernels() -> bool:
    from ..ops import _ext
    return _ext.available()
