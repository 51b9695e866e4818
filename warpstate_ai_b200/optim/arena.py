"""Flat parameter arena: FP32 master weights, FP32 gradients, BF16 compute mirror.

All parameters of a model are re-homed as views into one contiguous FP32 buffer (``master``);
their gradients are views into a second buffer (``grad``) and a BF16 mirror of the weights
lives in a third (``bf16``).  This is what lets the framework

* accumulate weight gradients in FP32 directly from the dW GEMM epilogue (``p.main_grad``),
* run clip + AdamW + BF16 re-cast as three kernels over the whole model,
* hand contiguous, fixed-address ranges ("buckets") to the gradient reduce kernels, and
* shard optimizer state by slicing one flat index space.

The precision contract of the reference is kept: FP32 master parameters, FP32 gradients, FP32
AdamW moments, BF16 compute copies (reference run_40b.py:523,534-535,744).

Layout: parameters are laid out in *bucket order* -- the order in which their gradients become
final during backward, reversed -- so that a bucket is one contiguous range: the "tail" group
(embedding, depth modulation, final norm: final only at the very end of backward) first, then
core 0 .. core n-1.  Backward finishes core n-1 first, so buckets complete from the end of the
buffer towards its start.  `order` keeps the model's ``parameters()`` order for checkpoint and
optimizer-state compatibility.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

import torch

ALIGN = 256  # elements; keeps every parameter 1 KiB-aligned in FP32 and 512 B-aligned in BF16


@dataclass
class Slot:
    name: str
    param: torch.nn.Parameter
    offset: int
    numel: int
    shape: torch.Size
    bucket: int


@dataclass
class Bucket:
    index: int
    start: int  # element offset in the arena (inclusive)
    stop: int   # exclusive, padded to ALIGN
    names: list


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def default_groups(model: torch.nn.Module, bucket_cap_bytes: int = 0) -> list[list[tuple[str, torch.nn.Parameter]]]:
    """Group named parameters by gradient-readiness: tail group first, then one group per core.  With a
    positive ``bucket_cap_bytes`` consecutive cores share a group while their FP32 gradients fit the cap
    (what a DDP bucket cap does for small models, reference ops/distributed_execution.py:16-79); a core
    larger than the cap stays one group and is split at reduction time by the synchroniser."""
    named = list(model.named_parameters())
    cores: dict[int, list] = {}
    tail = []
    for name, p in named:
        if name.startswith("cores."):
            cores.setdefault(int(name.split(".")[1]), []).append((name, p))
        else:
            tail.append((name, p))
    groups = [tail] if tail else []
    open_group, open_bytes = None, 0
    for index in sorted(cores):
        size = 4 * sum(_round_up(p.numel(), ALIGN) for _, p in cores[index])
        if open_group is not None and bucket_cap_bytes > 0 and open_bytes + size <= bucket_cap_bytes:
            open_group.extend(cores[index])
            open_bytes += size
        else:
            open_group, open_bytes = list(cores[index]), size
            groups.append(open_group)
    return groups


class ParamArena:
    def __init__(self, model: torch.nn.Module, device: torch.device | None = None,
                 bf16_mirror: bool | None = None, groups=None, symmetric_alloc=None, bucket_cap_bytes: int = 0):
        params = list(model.parameters())
        if not params:
            raise ValueError("model has no parameters")
        self.device = device or params[0].device
        self.order = list(model.named_parameters())
        groups = groups if groups is not None else default_groups(model, bucket_cap_bytes)
        self.slots: list[Slot] = []
        self.buckets: list[Bucket] = []
        offset = 0
        seen = set()
        for b, group in enumerate(groups):
            start = offset
            names = []
            for name, p in group:
                if id(p) in seen:
                    continue
                seen.add(id(p))
                self.slots.append(Slot(name, p, offset, p.numel(), p.shape, b))
                names.append(name)
                offset = _round_up(offset + p.numel(), ALIGN)
            self.buckets.append(Bucket(b, start, offset, names))
        if len(seen) != len({id(p) for p in params}):
            raise ValueError("parameter groups do not cover the model")
        self.numel = offset
        self.by_name = {s.name: s for s in self.slots}
        alloc = symmetric_alloc or (lambda n, dtype: torch.zeros(n, dtype=dtype, device=self.device))
        self.master = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        self.grad = alloc(self.numel, torch.float32)
        if bf16_mirror is None:
            bf16_mirror = self.device.type == "cuda"
        self.bf16 = torch.zeros(self.numel, dtype=torch.bfloat16, device=self.device) if bf16_mirror else None
        with torch.no_grad():
            for s in self.slots:
                view = self.master[s.offset:s.offset + s.numel].view(s.shape)
                view.copy_(s.param.detach().to(self.device, torch.float32))
                s.param.data = view
        self.bind_grads()
        self.refresh_bf16()

    # ------------------------------------------------------------------ views
    def view(self, buffer: torch.Tensor, slot: Slot) -> torch.Tensor:
        return buffer[slot.offset:slot.offset + slot.numel].view(slot.shape)

    def bind_grads(self) -> None:
        """(Re)attach ``p.grad`` / ``p.main_grad`` / ``p.bf16_view`` to the arena views."""
        for s in self.slots:
            g = self.view(self.grad, s)
            s.param.grad = g
            s.param.main_grad = g
            if self.bf16 is not None:
                s.param.bf16_view = self.view(self.bf16, s)

    def adopt_master(self, tensor: torch.Tensor) -> None:
        """Move the FP32 master weights into ``tensor`` (e.g. symmetric memory) and re-point every
        parameter at its new storage."""
        if tensor.numel() != self.numel or tensor.dtype != torch.float32:
            raise ValueError("replacement master buffer has the wrong size or dtype")
        with torch.no_grad():
            tensor.copy_(self.master)
            self.master = tensor
            for s in self.slots:
                s.param.data = self.view(self.master, s)

    def zero_grad(self) -> None:
        self.grad.zero_()

    def refresh_bf16(self) -> None:
        if self.bf16 is None:
            return
        if self.master.is_cuda:
            torch.ops.ws_b200.cast_bf16(self.master, self.bf16) if _kernels() else self.bf16.copy_(self.master)
        else:
            self.bf16.copy_(self.master)

    def collect_stray_grads(self) -> None:
        """Fold gradients that autograd placed outside the arena (a fresh ``p.grad`` tensor)
        back into it.  Happens only if user code replaced ``p.grad``."""
        for s in self.slots:
            g = s.param.grad
            target = self.view(self.grad, s)
            if g is not None and g.data_ptr() != target.data_ptr():
                target.add_(g.to(target.dtype))
                s.param.grad = target

    # ------------------------------------------------------------------ state dict helpers
    def named_master(self) -> Iterable[tuple[str, torch.Tensor]]:
        for name, p in self.order:
            yield name, p.data


def _kernels() -> bool:
    from ..ops import _ext
    return _ext.available()
