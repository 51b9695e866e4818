"""WarpState with row-sharded projection weights (parameters, gradients and Adam moments of the four
projections of every core live on their row owners only).

`shard_core_linears(model, rank, world)` replaces `in_proj`, `out_proj`, `ffn.up_gate` and `ffn.down` of
every core -- 96.6 % of the 2.005 B parameters -- by `ShardedLinear` layers.  A layer's first use after an
optimizer step gathers the FP32 rows from their owners, casts them and multiplies in one launch (on a GPU
with symmetric memory; an all-gather followed by a cast elsewhere), later uses in the same update reuse
the gathered BF16 weight; its backward sends every owner the sum over ranks of the gradient of its rows.
The remaining parameters (embedding, norms, per-head logits, depth modulation) stay replicated and their
gradients are summed with `allreduce_replicated_grads`.  `ShardedRowsAdamW` steps the owned rows,
any ordinary optimizer the replicated rest.

The cores then run module by module (norm, projection, attention + memory, projection, norm, SwiGLU) instead
of through the fused layer kernels, which read whole weight tensors; this is the functional sharded layout,
not the fastest path of the framework.  Activation checkpointing must be off (a recomputed forward would
consume the "first use" of a layer).

`gather_state_dict` rebuilds the unsharded state dict with the reference's keys
(`cores.{i}.in_proj.weight`, ..., reference warpstate/model.py:73-105), so checkpoints keep their format.
The reference itself has no parameter sharding (reference run_40b.py:601-603 wraps the model in DDP).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .sharded_linear import ShardedLinear, ShardedWeight

_PROJECTIONS = (("in_proj", None), ("out_proj", None), ("up_gate", "ffn"), ("down", "ffn"))


def _holder(core, parent: str | None):
    return getattr(core, parent) if parent else core


def shard_core_linears(model, rank: int, world: int, group=None, symmetric: bool | None = None) -> list[ShardedLinear]:
    """Replace the four projections of every core in place; returns the new layers (core-major order).

    ``symmetric``: shards in symmetric memory with the fused gather kernel (default on CUDA when
    ``world > 1`` or always on CUDA), otherwise the collective form.  Every rank must hold the same weights
    when this is called (they are sharded from the local copy).
    """
    if model.cfg.gradient_checkpointing:
        raise ValueError("sharded projections need gradient_checkpointing=False")
    layers = []
    for core in model.cores:
        for name, parent in _PROJECTIONS:
            holder = _holder(core, parent)
            linear = getattr(holder, name)
            weight = linear.weight.detach()
            use_symmetric = weight.is_cuda if symmetric is None else symmetric
            if use_symmetric and world > 1:
                sw = ShardedWeight.from_full(weight, rank, world, group)
            elif use_symmetric:
                sw = ShardedWeight.emulated(weight, 1)
            else:
                sw = ShardedWeight.from_full_collective(weight, rank, world, group)
            layer = ShardedLinear(sw, group)
            setattr(holder, name, layer)
            layers.append(layer)
        core.sharded_linears = True
    model.sharded_linears = True
    return layers


def replicated_parameters(model) -> list[torch.nn.Parameter]:
    """The parameters that stay whole on every rank (everything but the sharded rows and their anchors)."""
    return [p for name, p in model.named_parameters() if not name.endswith("_anchor")]


def allreduce_replicated_grads(model, group=None, average: bool = False) -> None:
    """Sum (or average) the gradients of the replicated parameters over the ranks, in one flat buffer."""
    params = [p for p in replicated_parameters(model) if p.grad is not None]
    if not params or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    flat = torch.cat([p.grad.reshape(-1).float() for p in params])
    dist.all_reduce(flat, group=group)
    if average:
        flat /= dist.get_world_size(group)
    offset = 0
    for p in params:
        n = p.grad.numel()
        p.grad.copy_(flat[offset:offset + n].view_as(p.grad))
        offset += n


def gather_state_dict(model, group=None) -> dict[str, torch.Tensor]:
    """The unsharded FP32 state dict under the reference's keys (collective: every rank calls it)."""
    state = {k: v for k, v in model.state_dict().items() if not k.endswith("_anchor")}
    for index, core in enumerate(model.cores):
        for name, parent in _PROJECTIONS:
            layer = getattr(_holder(core, parent), name)
            if not isinstance(layer, ShardedLinear):
                continue
            sw = layer.weight
            if sw.world > 1:
                parts = [torch.empty_like(sw.shard) for _ in range(sw.world)]
                dist.all_gather(parts, sw.shard.contiguous(), group=group)
            else:
                parts = [sw.shard]
            rows = torch.cat([p.view(sw.rows, sw.k) for p in parts], dim=0)[:sw.n]
            key = f"cores.{index}." + (f"{parent}." if parent else "") + f"{name}.weight"
            state[key] = rows.clone()
    return state


def sharded_bytes(layers) -> dict[str, int]:
    """Bytes this rank holds for the sharded projections: FP32 master rows, and the BF16 landing buffers."""
    return {"master_rows": sum(4 * layer.weight.shard.numel() for layer in layers),
            "landing_bf16": sum(2 * layer.weight.gathered.numel() for layer in layers)}
