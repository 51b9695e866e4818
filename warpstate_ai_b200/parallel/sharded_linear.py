"""Linear layer over a weight whose FP32 master rows are sharded across the GPUs of a node.

`ShardedWeight` keeps rank r's rows ``[r * rows_per_shard, (r + 1) * rows_per_shard)`` of a
``[n, k]`` FP32 weight in symmetric memory.  `forward(x)` is ONE kernel launch
(`gemm2_kernel<..., GATHER=true>`, `ops/csrc/gemm2_tcgen05.cu`): four warps of every CTA pull the
shards -- peer loads over NVLink for the rows other ranks own -- cast them to BF16 into a local
landing buffer and publish per-128-row-block counters, while the TMA/tcgen05 tile loop of the
same CTAs consumes each block of weight rows as soon as it is complete.  All-gather, cast and
GEMM overlap tile by tile; the gathered BF16 weight is left in the landing buffer, so the
backward pass (dX = dY W, dW = dY^T X) and the remaining micro-batches of the update reuse it
with the ordinary GEMM kernels.

The reference has no parameter sharding (its only strategy is replicated data parallelism,
reference run_40b.py:601-603); this is the per-core "gather the weights, cast them, feed the first
GEMM" step of a ZeRO-3 layout, built so that the gather costs link time only for the first block.

Rules the caller keeps:

* every rank calls `forward` with the same sequence of weights (the kernel itself does not
  synchronise ranks: it only READS peer memory);
* no rank writes its shard between `publish()` (a barrier) and the last `forward` of any rank
  that reads it -- `publish()` is called after the optimizer step that changed the shard.

CPU / single-process use: `world == 1`, or several "ranks" emulated by shards that all live on
one device (`ShardedWeight.emulated`), which exercises the same kernel and index arithmetic.
"""
from __future__ import annotations

import torch

from ..ops import gemm as G


def rows_per_shard(n: int, world: int) -> int:
    """Rows each rank owns: ceil(n / world) rounded up to the gather granule of 8 rows."""
    per = (n + world - 1) // world
    return (per + 7) // 8 * 8


class ShardedWeight:
    """Row-sharded FP32 weight with a fused gather + cast + GEMM forward."""

    def __init__(self, n: int, k: int, rank: int, world: int, shard: torch.Tensor, shard_ptrs: list[int],
                 barrier=None, swiglu: bool = False):
        if n % 8 or k % 8:
            raise ValueError("n and k must be multiples of 8")
        if swiglu and (n % 2 or (n // 2) % 128):
            raise ValueError("a SwiGLU weight needs 2*h rows (up, then gate) with h a multiple of 128")
        self.swiglu = swiglu                    # W = [2h, k]: forward returns (packed, silu(gate) * up)
        self.n, self.k, self.rank, self.world = n, k, rank, world
        self.rows = rows_per_shard(n, world)
        if shard.dtype != torch.float32 or shard.numel() < self.rows * k:
            raise ValueError("shard must be FP32 with rows_per_shard * k elements")
        self.shard = shard                      # this rank's rows (FP32 master)
        self.shard_ptrs = list(shard_ptrs)
        self._barrier = barrier
        device = shard.device
        self.gathered = torch.empty(n, k, device=device, dtype=torch.bfloat16)   # landing buffer
        self.flags = torch.zeros((n + 127) // 128 + 1, device=device, dtype=torch.int32)   # one word per 128 rows + chunk counter
        self.error_flag = G.error_flag(device) if device.type == "cuda" else None
        self.group = None                       # process group of the collective fallback
        self.gathered_valid = False
        self.shard_grad = None                  # FP32 gradient of this rank's rows (set by ShardedLinear)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_full(cls, weight: torch.Tensor, rank: int, world: int, group=None, swiglu: bool = False) -> "ShardedWeight":
        """Shard a full ``[n, k]`` weight (identical on every rank) into symmetric memory."""
        from . import symm
        n, k = weight.shape
        per = rows_per_shard(n, world)
        buf = symm.allocate(per * k, torch.float32, weight.device, group)
        lo, hi = rank * per, min(n, (rank + 1) * per)
        if hi > lo:
            buf.tensor[:(hi - lo) * k].copy_(weight[lo:hi].reshape(-1).float())
        self = cls(n, k, rank, world, buf.tensor, buf.peer_ptrs, barrier=buf.barrier, swiglu=swiglu)
        self._sym = buf
        self.publish()
        return self

    @classmethod
    def from_full_collective(cls, weight: torch.Tensor, rank: int, world: int, group=None,
                             swiglu: bool = False) -> "ShardedWeight":
        """The same ownership without symmetric memory (CPU / gloo, or a GPU job without peer access):
        `forward` gathers the shards with an ordinary all-gather, then casts and multiplies.  The host-side
        logic -- ownership, publish, cached re-use, gradient scatter -- is the one of the fused path."""
        n, k = weight.shape
        per = rows_per_shard(n, world)
        shard = torch.zeros(per * k, device=weight.device, dtype=torch.float32)
        lo, hi = rank * per, min(n, (rank + 1) * per)
        if hi > lo:
            shard[:(hi - lo) * k].copy_(weight[lo:hi].reshape(-1).float())
        self = cls(n, k, rank, world, shard, [], swiglu=swiglu)
        self.group = group
        self._collective = True
        return self

    @classmethod
    def emulated(cls, weight: torch.Tensor, world: int, swiglu: bool = False) -> "ShardedWeight":
        """All ``world`` shards on one device: the kernel and its index arithmetic without peers."""
        n, k = weight.shape
        per = rows_per_shard(n, world)
        shards = []
        for r in range(world):
            t = torch.zeros(per * k, device=weight.device, dtype=torch.float32)
            lo, hi = r * per, min(n, (r + 1) * per)
            if hi > lo:
                t[:(hi - lo) * k].copy_(weight[lo:hi].reshape(-1).float())
            shards.append(t)
        self = cls(n, k, 0, world, shards[0], [t.data_ptr() for t in shards], swiglu=swiglu)
        self._keep = shards
        return self

    # ------------------------------------------------------------------ use
    def publish(self) -> None:
        """Make this rank's shard visible to the peers' next `forward` (device barrier over the node)
        and mark the landing buffer stale."""
        self.gathered_valid = False
        if self._barrier is not None:
            torch.cuda.current_stream(self.shard.device).synchronize()
            self._barrier()

    def forward(self, x: torch.Tensor, budget_seconds: float = 2.0):
        """``x [m, k]`` BF16 -> ``x @ W^T [m, n]`` BF16; gathers and casts W in the same launch.
        A SwiGLU weight returns ``(packed [m, 2h], silu(gate) * up [m, h])`` like `ops.gemm.linear_swiglu`."""
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        if getattr(self, "_collective", False):
            self._gather_collective()
            return self._math_forward(x)
        out, act = torch.ops.ws_b200.gather_cast_linear(
            x.contiguous(), self.shard_ptrs, self.n // 2 if self.swiglu else self.n, self.rows, self.gathered,
            self.flags, self.error_flag, float(budget_seconds), self.swiglu, True)
        self.gathered_valid = True
        return (out, act) if self.swiglu else out

    def forward_cached(self, x: torch.Tensor):
        """Later micro-batches of the same update: the landing buffer already holds the BF16 weight."""
        if not self.gathered_valid:
            return self.forward(x)
        if getattr(self, "_collective", False):
            return self._math_forward(x)
        return G.linear_swiglu(x, self.gathered) if self.swiglu else G.linear(x, self.gathered)

    # ------------------------------------------------------------------ collective fallback
    def _gather_collective(self) -> None:
        import torch.distributed as dist
        if self.world > 1:
            parts = [torch.empty_like(self.shard) for _ in range(self.world)]
            dist.all_gather(parts, self.shard, group=self.group)
        else:
            parts = [self.shard]
        rows = torch.cat([p.view(self.rows, self.k) for p in parts], dim=0)[:self.n]
        self.gathered.copy_(rows)               # FP32 -> BF16, the cast the kernel does on the fly
        self.gathered_valid = True

    def _math_forward(self, x: torch.Tensor):
        both = (x.float() @ self.gathered.float().T)
        if not self.swiglu:
            return both.to(torch.bfloat16)
        h = self.n // 2
        packed = both.to(torch.bfloat16)
        up, gate = packed[:, :h].float(), packed[:, h:].float()
        return packed, (torch.nn.functional.silu(gate) * up).to(torch.bfloat16)

    def full_weight(self) -> torch.Tensor:
        """The whole FP32 weight, read shard by shard (emulated shards only; for tests)."""
        keep = getattr(self, "_keep", None)
        if keep is None:
            raise RuntimeError("full_weight() needs emulated shards")
        rows = torch.cat([t.view(self.rows, self.k) for t in keep], dim=0)
        return rows[:self.n]


class _ShardedLinearFn(torch.autograd.Function):
    """y = x W^T over a `ShardedWeight`; dX from the gathered BF16 weight, dW reduce-scattered to its owners."""

    @staticmethod
    def forward(ctx, x, anchor, sw: ShardedWeight, fresh: bool, group):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        x2 = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
        x2 = x2.contiguous()
        y = sw.forward(x2) if fresh else sw.forward_cached(x2)
        ctx.sw, ctx.group, ctx.shape, ctx.x_dtype = sw, group, shape, x.dtype
        ctx.save_for_backward(x2)
        return y.view(*shape[:-1], sw.n)

    @staticmethod
    def backward(ctx, dy):
        import torch.distributed as dist
        sw: ShardedWeight = ctx.sw
        (x2,) = ctx.saved_tensors
        dy2 = dy.reshape(-1, sw.n)
        dy2 = (dy2 if dy2.dtype == torch.bfloat16 else dy2.to(torch.bfloat16)).contiguous()
        collective = getattr(sw, "_collective", False)
        # full dW in FP32 (rows padded to world * rows_per_shard), then each owner keeps the sum of its rows
        full = torch.zeros(sw.rows * sw.world, sw.k, device=dy2.device, dtype=torch.float32)
        if collective:
            dx = (dy2.float() @ sw.gathered.float()).to(torch.bfloat16).view(ctx.shape).to(ctx.x_dtype)
            full[:sw.n] = dy2.float().T @ x2.float()
        else:
            dx = G.grad_input(dy2, sw.gathered).view(ctx.shape).to(ctx.x_dtype)
            G.grad_weight_accumulate(dy2, x2, full[:sw.n])
        if collective and sw.world > 1 and dist.is_initialized():
            dist.all_reduce(full, group=ctx.group if ctx.group is not None else sw.group)  # gloo has no reduce-scatter
            mine = full[sw.rank * sw.rows:(sw.rank + 1) * sw.rows].clone()
        elif sw.world > 1 and dist.is_initialized():
            mine = torch.empty(sw.rows, sw.k, device=dy2.device, dtype=torch.float32)
            dist.reduce_scatter_tensor(mine, full, group=ctx.group)
        else:
            mine = full[:sw.rows]
        if sw.shard_grad is None:
            sw.shard_grad = mine.clone() if mine.data_ptr() == full.data_ptr() else mine
        else:
            sw.shard_grad += mine
        return dx, None, None, None, None


class ShardedLinear(torch.nn.Module):
    """A bias-free linear layer whose FP32 weight rows live sharded across the ranks of a node.

    ``forward(x)`` runs the fused gather + cast + GEMM the first time after `publish()` and the
    plain GEMM on the landing buffer afterwards; the weight gradient of this rank's rows is summed
    over ranks into ``weight.shard_grad`` (FP32, ``[rows_per_shard, k]``).  After the owner has
    updated ``weight.shard`` it calls ``publish()``.
    """

    def __init__(self, weight: ShardedWeight, group=None):
        super().__init__()
        if weight.swiglu:
            raise ValueError("ShardedLinear takes a plain weight; a SwiGLU weight is used through ShardedWeight.forward")
        self.weight = weight
        self.group = group
        weight.shard_grad = None
        # autograd needs one differentiable input even when x comes from a frozen producer
        self._anchor = torch.nn.Parameter(torch.zeros((), device=weight.shard.device))

    def publish(self) -> None:
        self.weight.publish()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _ShardedLinearFn.apply(x, self._anchor, self.weight, not self.weight.gathered_valid, self.group)


class ShardedRowsAdamW:
    """AdamW on the rows each rank owns of one or more `ShardedLinear` layers.

    Only the owner holds the FP32 master rows, their gradient (already summed over ranks by the layer's
    backward) and their two moments: parameter, gradient and optimizer memory per rank are 1/world of the
    layer's.  `step()` updates the owned rows in place and publishes them; `zero_grad()` drops the row
    gradients.  The update is `torch.optim.AdamW`'s (decoupled weight decay, bias-corrected moments), the
    optimizer the reference uses on every parameter (reference run_40b.py:534-535).
    """

    def __init__(self, layers, lr: float = 1e-3, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1):
        self.layers = list(layers)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.steps = 0
        self.m = [torch.zeros_like(layer.weight.shard) for layer in self.layers]
        self.v = [torch.zeros_like(layer.weight.shard) for layer in self.layers]

    def zero_grad(self) -> None:
        for layer in self.layers:
            layer.weight.shard_grad = None

    @torch.no_grad()
    def step(self, lr: float | None = None, grad_scale: float = 1.0) -> None:
        lr = self.lr if lr is None else lr
        self.steps += 1
        b1, b2 = self.betas
        c1, c2 = 1.0 - b1 ** self.steps, 1.0 - b2 ** self.steps
        for layer, m, v in zip(self.layers, self.m, self.v):
            sw = layer.weight
            if sw.shard_grad is not None:
                g = sw.shard_grad.reshape(-1)[:sw.shard.numel()] * grad_scale
                p = sw.shard
                p.mul_(1.0 - lr * self.weight_decay)
                m.mul_(b1).add_(g, alpha=1.0 - b1)
                v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
                p.addcdiv_(m / c1, (v / c2).sqrt_().add_(self.eps), value=-lr)
            layer.publish()

    def memory_bytes(self) -> int:
        return sum(4 * (m.numel() + v.numel()) for m, v in zip(self.m, self.v))

    # ------------------------------------------------------------------ unsharded optimizer state
    def gather_state(self, group=None) -> dict:
        """Step count and whole-weight moments (``[n, k]`` per layer), identical on every rank: the form a
        checkpoint keeps, so that a run can resume on a different number of ranks (collective call)."""
        import torch.distributed as dist

        def whole(layer, rows_tensor):
            sw = layer.weight
            if sw.world > 1:
                parts = [torch.empty_like(rows_tensor) for _ in range(sw.world)]
                dist.all_gather(parts, rows_tensor.contiguous(), group=group)
            else:
                parts = [rows_tensor]
            return torch.cat([p.view(sw.rows, sw.k) for p in parts], dim=0)[:sw.n].clone()

        return {"steps": self.steps,
                "exp_avg": [whole(layer, m) for layer, m in zip(self.layers, self.m)],
                "exp_avg_sq": [whole(layer, v) for layer, v in zip(self.layers, self.v)]}

    def load_state(self, state: dict) -> None:
        """Adopt a `gather_state` result: every rank keeps the moments of the rows it owns now."""
        if len(state["exp_avg"]) != len(self.layers):
            raise ValueError("optimizer state does not match the number of sharded layers")
        self.steps = int(state["steps"])
        for layer, m, v, full_m, full_v in zip(self.layers, self.m, self.v, state["exp_avg"], state["exp_avg_sq"]):
            sw = layer.weight
            if tuple(full_m.shape) != (sw.n, sw.k):
                raise ValueError(f"moment shape {tuple(full_m.shape)} does not match the weight {(sw.n, sw.k)}")
            lo, hi = sw.rank * sw.rows, min(sw.n, (sw.rank + 1) * sw.rows)
            for own, full in ((m, full_m), (v, full_v)):
                own.zero_()
                if hi > lo:
                    own[:(hi - lo) * sw.k].copy_(full[lo:hi].reshape(-1).to(own.device, own.dtype))
