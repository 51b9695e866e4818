"""Sharded optimizer for data-parallel training (ZeRO stage 1 with a fused weight broadcast).

The reference has replicated data parallelism only (DDP, run_40b.py:601-603): every rank keeps
all of AdamW's state and repeats the whole update.  Here each rank owns, inside every gradient
bucket of the `ParamArena`, the slice that the in-kernel reduce-scatter leaves on it
(`grad_reduce_kernel` with ``push = 0``, ops/csrc/comm.cu: slice ``r`` of a bucket of ``n4``
float4 words is ``[ceil(n4/world)*r, min(ceil(n4/world)*(r+1), n4))``).  A rank

* receives only its slice of the averaged gradients (half the NVLink bytes of an all-reduce),
* keeps AdamW moments for its slices only (16 bytes/param divided by the world size),
* updates its slices and, in the same kernel (`adamw_shard_push_kernel`), stores the new FP32
  master and BF16 compute weights into every rank's replicas over NVLink -- the all-gather of a
  ZeRO design with no separate collective and no staging copy.

The FP32 master stays whole on every rank because the forward pass reads some parameters in
FP32 (embedding rows, norm weights, decay logits, depth modulation); with ``push_master=False``
only the BF16 mirror is broadcast and `gather_master()` must run before anything reads FP32
weights that another rank owns.  Checkpoints stay in the reference's unsharded format:
`state_dict()` gathers the moments and emits the same structure as
``torch.optim.AdamW.state_dict()``.

Without symmetric memory (CPU/gloo tests, NCCL fallback) the same ownership is used with
``all_gather`` of the updated slices; the update is the replicated optimizer's, element for element, given
the same clip coefficient (the norm is summed per slice in FP64 and rounded once, so it agrees with the
one-rank norm except where the order of the FP64 additions moves the rounded value).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..optim.arena import ParamArena


def bucket_slice(start: int, stop: int, rank: int, world: int) -> tuple[int, int]:
    """Element range of bucket ``[start, stop)`` owned by ``rank`` (same split as the kernel)."""
    n4 = (stop - start) // 4
    per = (n4 + world - 1) // world
    lo = min(per * rank, n4)
    hi = min(lo + per, n4)
    return start + 4 * lo, start + 4 * hi


class ShardedAdamW:
    """Drop-in for `ArenaAdamW` (same attributes and methods) that owns 1/world of every bucket."""

    def __init__(self, arena: ParamArena, *, rank: int, world: int, group=None, sync=None, lr: float = 1.5e-4,
                 betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1, max_grad_norm: float | None = 1.0,
                 push_master: bool = True):
        self.arena, self.rank, self.world, self.group, self.sync = arena, rank, world, group, sync
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.push_master = push_master
        # the ranges one reduction launch handles (whole buckets, or pieces under a bucket cap): ownership follows
        # the kernel's split of each of them
        if sync is not None and hasattr(sync, "pieces_of") and getattr(sync, "arena", None) is arena:
            self.pieces = [(start, start + count) for b in arena.buckets for start, count in sync.pieces_of(b.index)]
        else:
            self.pieces = [(b.start, b.stop) for b in arena.buckets]
        self.ranges = [bucket_slice(start, stop, rank, world) for start, stop in self.pieces]
        self.offsets = [0]
        for lo, hi in self.ranges:
            self.offsets.append(self.offsets[-1] + (hi - lo))
        n = self.offsets[-1]
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=arena.device)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=arena.device)
        self.last_stats = None
        self.master_stale = False
        self.mirror_sym = None
        self.fused = bool(sync is not None and getattr(sync, "kind", "").startswith("fused") and arena.bf16 is not None)
        if self.fused:
            self._adopt_symmetric_mirror()
            sync.push = False  # reduce-scatter: the reduced slice stays on its owner

    # ------------------------------------------------------------------ set-up
    def _adopt_symmetric_mirror(self) -> None:
        """Move the BF16 compute mirror into symmetric memory so that peers can store into it."""
        from . import symm
        a = self.arena
        self.mirror_sym = symm.allocate(a.numel, torch.bfloat16, a.device, self.group)
        self.mirror_sym.tensor.copy_(a.bf16)
        a.bf16 = self.mirror_sym.tensor
        a.bind_grads()
        self.master_sym = None
        if self.push_master:
            self.master_sym = symm.allocate(a.numel, torch.float32, a.device, self.group)
            a.adopt_master(self.master_sym.tensor)
        self.mirror_sym.barrier()

    def owned(self, tensor: torch.Tensor):
        """Views of ``tensor`` (arena-sized) over this rank's slices."""
        return [tensor[lo:hi] for lo, hi in self.ranges]

    # ------------------------------------------------------------------ step
    def zero_grad(self, set_to_none: bool = False) -> None:
        self.arena.zero_grad()

    def clip_stats(self, extra_sumsq: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
        """``[||g||, clip coefficient, ||g||^2, skip, ...]`` of the global gradient.

        With the fused synchroniser the trainer does not come here: the reduce-scatter kernel has already
        left per-CTA sums of squares of the slices this rank owns and `FusedGradSync.exchange_stats`
        combines them over ranks.  With a collective synchroniser every rank holds the whole averaged
        gradient after the all-reduce, so on CUDA the norm is the deterministic two-stage kernel over the
        arena, as in the replicated optimizer; on CPU the owned slices are summed in FP64 and all-reduced."""
        from ..optim.adamw import host_clip_stats
        max_norm = self.max_grad_norm if self.max_grad_norm is not None else 0.0
        grad = self.arena.grad
        if grad.is_cuda and not self.fused:
            from ..ops import _ext
            if _ext.available():
                return torch.ops.ws_b200.grad_norm_clip(grad, float(max_norm), extra_sumsq, status)
        parts = [g.double().pow(2).sum() for g in self.owned(grad) if g.numel()]
        sumsq = torch.stack(parts).sum() if parts else torch.zeros((), dtype=torch.float64, device=self.arena.device)
        sumsq = sumsq.reshape(1)
        if self.world > 1:
            dist.all_reduce(sumsq, op=dist.ReduceOp.SUM, group=self.group)
        sumsq = sumsq.float()      # rounded once, after the ranks' FP64 sums are combined, as the one-rank sum is
        if extra_sumsq is not None:
            sumsq = sumsq + extra_sumsq.reshape(1)
        return host_clip_stats(sumsq, max_norm, status)

    @torch.no_grad()
    def step(self, lr: float | None = None, stats: torch.Tensor | None = None) -> torch.Tensor:
        if lr is not None:
            self.lr = lr
        if stats is None:
            stats = self.clip_stats()
        self.last_stats = stats
        self.step_count += 1
        if self.fused:
            self._step_fused(stats)
        else:
            self._step_collective(stats)
        self.master_stale = self.fused and self.world > 1 and not self.push_master
        return stats

    def _step_fused(self, stats: torch.Tensor) -> None:
        a = self.arena
        b1, b2 = self.betas
        # without push_master only this rank's entry of the table is written
        master_ptrs = self.master_sym.peer_ptrs if self.push_master else [a.master.data_ptr()] * self.world
        for index, (lo, hi) in enumerate(self.ranges):
            if hi <= lo:
                continue
            o0, o1 = self.offsets[index], self.offsets[index + 1]
            torch.ops.ws_b200.adamw_shard_push(master_ptrs, self.mirror_sym.peer_ptrs, self.rank, self.world, a.grad,
                                               self.exp_avg[o0:o1], self.exp_avg_sq[o0:o1], lo, hi - lo,
                                               float(self.lr), b1, b2, self.eps, self.weight_decay, self.step_count,
                                               stats[1:2], self.push_master, stats[3:4])
        self.sync.node_barrier()  # every rank's stores have landed before anyone's next forward

    def _step_collective(self, stats: torch.Tensor) -> None:
        a = self.arena
        b1, b2 = self.betas
        bias1 = 1 - b1 ** self.step_count
        bias2 = 1 - b2 ** self.step_count
        for index, (lo, hi) in enumerate(self.ranges):
            if hi <= lo:
                continue
            o0, o1 = self.offsets[index], self.offsets[index + 1]
            p, g = a.master[lo:hi], a.grad[lo:hi]
            m, v = self.exp_avg[o0:o1], self.exp_avg_sq[o0:o1]
            if p.is_cuda:
                from ..ops import _ext
                if _ext.available():
                    torch.ops.ws_b200.adamw_step(p, g, m, v, None, float(self.lr), b1, b2, self.eps,
                                                 self.weight_decay, self.step_count, stats[1:2], 1.0, stats[3:4])
                    continue
            if float(stats[3]) != 0.0:
                continue
            grad = g * stats[1]
            p.mul_(1 - self.lr * self.weight_decay)
            m.lerp_(grad, 1 - b1)
            v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
            denom = (v.sqrt() / math.sqrt(bias2)).add_(self.eps)
            p.addcdiv_(m, denom, value=-self.lr / bias1)
        self.gather_into(a.master)
        a.refresh_bf16()

    def rollback_step(self) -> None:
        """Undo the step count of an update that the device skipped (``stats[3]`` set)."""
        self.step_count = max(0, self.step_count - 1)

    # ------------------------------------------------------------------ gathers
    def gather_into(self, full: torch.Tensor) -> None:
        """Make ``full`` (arena-sized) whole on every rank from each rank's owned slices."""
        if self.world == 1:
            return
        for start, stop in self.pieces:
            n4 = (stop - start) // 4
            per = 4 * ((n4 + self.world - 1) // self.world)
            if per == 0:
                continue
            lo, hi = bucket_slice(start, stop, self.rank, self.world)
            mine = torch.zeros(per, dtype=full.dtype, device=full.device)
            mine[:hi - lo].copy_(full[lo:hi])
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=self.group)
            for r, part in enumerate(parts):
                rlo, rhi = bucket_slice(start, stop, r, self.world)
                if r != self.rank and rhi > rlo:
                    full[rlo:rhi].copy_(part[:rhi - rlo])

    def gather_master(self) -> None:
        """Refresh the FP32 master weights that other ranks own (before a checkpoint or export)."""
        if self.master_stale:
            self.gather_into(self.arena.master)
            self.master_stale = False

    def gather_full(self, compact: torch.Tensor) -> torch.Tensor:
        """Arena-sized tensor assembled from every rank's compact per-slice storage."""
        full = torch.zeros(self.arena.numel, dtype=compact.dtype, device=compact.device)
        for index, (lo, hi) in enumerate(self.ranges):
            full[lo:hi].copy_(compact[self.offsets[index]:self.offsets[index + 1]])
        self.gather_into(full)
        return full

    # ------------------------------------------------------------------ torch-compatible state
    def state_dict(self) -> dict:
        """Unsharded ``torch.optim.AdamW``-style state (collective: call on every rank)."""
        from ..optim.adamw import ArenaAdamW
        self.gather_master()
        whole = ArenaAdamW.__new__(ArenaAdamW)
        whole.arena, whole.lr, whole.betas, whole.eps = self.arena, self.lr, self.betas, self.eps
        whole.weight_decay, whole.step_count = self.weight_decay, self.step_count
        whole.exp_avg = self.gather_full(self.exp_avg)
        whole.exp_avg_sq = self.gather_full(self.exp_avg_sq)
        return whole.state_dict()

    def load_state_dict(self, sd: dict) -> None:
        from ..optim.adamw import ArenaAdamW
        whole = ArenaAdamW.__new__(ArenaAdamW)
        whole.arena, whole.lr, whole.betas, whole.eps = self.arena, self.lr, self.betas, self.eps
        whole.weight_decay, whole.step_count = self.weight_decay, 0
        whole.lo, whole.hi = 0, self.arena.numel
        # one arena-sized scratch at a time, on the host for large models
        where = "cpu" if self.arena.numel > (1 << 28) else self.arena.device
        whole.exp_avg = torch.zeros(self.arena.numel, dtype=torch.float32, device=where)
        whole.exp_avg_sq = torch.zeros(self.arena.numel, dtype=torch.float32, device=where)
        whole.load_state_dict(sd)
        self.lr, self.betas, self.eps, self.weight_decay = whole.lr, whole.betas, whole.eps, whole.weight_decay
        self.step_count = whole.step_count
        for index, (lo, hi) in enumerate(self.ranges):
            self.exp_avg[self.offsets[index]:self.offsets[index + 1]].copy_(whole.exp_avg[lo:hi])
            self.exp_avg_sq[self.offsets[index]:self.offsets[index + 1]].copy_(whole.exp_avg_sq[lo:hi])

    def memory_bytes(self) -> int:
        return 2 * self.exp_avg.numel() * 4
