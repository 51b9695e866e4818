"""Gradient synchronisation for replicated data parallelism.

Contract (what the reference gets from DistributedDataParallel with ``no_sync`` on all but the
last micro-batch, FP32 buckets averaged over ranks; reference run_40b.py:601-603,742 and
ops/distributed_execution.py:16-79): after `finish_update()` every rank's gradient arena holds
the rank-average of the accumulated FP32 gradients, bit-identical on all ranks.

Two implementations:

* `FusedGradSync`   -- the product path.  The gradient arena lives in symmetric memory; each
  bucket (one per core, plus a tail bucket with embedding / depth modulation / final norm) is
  reduced by ONE kernel (`grad_allreduce_kernel`, ops/csrc/comm.cu) that pulls the rank's slice
  from all peers over NVLink (or reduces it in the switch with multimem), applies the 1/world
  scale and pushes the result to all peers.  Buckets are launched on a side stream as soon as the
  last micro-batch's backward has finished the corresponding core, so the transfer overlaps the
  remaining backward GEMMs.
* `CollectiveGradSync` -- the baseline and oracle: `torch.distributed.all_reduce` per bucket
  (NCCL on CUDA, gloo on CPU).
"""
from __future__ import annotations

import contextlib
import os

import torch
import torch.distributed as dist


class GradSyncBase:
    kind = "none"

    def __init__(self, device: torch.device, world: int, rank: int, group=None, bucket_cap_bytes: int = 0):
        self.device, self.world, self.rank, self.group = device, world, rank, group
        self.bucket_cap_bytes = int(bucket_cap_bytes)   # largest range one reduction handles (0: whole buckets)
        self.arena = None
        self.core_bucket: dict[int, int] = {}
        self.reduced: set[int] = set()
        self.seq = 0

    # ---- hooks used by the trainer
    def alloc_grad_buffer(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        return torch.zeros(numel, dtype=dtype, device=self.device)

    def attach(self, arena, model) -> None:
        self.arena = arena
        self.model = model
        for bucket in arena.buckets:
            cores = {int(n.split(".")[1]) for n in bucket.names if n.startswith("cores.")}
            if cores and all(n.startswith("cores.") for n in bucket.names):
                # backward finishes the cores of a bucket from the highest index down: the lowest one completes it
                self.core_bucket[min(cores)] = bucket.index
        self.core_index = {id(core): i for i, core in enumerate(getattr(model, "cores", []))}

    def begin_update(self) -> None:
        self.seq += 1
        self.reduced.clear()

    @contextlib.contextmanager
    def last_micro_batch(self):
        from ..ops import fused
        fused.set_core_grad_hook(self._core_done)
        try:
            yield
        finally:
            fused.set_core_grad_hook(None)

    def _core_done(self, core) -> None:
        index = self.core_index.get(id(core))
        bucket = self.core_bucket.get(index)
        if bucket is not None and bucket not in self.reduced:
            self.reduce_bucket(bucket)

    def finish_update(self):
        for bucket in reversed(range(len(self.arena.buckets))):
            if bucket not in self.reduced:
                self.reduce_bucket(bucket)
        self.wait()
        return None

    def reduce_scalar(self, t: torch.Tensor) -> None:
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)

    def status_word(self):
        return None

    def pieces_of(self, bucket: int) -> list[tuple[int, int]]:
        """``(start, count)`` ranges of a bucket, none larger than the cap (whole bucket without a cap)."""
        b = self.arena.buckets[bucket]
        total = b.stop - b.start
        cap = (self.bucket_cap_bytes // 4) // 1024 * 1024
        if cap <= 0 or total <= cap:
            return [(b.start, total)]
        return [(b.start + off, min(cap, total - off)) for off in range(0, total, cap)]

    # ---- implemented by subclasses
    def reduce_bucket(self, bucket: int) -> None:
        raise NotImplementedError

    def wait(self) -> None:
        pass


class CollectiveGradSync(GradSyncBase):
    """all_reduce(SUM) / world per bucket through torch.distributed (NCCL or gloo)."""

    def __init__(self, device, world, rank, group=None, bucket_cap_bytes: int = 0):
        super().__init__(device, world, rank, group, bucket_cap_bytes)
        self.kind = "nccl" if device.type == "cuda" else "gloo"
        self.stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self.pending = []

    def reduce_bucket(self, bucket: int) -> None:
        views = [self.arena.grad[start:start + count] for start, count in self.pieces_of(bucket)]
        self.reduced.add(bucket)
        if self.stream is None:
            for view in views:
                dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group)
                view.mul_(1.0 / self.world)
            return
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            for view in views:
                dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group)
                view.mul_(1.0 / self.world)

    def wait(self) -> None:
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)


class FusedGradSync(GradSyncBase):
    """One in-kernel all-reduce per bucket over symmetric memory (NVLink peer access / NVLS).

    Per bucket two launches on the side stream: a one-warp kernel that announces the bucket and waits for
    the peers' announcements, then the data kernel (``ctas`` CTAs), which therefore occupies SMs only
    while it moves data.  The data kernel also leaves per-CTA sums of squares of the slice it reduced;
    `exchange_stats` combines them over ranks (and the loss sum with them) in one more launch, so the
    update needs no library collective at all.

    A bucket may carry ``segments`` -- ``[(start, count, push), ...]`` set by a sharded-parameter
    layout (`parallel/fsdp.py`): reduce-scatter ranges for row-owned matrices and an all-reduce range
    for the replicated rest, all under the bucket's one pair of flags.
    """

    kind = "fused"

    def __init__(self, device, world, rank, group=None, ctas: int | None = None, budget_seconds: float | None = None,
                 use_nvls: bool | None = None, bucket_cap_bytes: int = 0):
        super().__init__(device, world, rank, group, bucket_cap_bytes)
        from ..ops import _ext
        _ext.require()
        self.ctas = int(ctas or os.environ.get("WARPSTATE_COMM_CTAS", 32))
        self.budget = float(budget_seconds or os.environ.get("WARPSTATE_COMM_WAIT_SECONDS", 20.0))
        if use_nvls is None and os.environ.get("WARPSTATE_COMM_PATH") in ("p2p", "nvls"):
            use_nvls = os.environ["WARPSTATE_COMM_PATH"] == "nvls"
        self.use_nvls = use_nvls
        self.stream = torch.cuda.Stream(device=device)
        self.grad_sym = None
        self.flag_sym = None
        self.status = torch.zeros(8, dtype=torch.int32, device=device)
        self.push = True  # False: reduce-scatter (the sharded optimizer keeps each slice on its owner)
        self.segments: dict[int, list[tuple[int, int, bool]]] = {}
        self.barrier_seq = 0

    def alloc_grad_buffer(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        from . import symm
        self.grad_sym = symm.allocate(numel, dtype, self.device, self.group)
        return self.grad_sym.tensor

    def attach(self, arena, model) -> None:
        super().attach(arena, model)
        from . import symm
        # one pair of flags (and one row of norm partials) per launch: a bucket above the cap is several launches
        self.launch_ids: dict[int, list[int]] = {}
        launches = 0
        for b in arena.buckets:
            count = 1 if getattr(arena, "segments", None) else len(self.pieces_of(b.index))
            self.launch_ids[b.index] = list(range(launches, launches + count))
            launches += count
        self.exchange_base = 2 * 8 * launches         # words after the launch flags: norm exchange ...
        self.barrier_base = self.exchange_base + 24   # ... and the node barrier
        words = self.barrier_base + 8
        self.flag_sym = symm.allocate(max(words, 64), torch.int32, self.device, self.group)
        self.partials = torch.zeros(launches * self.ctas, dtype=torch.float32, device=self.device)
        mc = self.grad_sym.multicast_ptr
        # Measured on 256 MiB FP32 (bus GB/s): two ranks -- peer loads 566-617, multimem 388; four ranks -- peer loads
        # 470-582, multimem 645 at any CTA count.  With one peer the switch has nothing to reduce; from four ranks on
        # its traffic per rank stays constant while peer loads grow with the peer count.
        if self.use_nvls is False or (self.use_nvls is None and self.world <= 2):
            mc = 0
        self.mc_ptr = mc
        self.kind = "fused-nvls" if mc else "fused-p2p"
        self.flag_sym.barrier()

    def reduce_bucket(self, bucket: int) -> None:
        self.reduced.add(bucket)
        segmented = self.segments.get(bucket)
        if segmented:
            work = [segmented]
        else:
            work = [[(start, count, self.push)] for start, count in self.pieces_of(bucket)]
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            for launch, segs in zip(self.launch_ids[bucket], work):
                torch.ops.ws_b200.grad_reduce_segments(
                    self.grad_sym.peer_ptrs, self.flag_sym.peer_ptrs, self.mc_ptr, self.rank, self.world,
                    [s[0] for s in segs], [s[1] for s in segs], [int(bool(s[2])) for s in segs], launch, self.seq,
                    1.0 / self.world, self.ctas, self.partials[launch * self.ctas:(launch + 1) * self.ctas],
                    self.status, self.budget)

    def wait(self) -> None:
        torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def finish_update(self):
        """Reduce what is left, join the side stream; returns this rank's partial sums of squares."""
        super().finish_update()
        return self.partials

    def exchange_stats(self, partials: torch.Tensor, max_norm: float, local_loss: torch.Tensor | None) -> torch.Tensor:
        """``[norm, coef, norm^2, skip, loss summed over ranks, ...]`` of the averaged gradient, bit-identical
        on every rank (one launch; slots in the flag buffers, added in rank order)."""
        return torch.ops.ws_b200.norm_exchange(self.flag_sym.peer_ptrs, self.rank, self.world, self.exchange_base,
                                               self.seq, partials, local_loss, float(max_norm), self.status,
                                               self.budget)

    def node_barrier(self) -> None:
        """Device-side barrier over the node on the current stream (bounded; failure lands in the status word)."""
        self.barrier_seq += 1
        torch.ops.ws_b200.node_barrier(self.flag_sym.peer_ptrs, self.rank, self.world, self.barrier_base,
                                       self.barrier_seq, self.status, self.budget)

    def status_word(self):
        return self.status[0]

    def describe_error(self) -> str:
        code, bucket, src, expected, seen = self.status[:5].tolist()
        what = {1: "waiting for a peer's gradients to be ready", 2: "waiting for peers to finish writing",
                3: "waiting for a peer's share of the gradient norm", 4: "in the node barrier"}.get(code, "?")
        return (f"rank {self.rank}: gradient synchronisation gave up {what}: bucket {bucket}, peer {src}, "
                f"expected {expected}, saw {seen}")


def make_grad_sync(device: torch.device, world: int, rank: int, group=None, kind: str = "auto",
                   bucket_cap_bytes: int = 0):
    if world <= 1:
        return None
    if kind == "auto":
        kind = "fused" if device.type == "cuda" else "collective"
    if kind == "fused":
        return FusedGradSync(device, world, rank, group, bucket_cap_bytes=bucket_cap_bytes)
    if kind in ("collective", "nccl", "gloo"):
        return CollectiveGradSync(device, world, rank, group, bucket_cap_bytes=bucket_cap_bytes)
    raise ValueError(f"unknown gradient synchronisation kind: {kind}")
