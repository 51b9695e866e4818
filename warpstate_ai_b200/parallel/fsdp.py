"""Fully sharded training state (ZeRO-3 style) for the WarpState core projections.

The reference trains with replicated data parallelism only (DDP, reference run_40b.py:601-603, and a
whole AdamW on every rank, run_40b.py:534-535).  This module shards what dominates the model -- the four
projection matrices of every core, 96.6 % of the 2.005 B parameters -- over the GPUs of a node:

* **parameters**: rank ``r`` keeps rows ``[r * n/world, (r + 1) * n/world)`` of every ``[n, k]``
  projection as FP32 master rows in ONE symmetric-memory buffer (`master`), nothing else of it;
* **gradients**: weight gradients accumulate in FP32 straight from the dW GEMM epilogue into the
  gradient arena (as in the replicated trainer); when a core's backward of the last micro-batch is
  done, ONE launch (`grad_reduce_kernel`, ops/csrc/comm.cu) reduce-scatters its four matrices to
  their row owners and all-reduces its small parameters, overlapped with the remaining backward;
* **optimizer state**: AdamW moments exist only for the owned rows (plus the replicated rest);
* **compute weights**: before a core runs, its BF16 weights are assembled in a landing slot from the
  owners' FP32 rows over NVLink.  In the forward pass `in_proj` and `up_gate` do that inside their own
  GEMM launch (gather + FP32->BF16 cast + tcgen05 tile loop, `gemm2_kernel<GATHER>`), `out_proj` and
  `down` are fetched by `gather_cast_kernel` on a side stream while the attention block runs; for the
  backward pass the previous core's four matrices are fetched on the side stream under the current
  core's backward.  ``mode="stream"`` keeps two slots (weights are re-gathered for every use, per-rank
  BF16 weight memory is two cores' worth); ``mode="resident"`` keeps one slot per core, filled once per
  update.

Embedding (tied LM head), norms, per-head logits and depth modulation stay replicated: their
gradients are all-reduced and every rank repeats their (small) AdamW update.

Everything that crosses ranks on the GPU path is this package's own kernels over peer memory; no
tensor map covers a peer's buffer and no library kernel is handed a peer pointer.  On CPU (gloo) the
same ownership, optimizer and checkpoint logic runs with ordinary collectives: the full FP32 weights
are materialised around each micro-batch for the PyTorch modules.

Checkpoints stay unsharded and keyed like the reference's (`model_state_dict`, `optimizer.state_dict`),
so a run can resume replicated, or sharded over a different number of ranks.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..optim.adamw import host_adamw, host_clip_stats
from ..optim.arena import ALIGN, Bucket, Slot, default_groups

PROJECTIONS = ("in_proj.weight", "out_proj.weight", "ffn.up_gate.weight", "ffn.down.weight")
SHORT = {"in_proj.weight": "in", "out_proj.weight": "out", "ffn.up_gate.weight": "ug", "ffn.down.weight": "down"}


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def is_sharded_name(name: str) -> bool:
    return name.startswith("cores.") and name.split(".", 2)[2] in PROJECTIONS


@dataclass
class Matrix:
    """One sharded projection: where its gradient lives in the arena and its rows in the master shard."""
    name: str
    core: int
    kind: str          # in | out | ug | down
    n: int
    k: int
    rows: int          # rows per rank
    goff: int          # element offset of the full [n, k] gradient in the arena
    moff: int          # element offset of this rank's [rows, k] master rows in `master`
    param: torch.nn.Parameter = field(repr=False, default=None)


class ShardedArena:
    """Gradient arena over ALL parameters (same bucket order as `optim.ParamArena`: tail, then one bucket
    per core) with a compact FP32 master / BF16 mirror for the replicated parameters only.

    Inside a core's bucket the small parameters come first, then the four matrices, so that a bucket is
    five contiguous segments: one all-reduce range and four reduce-scatter ranges."""

    def __init__(self, model, rank: int, world: int, device: torch.device, symmetric_alloc=None):
        self.device, self.rank, self.world = device, rank, world
        self.order = list(model.named_parameters())
        groups = default_groups(model)
        self.slots: list[Slot] = []
        self.buckets: list[Bucket] = []
        self.segments: dict[int, list[tuple[int, int, bool]]] = {}
        self.matrices: list[Matrix] = []
        self.rep_runs: list[tuple[int, int, int]] = []   # (grad offset, count, compact master offset)
        offset = moff_rep = moff_sh = 0
        seen = set()
        for b, group in enumerate(groups):
            start = offset
            small = [(n, p) for n, p in group if not is_sharded_name(n)]
            big = [(n, p) for n, p in group if is_sharded_name(n)]
            names, segs = [], []
            run_start = offset
            for name, p in small:
                if id(p) in seen:
                    continue
                seen.add(id(p))
                self.slots.append(Slot(name, p, offset, p.numel(), p.shape, b))
                names.append(name)
                offset = _round_up(offset + p.numel(), ALIGN)
            if offset > run_start:
                self.rep_runs.append((run_start, offset - run_start, moff_rep))
                moff_rep += offset - run_start
                segs.append((run_start, offset - run_start, True))
            for name, p in big:
                if id(p) in seen:
                    raise ValueError(f"{name}: a sharded projection cannot be shared between modules")
                seen.add(id(p))
                n, k = p.shape
                if n % world or (n // world) % 8 or k % 8 or (n * k) % ALIGN:
                    raise ValueError(f"{name} [{n}, {k}] cannot be row-sharded over {world} ranks "
                                     "(rows per rank must be a multiple of 8)")
                core = int(name.split(".")[1])
                rows = n // world
                self.slots.append(Slot(name, p, offset, p.numel(), p.shape, b))
                self.matrices.append(Matrix(name, core, SHORT[name.split(".", 2)[2]], n, k, rows, offset, moff_sh, p))
                names.append(name)
                segs.append((offset, n * k, False))
                moff_sh += rows * k
                offset += n * k
            self.buckets.append(Bucket(b, start, offset, names))
            self.segments[b] = segs
        if len(seen) != len({id(p) for p in model.parameters()}):
            raise ValueError("parameter groups do not cover the model")
        self.numel = offset
        self.rep_numel, self.shard_numel = moff_rep, moff_sh
        self.by_name = {s.name: s for s in self.slots}
        self.matrix_by_name = {m.name: m for m in self.matrices}
        alloc = symmetric_alloc or (lambda n, dtype: torch.zeros(n, dtype=dtype, device=device))
        self.grad = alloc(self.numel, torch.float32)
        self.master = torch.zeros(self.rep_numel, dtype=torch.float32, device=device)       # replicated parameters
        self.bf16 = torch.zeros(self.rep_numel, dtype=torch.bfloat16, device=device) if device.type == "cuda" else None

    # ---- replicated parameters: compact views
    def rep_offset(self, slot: Slot) -> int:
        for gstart, count, mstart in self.rep_runs:
            if gstart <= slot.offset < gstart + count:
                return mstart + (slot.offset - gstart)
        raise KeyError(slot.name)

    def zero_grad(self) -> None:
        self.grad.zero_()

    def collect_stray_grads(self) -> None:
        for s in self.slots:
            g = s.param.grad
            target = self.grad[s.offset:s.offset + s.numel].view(s.shape)
            if g is not None and g.data_ptr() != target.data_ptr():
                target.add_(g.to(target.dtype))
                s.param.grad = target

    def refresh_bf16(self) -> None:
        if self.bf16 is None:
            return
        from ..ops import _ext
        if self.master.is_cuda and _ext.available() and self.master.numel() % 4 == 0:
            torch.ops.ws_b200.cast_bf16(self.master, self.bf16)
        else:
            self.bf16.copy_(self.master)


class _Slot:
    """BF16 landing buffers for one core's four matrices."""

    def __init__(self, shapes: dict, device):
        self.w = {kind: torch.empty(n, k, dtype=torch.bfloat16, device=device) for kind, (n, k) in shapes.items()}
        self.flags = {kind: torch.zeros((shapes[kind][0] + 127) // 128 + 1, dtype=torch.int32, device=device)
                      for kind in ("in", "ug")}
        self.core = -1
        self.version = -1
        self.have: dict[str, object] = {}     # kind -> None (ordered on the compute stream) or a CUDA event
        self.last_use = None                  # event on the compute stream after the slot's last reader


class CoreWeights:
    """What `ops.fused.CoreFn` asks for a core's projection weights when they are sharded (the replicated
    counterpart is `ops.fused.LocalWeights`)."""

    def __init__(self, state: "ShardedParamState", core: int):
        self.state, self.core = state, core

    # ---- forward
    def begin_forward(self) -> None:
        self.state.fetch(self.core, ("out", "down"))

    def in_proj(self, z):
        return self.state.fused_linear(self.core, "in", z)

    def up_gate(self, z):
        return self.state.fused_linear(self.core, "ug", z)

    def out_w(self):
        return self.state.weight(self.core, "out")

    def down_w(self):
        return self.state.weight(self.core, "down")

    def end_forward(self) -> None:
        self.state.mark_used(self.core)

    # ---- backward
    def begin_backward(self) -> None:
        self.state.fetch(self.core, ("down", "ug", "out", "in"))
        if self.core > 0:
            self.state.fetch(self.core - 1, ("down", "ug", "out", "in"))

    def backward_weights(self):
        s = self.state
        return s.weight(self.core, "in"), s.weight(self.core, "out"), s.weight(self.core, "ug"), s.weight(self.core, "down")

    def end_backward(self) -> None:
        self.state.mark_used(self.core)


class ShardedParamState:
    """Owns the sharded arena, the master shard, the landing slots and the optimizer of one rank."""

    def __init__(self, model, *, device: torch.device, rank: int, world: int, group=None, sync=None,
                 mode: str = "stream", lr: float = 1.5e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float | None = 1.0):
        if mode not in ("stream", "resident"):
            raise ValueError("mode must be 'stream' or 'resident'")
        if getattr(model.cfg, "n_cores", 0) != getattr(model.cfg, "logical_depth", 0):
            raise ValueError("sharded parameters need one core per logical depth (no core sharing)")
        self.model, self.device, self.rank, self.world, self.group, self.sync = model, device, rank, world, group, sync
        self.mode = mode
        self.cuda = device.type == "cuda"
        self.fused_comm = bool(self.cuda and sync is not None and getattr(sync, "kind", "").startswith("fused"))
        alloc = sync.alloc_grad_buffer if sync is not None else None
        self.arena = ShardedArena(model, rank, world, device, symmetric_alloc=alloc)
        a = self.arena
        # ---- master rows in symmetric memory (peers read them), replicated rest in the compact arena
        self.master_sym = None
        if self.cuda and world > 1:
            from . import symm
            self.master_sym = symm.allocate(a.shard_numel, torch.float32, device, group)
            self.master = self.master_sym.tensor
            self.master_ptrs = list(self.master_sym.peer_ptrs)
        else:
            self.master = torch.zeros(a.shard_numel, dtype=torch.float32, device=device)
            self.master_ptrs = [self.master.data_ptr()] * world if world == 1 else []
        with torch.no_grad():
            for s in a.slots:
                m = a.matrix_by_name.get(s.name)
                g = a.grad[s.offset:s.offset + s.numel].view(s.shape)
                if m is None:
                    off = a.rep_offset(s)
                    view = a.master[off:off + s.numel].view(s.shape)
                    view.copy_(s.param.detach().to(device, torch.float32))
                    s.param.data = view
                    if a.bf16 is not None:
                        s.param.bf16_view = a.bf16[off:off + s.numel].view(s.shape)
                else:
                    rows = self.master[m.moff:m.moff + m.rows * m.k].view(m.rows, m.k)
                    rows.copy_(s.param.detach()[rank * m.rows:(rank + 1) * m.rows].to(device, torch.float32))
                    s.param.data = rows            # the full weight is gone from this rank
                    s.param.ws_sharded = m
                s.param.grad = None if m is not None else g
                s.param.main_grad = g
        a.refresh_bf16()
        if sync is not None:
            sync.attach(a, model)
            if hasattr(sync, "segments"):
                sync.segments = dict(a.segments)
        # ---- landing slots and streams (GPU)
        self.version = 0
        self.n_cores = len(model.cores)
        self.by_core: dict[int, dict[str, Matrix]] = {}
        for m in a.matrices:
            self.by_core.setdefault(m.core, {})[m.kind] = m
        if self.cuda:
            shapes = {kind: (m.n, m.k) for kind, m in self.by_core[0].items()}
            count = self.n_cores if mode == "resident" else min(2, self.n_cores)
            self.slots = [_Slot(shapes, device) for _ in range(count)]
            self.side = torch.cuda.Stream(device=device)
            self.gather_ctas = int(os.environ.get("WARPSTATE_GATHER_CTAS", 24))
            from ..ops import gemm as G
            self.error_flag = G.error_flag(device)
            for index, core in enumerate(model.cores):
                core.ws_weights = CoreWeights(self, index)
        self.full_cache: dict[str, torch.Tensor] = {}
        self.optimizer = ShardedParamAdamW(self, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                           max_grad_norm=max_grad_norm)
        self.publish()

    # ------------------------------------------------------------------ landing slots (GPU)
    def shard_ptrs(self, m: Matrix) -> list[int]:
        return [p + 4 * m.moff for p in self.master_ptrs]

    def _slot(self, core: int) -> _Slot:
        slot = self.slots[core % len(self.slots)]
        if slot.core != core or slot.version != self.version:
            slot.core, slot.version, slot.have = core, self.version, {}
        return slot

    def fetch(self, core: int, kinds) -> None:
        """Start gathering the named matrices of ``core`` on the side stream (no-op for what is there)."""
        slot = self._slot(core)
        missing = [k for k in kinds if k not in slot.have]
        if not missing:
            return
        main = torch.cuda.current_stream(self.device)
        if slot.last_use is not None:
            self.side.wait_event(slot.last_use)          # the slot's previous readers are done
        else:
            self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            for kind in missing:
                m = self.by_core[core][kind]
                torch.ops.ws_b200.gather_cast(self.shard_ptrs(m), m.rows, slot.w[kind], self.gather_ctas)
                event = torch.cuda.Event()
                event.record(self.side)
                slot.have[kind] = event

    def weight(self, core: int, kind: str) -> torch.Tensor:
        """The BF16 weight, usable on the current stream."""
        slot = self._slot(core)
        if kind not in slot.have:
            self.fetch(core, (kind,))
        event = slot.have[kind]
        if event is not None:
            torch.cuda.current_stream(self.device).wait_event(event)
            slot.have[kind] = None
        return slot.w[kind]

    def fused_linear(self, core: int, kind: str, z: torch.Tensor):
        """``z @ W^T`` (``in``) or the SwiGLU pair (``ug``): when the slot does not hold W yet, ONE launch
        gathers the owners' FP32 rows, casts them into the slot and multiplies."""
        from ..ops import gemm as G
        slot = self._slot(core)
        m = self.by_core[core][kind]
        swiglu = kind == "ug"
        if kind in slot.have:
            w = self.weight(core, kind)
            return G.linear_swiglu(z, w) if swiglu else G.linear(z, w)
        out, act = torch.ops.ws_b200.gather_cast_linear(z, self.shard_ptrs(m), m.n // 2 if swiglu else m.n, m.rows,
                                                        slot.w[kind], slot.flags[kind], self.error_flag, 2.0, swiglu, True)
        slot.have[kind] = None
        return (out, act) if swiglu else out

    def mark_used(self, core: int) -> None:
        slot = self.slots[core % len(self.slots)]
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(self.device))
        slot.last_use = event

    def publish(self) -> None:
        """After the owners changed their rows: order the change before any peer's next gather and
        invalidate every landing slot."""
        self.version += 1
        self.full_cache.clear()
        if self.world > 1:
            if self.fused_comm:
                self.sync.node_barrier()
            elif self.cuda:
                torch.cuda.current_stream(self.device).synchronize()
                dist.barrier(group=self.group)

    # ------------------------------------------------------------------ CPU / collective path
    def gather_full(self, m: Matrix) -> torch.Tensor:
        """The whole FP32 ``[n, k]`` weight from every rank's rows (collective)."""
        rows = self.master[m.moff:m.moff + m.rows * m.k]
        if self.world == 1:
            return rows.view(m.n, m.k).clone()
        parts = [torch.empty_like(rows) for _ in range(self.world)]
        dist.all_gather(parts, rows.contiguous(), group=self.group)
        return torch.cat(parts).view(m.n, m.k)

    def before_micro(self) -> None:
        """CPU path: give the PyTorch modules whole weights for this micro-batch."""
        if self.cuda:
            return
        for m in self.arena.matrices:
            full = self.full_cache.get(m.name)
            if full is None:
                full = self.full_cache[m.name] = self.gather_full(m)
            m.param.data = full

    def after_micro(self) -> None:
        if self.cuda:
            return
        self.arena.collect_stray_grads()
        for m in self.arena.matrices:
            m.param.grad = None
            m.param.data = self.master[m.moff:m.moff + m.rows * m.k].view(m.rows, m.k)

    # ------------------------------------------------------------------ checkpoints
    def model_state_dict(self) -> dict[str, torch.Tensor]:
        """Unsharded FP32 state dict under the reference's keys (collective: every rank calls it)."""
        state = {}
        for name, tensor in self.model.state_dict().items():
            m = self.arena.matrix_by_name.get(name)
            state[name] = self.gather_full(m).cpu() if m is not None else tensor.detach().cpu().clone()
        return state

    def load_model_state_dict(self, state: dict[str, torch.Tensor]) -> None:
        """Adopt an unsharded state dict: every rank keeps the rows it owns."""
        a = self.arena
        with torch.no_grad():
            for s in a.slots:
                src = state[s.name]
                m = a.matrix_by_name.get(s.name)
                if m is None:
                    s.param.data.copy_(src.to(self.device, torch.float32))
                else:
                    if tuple(src.shape) != (m.n, m.k):
                        raise ValueError(f"{s.name}: checkpoint shape {tuple(src.shape)} != {(m.n, m.k)}")
                    rows = self.master[m.moff:m.moff + m.rows * m.k].view(m.rows, m.k)
                    rows.copy_(src[self.rank * m.rows:(self.rank + 1) * m.rows].to(self.device, torch.float32))
        a.refresh_bf16()
        self.publish()

    def memory_report(self) -> dict[str, float]:
        """GiB this rank holds per kind of training state."""
        gib = 2.0 ** 30
        o = self.optimizer
        landing = sum(w.numel() * 2 for slot in getattr(self, "slots", []) for w in slot.w.values())
        return {"master_rows_gib": self.master.numel() * 4 / gib,
                "replicated_master_gib": self.arena.master.numel() * 4 / gib,
                "replicated_bf16_gib": (self.arena.bf16.numel() * 2 / gib) if self.arena.bf16 is not None else 0.0,
                "moments_gib": 2 * (o.m_sh.numel() + o.m_rep.numel()) * 4 / gib,
                "grad_arena_gib": self.arena.grad.numel() * 4 / gib,
                "landing_bf16_gib": landing / gib}


class ShardedParamAdamW:
    """AdamW over the owned rows and the replicated rest (same rule and defaults as the replicated
    `optim.ArenaAdamW`; torch-format state dicts, gathered)."""

    def __init__(self, state: ShardedParamState, lr, betas, eps, weight_decay, max_grad_norm):
        self.state = state
        self.arena = state.arena
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        a = state.arena
        dev = state.device
        self.m_sh = torch.zeros(a.shard_numel, dtype=torch.float32, device=dev)
        self.v_sh = torch.zeros(a.shard_numel, dtype=torch.float32, device=dev)
        self.m_rep = torch.zeros(a.rep_numel, dtype=torch.float32, device=dev)
        self.v_rep = torch.zeros(a.rep_numel, dtype=torch.float32, device=dev)
        self.last_stats = None

    def zero_grad(self, set_to_none: bool = False) -> None:
        self.arena.zero_grad()

    def owned_grad(self, m: Matrix) -> torch.Tensor:
        lo = m.goff + self.state.rank * m.rows * m.k
        return self.arena.grad[lo:lo + m.rows * m.k]

    def clip_stats(self, extra_sumsq=None, status=None) -> torch.Tensor:
        """Collective-synchroniser path: after the all-reduce every rank holds the whole averaged gradient,
        so the norm is local (and identical everywhere).  The fused path takes its statistics from the
        reduce kernels instead (`FusedGradSync.exchange_stats`)."""
        max_norm = self.max_grad_norm if self.max_grad_norm is not None else 0.0
        g = self.arena.grad
        if g.is_cuda:
            from ..ops import _ext
            if _ext.available():
                return torch.ops.ws_b200.grad_norm_clip(g, float(max_norm), extra_sumsq, status)
        sumsq = g.double().pow(2).sum().float()
        if extra_sumsq is not None:
            sumsq = sumsq + extra_sumsq.reshape(())
        return host_clip_stats(sumsq, max_norm, status)

    def _segments(self):
        """(parameter, gradient, exp_avg, exp_avg_sq, bf16 or None) flat views, one per contiguous run."""
        a, st = self.arena, self.state
        for gstart, count, mstart in a.rep_runs:
            yield (a.master[mstart:mstart + count], a.grad[gstart:gstart + count], self.m_rep[mstart:mstart + count],
                   self.v_rep[mstart:mstart + count], a.bf16[mstart:mstart + count] if a.bf16 is not None else None)
        for m in a.matrices:
            n = m.rows * m.k
            yield (st.master[m.moff:m.moff + n], self.owned_grad(m), self.m_sh[m.moff:m.moff + n],
                   self.v_sh[m.moff:m.moff + n], None)

    @torch.no_grad()
    def step(self, lr: float | None = None, stats: torch.Tensor | None = None) -> torch.Tensor:
        if lr is not None:
            self.lr = lr
        if stats is None:
            stats = self.clip_stats()
        self.last_stats = stats
        self.step_count += 1
        b1, b2 = self.betas
        kernels = False
        if self.state.cuda:
            from ..ops import _ext
            kernels = _ext.available()
        if not kernels and float(stats[3]) != 0.0:
            return stats
        for p, g, m, v, pb in self._segments():
            if kernels:
                torch.ops.ws_b200.adamw_step(p, g, m, v, pb, float(self.lr), b1, b2, self.eps, self.weight_decay,
                                             self.step_count, stats[1:2], 1.0, stats[3:4])
            else:
                host_adamw(p, g * stats[1], m, v, self.lr, b1, b2, self.eps, self.weight_decay, self.step_count)
                if pb is not None:
                    pb.copy_(p)
        self.state.publish()
        return stats

    def rollback_step(self) -> None:
        self.step_count = max(0, self.step_count - 1)

    # ------------------------------------------------------------------ torch-compatible, unsharded state
    def _gather_rows(self, m: Matrix, flat: torch.Tensor) -> torch.Tensor:
        rows = flat[m.moff:m.moff + m.rows * m.k]
        st = self.state
        if st.world == 1:
            return rows.view(m.n, m.k).cpu().clone()
        parts = [torch.empty_like(rows) for _ in range(st.world)]
        dist.all_gather(parts, rows.contiguous(), group=st.group)
        return torch.cat(parts).view(m.n, m.k).cpu()

    def state_dict(self) -> dict:
        """Same structure as ``torch.optim.AdamW.state_dict()`` over the whole model (collective)."""
        a = self.arena
        state = {}
        for index, (name, _p) in enumerate(a.order):
            if self.step_count == 0:
                continue
            s = a.by_name[name]
            m = a.matrix_by_name.get(name)
            if m is None:
                off = a.rep_offset(s)
                avg = self.m_rep[off:off + s.numel].view(s.shape).cpu().clone()
                sq = self.v_rep[off:off + s.numel].view(s.shape).cpu().clone()
            else:
                avg, sq = self._gather_rows(m, self.m_sh), self._gather_rows(m, self.v_sh)
            state[index] = {"step": torch.tensor(float(self.step_count)), "exp_avg": avg, "exp_avg_sq": sq}
        group = {"lr": self.lr, "betas": tuple(self.betas), "eps": self.eps, "weight_decay": self.weight_decay,
                 "amsgrad": False, "maximize": False, "foreach": None, "capturable": False,
                 "differentiable": False, "fused": True, "decoupled_weight_decay": True,
                 "params": list(range(len(a.order)))}
        return {"state": state, "param_groups": [group]}

    def load_state_dict(self, sd: dict) -> None:
        a, st = self.arena, self.state
        group = sd["param_groups"][0]
        self.lr = group.get("lr", self.lr)
        self.betas = tuple(group.get("betas", self.betas))
        self.eps = group.get("eps", self.eps)
        self.weight_decay = group.get("weight_decay", self.weight_decay)
        steps = set()
        for t in (self.m_sh, self.v_sh, self.m_rep, self.v_rep):
            t.zero_()
        for index, (name, _p) in enumerate(a.order):
            entry = sd["state"].get(index)
            if entry is None:
                continue
            s = a.by_name[name]
            m = a.matrix_by_name.get(name)
            for key, rep, sh in (("exp_avg", self.m_rep, self.m_sh), ("exp_avg_sq", self.v_rep, self.v_sh)):
                src = entry[key]
                if m is None:
                    off = a.rep_offset(s)
                    rep[off:off + s.numel].copy_(src.reshape(-1).to(rep.device, rep.dtype))
                else:
                    rows = src.reshape(m.n, m.k)[st.rank * m.rows:(st.rank + 1) * m.rows]
                    sh[m.moff:m.moff + m.rows * m.k].copy_(rows.reshape(-1).to(sh.device, sh.dtype))
            steps.add(int(float(entry["step"])))
        if len(steps) > 1:
            raise ValueError(f"optimizer state has parameters at different steps: {sorted(steps)}")
        self.step_count = steps.pop() if steps else 0
