"""Training engine: one optimizer update = gradient accumulation over micro-batches, gradient
synchronisation, clip, AdamW, loss reduction.

Semantics follow the reference hot loop (run_40b.py:719-764):

* each micro-batch's mean loss is scaled by ``valid * world / target`` before backward so that
  the data-parallel *average* of gradients equals the gradient of the global token-mean loss;
* ranks whose slice of the final update is empty still run forward/backward (all labels masked
  gives a finite zero loss) so that collectives stay matched;
* gradients are synchronised only for the last micro-batch (earlier ones accumulate locally);
* clip to global norm 1.0, AdamW, then the scalar ``loss_sum`` is summed over ranks.

Differences that are deliberate: gradients live in a flat FP32 arena and are accumulated by the
dW GEMM epilogues; clip/AdamW/BF16 re-cast are three kernels; the non-finite check reads the
norm together with the loss (one host sync per update).
"""
from __future__ import annotations

import contextlib
import math
import time
from dataclasses import dataclass, field
from typing import Callable, Iterable

import torch

from ..data.tokens import HostBatcher, update_slices
from ..optim import ArenaAdamW, ParamArena
from ..ops import fused


@dataclass
class UpdateResult:
    loss: float
    grad_norm: float
    tokens: int
    seconds: float
    clip_coef: float = 1.0
    extras: dict = field(default_factory=dict)


def autocast_for(device: torch.device, enabled: bool = True):
    if device.type == "cuda" and enabled:
        return torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=False)
    return contextlib.nullcontext()


class Trainer:
    """Owns the arena, the optimizer and the gradient synchroniser of one rank."""

    def __init__(self, model: torch.nn.Module, *, device: torch.device, rank: int = 0, world_size: int = 1,
                 lr: float = 1.5e-4, weight_decay: float = 0.1, betas=(0.9, 0.95), eps: float = 1e-8,
                 max_grad_norm: float | None = 1.0, grad_sync=None, bf16_autocast: bool = True,
                 process_group=None, shard_optimizer: bool = False, shard_params: str | None = None,
                 bucket_cap_bytes: int = 0):
        """``shard_params``: None (replicated parameters), ``"stream"`` or ``"resident"`` -- parameters,
        gradients and optimizer state of the core projections sharded over the ranks
        (`parallel.fsdp.ShardedParamState`)."""
        self.model = model
        self.device = device
        self.rank, self.world_size = rank, world_size
        self.bf16_autocast = bf16_autocast
        self.process_group = process_group
        if grad_sync is None and world_size > 1:
            from ..parallel.grad_sync import make_grad_sync
            grad_sync = make_grad_sync(device, world_size, rank, process_group, bucket_cap_bytes=bucket_cap_bytes)
        self.sync = grad_sync
        self.sharded = None
        if shard_params:
            from ..parallel.fsdp import ShardedParamState
            self.sharded = ShardedParamState(model, device=device, rank=rank, world=world_size, group=process_group,
                                             sync=grad_sync, mode=shard_params, lr=lr, betas=betas, eps=eps,
                                             weight_decay=weight_decay, max_grad_norm=max_grad_norm)
            self.arena, self.optimizer = self.sharded.arena, self.sharded.optimizer
        else:
            alloc = grad_sync.alloc_grad_buffer if grad_sync is not None else None
            self.arena = ParamArena(model, device=device, symmetric_alloc=alloc, bucket_cap_bytes=bucket_cap_bytes)
            if self.sync is not None:
                self.sync.attach(self.arena, model)
            if shard_optimizer and world_size > 1:
                from ..parallel.zero import ShardedAdamW
                self.optimizer = ShardedAdamW(self.arena, rank=rank, world=world_size, group=process_group,
                                              sync=self.sync, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                              max_grad_norm=max_grad_norm)
            else:
                self.optimizer = ArenaAdamW(self.arena, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                            max_grad_norm=max_grad_norm)
        self.loss_sum = torch.zeros((), dtype=torch.float32, device=device)
        self.loss_in_stats = False

    # ------------------------------------------------------------------ pieces of one update
    def begin_update(self) -> None:
        self.arena.zero_grad()
        self.loss_sum.zero_()
        if self.sync is not None:
            self.sync.begin_update()

    def micro_step(self, loss_fn: Callable[[], tuple[torch.Tensor, float]], last: bool) -> None:
        """``loss_fn() -> (loss tensor, weight)``; backward of ``loss * weight``."""
        ctx = self.sync.last_micro_batch() if (self.sync is not None and last) else contextlib.nullcontext()
        if self.sharded is not None:
            self.sharded.before_micro()
        with ctx:
            with autocast_for(self.device, self.bf16_autocast):
                loss, weight, report = loss_fn()
            (loss * weight).backward()
        if self.sharded is not None:
            self.sharded.after_micro()
        self.loss_sum += loss.detach().float() * report

    def finish_update(self, lr: float) -> torch.Tensor:
        """Synchronise gradients, clip, step.  Returns device stats ``[norm, coef, norm^2, skip, loss, ...]``.

        The update is gated on the device: when the gradient norm is not finite, or a bounded wait of the
        gradient exchange ran out, ``stats[3]`` is set and the optimizer kernels change nothing.  The host
        learns of it in `read_update_scalars` (the one read per update) and raises there with parameters
        and moments still those of the previous update -- the reference raises before ``optimizer.step``
        too (``clip_grad_norm_(error_if_nonfinite=True)``, run_40b.py:751)."""
        self.arena.collect_stray_grads()
        partials = self.sync.finish_update() if self.sync is not None else None
        max_norm = self.optimizer.max_grad_norm if self.optimizer.max_grad_norm is not None else 0.0
        self.loss_in_stats = partials is not None
        if partials is not None:
            # fused synchroniser: its kernels left per-CTA sums of squares; one launch combines them and the loss
            stats = self.sync.exchange_stats(partials, max_norm, self.loss_sum)
        else:
            status = self.sync.status_word() if self.sync is not None else None
            stats = self.optimizer.clip_stats(None, status)
        self.optimizer.step(lr=lr, stats=stats)
        if self.sync is not None and not self.loss_in_stats:
            self.sync.reduce_scalar(self.loss_sum)
        return stats

    def gather_for_checkpoint(self) -> None:
        """With a sharded optimizer: make the FP32 master weights whole on this rank (collective)."""
        gather = getattr(self.optimizer, "gather_master", None)
        if gather is not None:
            gather()

    def model_state_dict(self) -> dict:
        """The model's unsharded state dict under the reference's keys (collective when anything is sharded)."""
        if self.sharded is not None:
            return self.sharded.model_state_dict()
        self.gather_for_checkpoint()
        return self.model.state_dict()

    def load_model_state_dict(self, state: dict) -> None:
        if self.sharded is not None:
            self.sharded.load_model_state_dict(state)
            return
        self.model.load_state_dict(state)
        self.arena.refresh_bf16()

    def read_update_scalars(self, stats: torch.Tensor):
        """One device->host read per update: loss, gradient norm, clip coefficient, the skip flag and, with a
        fused gradient synchroniser, its error word.  Raises when the device skipped the update."""
        loss = stats[4] if getattr(self, "loss_in_stats", False) else self.loss_sum
        items = [loss, stats[0], stats[1], stats[3]]
        word = self.sync.status_word() if self.sync is not None else None
        if word is not None:
            items.append(word.float())
        host = torch.stack([t.reshape(()).float() for t in items]).tolist()
        if word is not None and host[4] != 0:
            self.optimizer.rollback_step()
            raise RuntimeError(self.sync.describe_error())
        if host[3] != 0 or not math.isfinite(host[1]):
            self.optimizer.rollback_step()
            raise RuntimeError(f"non-finite gradient norm {host[1]}; the update was skipped")
        return host[0], host[1], host[2]

    # ------------------------------------------------------------------ pretraining update
    def pretrain_update(self, data, cursor: int, target_tokens: int, micro_batch: int, seq_len: int,
                        lr: float, batcher: HostBatcher | None = None) -> UpdateResult:
        """One optimizer update over ``target_tokens`` global tokens starting at ``cursor``."""
        t0 = time.perf_counter()
        micro_tokens = micro_batch * seq_len
        slices = list(update_slices(target_tokens, micro_tokens, self.world_size, self.rank))
        batcher = batcher or HostBatcher(micro_batch, seq_len, self.device)
        self.begin_update()
        handle = batcher.stage(data, cursor + slices[0][0], slices[0][1])
        for index, (offset, valid) in enumerate(slices):
            x, y = batcher.take(handle)
            current = handle
            if index + 1 < len(slices):
                handle = batcher.stage(data, cursor + slices[index + 1][0], slices[index + 1][1])

            def loss_fn(x=x, y=y, valid=valid):
                _, loss = self.model(x, y, return_logits=False)
                return loss, valid * self.world_size / target_tokens, valid / target_tokens

            self.micro_step(loss_fn, last=index == len(slices) - 1)
            batcher.release(current)
        stats = self.finish_update(lr)
        loss, norm, coef = self.read_update_scalars(stats)  # the one host sync
        return UpdateResult(loss=loss, grad_norm=norm, tokens=target_tokens,
                            seconds=time.perf_counter() - t0, clip_coef=coef)

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def evaluate_tokens(self, data, cursors: Iterable[int], micro_batch: int, seq_len: int) -> float:
        """Mean next-token loss over fixed windows (the reference evaluates on rank 0 with the
        raw model at evenly spaced cursors, run_40b.py:650-669)."""
        was_training = self.model.training
        self.model.eval()
        total = 0.0
        count = 0
        from ..data.tokens import batches
        for cursor in cursors:
            x, y = batches(data, int(cursor), micro_batch, seq_len, micro_batch * seq_len, self.device)
            with autocast_for(self.device, self.bf16_autocast):
                _, loss = self.model(x, y, return_logits=False)
            value = float(loss)
            if not math.isfinite(value):
                raise RuntimeError("non-finite validation loss")
            total += value
            count += 1
        self.model.train(was_training)
        return total / max(1, count)
