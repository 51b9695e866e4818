"""Token-stream data path for pretraining.

`batches` and `update_slices` keep the reference's contracts (run_40b.py:347-358, 423-427):
a cyclic contiguous window of ``B*T+1`` tokens starting at an integer cursor, inputs and labels
shifted by one, labels past ``valid`` masked with -100; global update tokens are split into
disjoint per-rank, per-iteration slices and ranks whose slice is empty still run.  Resume state
is the single integer ``tokens_seen``.

`HostBatcher` adds what a saturated B200 needs: reusable pinned staging buffers, non-blocking
copies on a side stream and one-step lookahead, so the H2D copy of micro-batch i+1 overlaps the
compute of micro-batch i.
"""
from __future__ import annotations

import math
from typing import Iterator

import numpy as np
import torch


def window(data, cursor: int, count: int) -> np.ndarray:
    """``count`` tokens starting at ``cursor`` with wrap-around, as int64."""
    n = len(data)
    start = cursor % n
    if start + count <= n:
        return np.asarray(data[start:start + count], dtype=np.int64)
    idx = (np.arange(count, dtype=np.int64) + start) % n
    return np.asarray(data[idx], dtype=np.int64)


def host_batch(data, cursor: int, batch: int, length: int, valid: int):
    tokens = window(data, cursor, batch * length + 1)
    x = torch.from_numpy(tokens[:-1].reshape(batch, length).copy())
    y = torch.from_numpy(tokens[1:].reshape(batch, length).copy())
    y.view(-1)[valid:] = -100
    return x, y


def batches(data, cursor: int, batch: int, length: int, valid: int, device: torch.device):
    """One micro-batch ``(x, y)`` on ``device`` (pinned + non-blocking when CUDA)."""
    x, y = host_batch(data, cursor, batch, length, valid)
    if device.type == "cuda":
        x, y = x.pin_memory(), y.pin_memory()
    return x.to(device, non_blocking=True), y.to(device, non_blocking=True)


def update_slices(target: int, micro_tokens: int, world_size: int, rank: int) -> Iterator[tuple[int, int]]:
    """(offset, valid) per accumulation iteration for this rank; empty slices still yield."""
    for iteration in range(math.ceil(target / (world_size * micro_tokens))):
        offset = (iteration * world_size + rank) * micro_tokens
        yield offset, max(0, min(micro_tokens, target - offset))


class HostBatcher:
    """Pinned staging of micro-batches with a copy stream.  Three slots: the slot that `stage` refills for
    micro-batch k+1 was last read by micro-batch k-2, so the host never waits for the micro-batch the
    device is still working on and the launch queue stays ahead of the GPU."""

    def __init__(self, batch: int, length: int, device: torch.device, depth: int = 3):
        self.batch, self.length, self.device = batch, length, device
        self.cuda = device.type == "cuda"
        self.depth = depth
        self.slot = 0
        self.bytes_per_batch = 2 * batch * length * 8
        if self.cuda:
            self.stream = torch.cuda.Stream(device=device)
            self.pinned = [(torch.empty((batch, length), dtype=torch.int64).pin_memory(),
                            torch.empty((batch, length), dtype=torch.int64).pin_memory()) for _ in range(depth)]
            self.dev = [(torch.empty((batch, length), dtype=torch.int64, device=device),
                         torch.empty((batch, length), dtype=torch.int64, device=device)) for _ in range(depth)]
            self.ready = [torch.cuda.Event() for _ in range(depth)]
            self.consumed = [torch.cuda.Event() for _ in range(depth)]

    def stage(self, data, cursor: int, valid: int):
        """Start the transfer of one micro-batch; returns a handle for `take`."""
        x, y = host_batch(data, cursor, self.batch, self.length, valid)
        if not self.cuda:
            return (x, y)
        i = self.slot
        self.slot = (self.slot + 1) % self.depth
        self.consumed[i].synchronize()  # the device finished reading this slot's previous contents
        px, py = self.pinned[i]
        px.copy_(x)
        py.copy_(y)
        with torch.cuda.stream(self.stream):
            self.dev[i][0].copy_(px, non_blocking=True)
            self.dev[i][1].copy_(py, non_blocking=True)
            self.ready[i].record(self.stream)
        return i

    def take(self, handle):
        if not self.cuda:
            return handle
        torch.cuda.current_stream(self.device).wait_event(self.ready[handle])
        return self.dev[handle]

    def release(self, handle) -> None:
        if self.cuda:
            self.consumed[handle].record(torch.cuda.current_stream(self.device))


class SyntheticTokens:
    """Uniform-random token stream in [0, vocab) with the memmap interface (len, slicing)."""

    def __init__(self, n_tokens: int, vocab: int, seed: int = 0):
        rng = np.random.default_rng(seed)
        self.array = rng.integers(0, vocab, size=n_tokens, dtype=np.uint16 if vocab <= 65536 else np.int32)

    def __len__(self) -> int:
        return len(self.array)

    def __getitem__(self, key):
        return self.array[key]
