"""Capture / replay evidence for the decode engine's CUDA graph.

The reference counts CUDA-graph captures and replays of its compiled training step through private
Inductor hooks (reference ops/cudagraph_diagnostics.py:17-88) to tell a benchmark that really replays
graphs from one that silently fell back to eager launches.  This framework captures exactly one kind of
graph -- the decode step of `serve.engine.DecodeEngine`, once per batch size -- with the public
``torch.cuda.CUDAGraph`` API, so the counters live in the engine itself: every capture, replay, eager
step and invalidation is counted where it happens, no CUDA work or synchronisation is added, and a
context manager reports the deltas of an interval.

    with collect_graph_diagnostics(engine) as diag:
        ... decode ...
    diag.snapshot()  ->  {"capture_calls": 1, "replay_calls": 512, "eager_steps": 0, "invalidations": 0,
                          "kernels_per_replay": 198, "replay_calls_by_batch": {"64": 512}}
"""
from __future__ import annotations

from collections import Counter
from contextlib import contextmanager
from dataclasses import dataclass, field


@dataclass
class GraphCounters:
    capture_calls: int = 0          # graphs captured (one per batch size in use)
    replay_calls: int = 0           # steps served by replaying a captured graph
    eager_steps: int = 0            # steps launched kernel by kernel (graphs off, or the CPU path)
    invalidations: int = 0          # captured graphs dropped because the batch size changed
    kernels_per_replay: int = 0     # library kernels recorded by the last capture
    replay_calls_by_batch: Counter = field(default_factory=Counter)

    def as_dict(self) -> dict:
        return {"capture_calls": self.capture_calls, "replay_calls": self.replay_calls, "eager_steps": self.eager_steps,
                "invalidations": self.invalidations, "kernels_per_replay": self.kernels_per_replay,
                "replay_calls_by_batch": {str(k): v for k, v in sorted(self.replay_calls_by_batch.items())}}


class GraphDiagnostics:
    """Deltas of an engine's counters since the context was entered."""

    def __init__(self, counters: GraphCounters):
        self._counters = counters
        self._start = counters.as_dict()

    def snapshot(self) -> dict:
        now = self._counters.as_dict()
        out = {}
        for key, value in now.items():
            if key == "replay_calls_by_batch":
                before = self._start[key]
                out[key] = {b: n - before.get(b, 0) for b, n in value.items() if n - before.get(b, 0)}
            elif key == "kernels_per_replay":
                out[key] = value
            else:
                out[key] = value - self._start[key]
        return out


@contextmanager
def collect_graph_diagnostics(engine):
    yield GraphDiagnostics(engine.graph_counters)
