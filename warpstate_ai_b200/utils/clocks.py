"""Read-only GPU clock / throttle sampling with nvidia-smi during a timed region.

Nothing here changes a GPU setting.  `ClockSampler` starts ``nvidia-smi -lms`` as a child
process, stops exactly that process, and summarises SM clocks and the active clock-event reasons
(the reference logs the same telemetry around its GEMM benchmark, ops/benchmark_gemm.py:106-114).
"""
from __future__ import annotations

import shutil
import statistics
import subprocess
import tempfile

FIELDS = ["index", "clocks.sm", "clocks.max.sm", "power.draw", "clocks_event_reasons.active",
          "clocks_event_reasons.hw_slowdown", "clocks_event_reasons.hw_thermal_slowdown",
          "clocks_event_reasons.sw_thermal_slowdown", "clocks_event_reasons.sw_power_cap"]
REASONS = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]


class ClockSampler:
    def __init__(self, period_ms: int = 200):
        self.period_ms = period_ms
        self.proc = None
        self.file = None

    def start(self) -> None:
        if shutil.which("nvidia-smi") is None:
            return
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = subprocess.Popen(
            ["nvidia-smi", f"--query-gpu={','.join(FIELDS)}", "--format=csv,noheader,nounits",
             "-lms", str(self.period_ms)], stdout=self.file, stderr=subprocess.DEVNULL)

    def stop(self, gpu_indices=None) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        return summarise(self.file.read(), gpu_indices)


def summarise(text: str, gpu_indices=None) -> dict:
    clocks, maxes, powers = [], [], []
    reasons = set()
    for line in text.splitlines():
        parts = [p.strip() for p in line.split(",")]
        if len(parts) < len(FIELDS):
            continue
        try:
            index = int(parts[0])
            sm = float(parts[1])
            mx = float(parts[2])
        except ValueError:
            continue
        if gpu_indices is not None and index not in gpu_indices:
            continue
        try:
            power = float(parts[3])
        except ValueError:
            power = 0.0
        clocks.append((sm, power))
        maxes.append(mx)
        powers.append(power)
        for name, value in zip(REASONS, parts[5:9]):
            if value.lower().startswith("active"):
                reasons.add(name)
    if not clocks:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    # "under load": samples drawing at least half of the peak power seen
    peak = max(powers) if powers else 0.0
    loaded = [c for c, p in clocks if p >= 0.5 * peak] or [c for c, _ in clocks]
    return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(maxes), "reasons": sorted(reasons),
            "samples": len(clocks), "power_w_max": peak}
