"""Small shared utilities: rule tables, the read-only clock summary and the decode graph counters."""
import math

import pytest
import torch

from warpstate_ai_b200.serve.graph_stats import GraphCounters, collect_graph_diagnostics
from warpstate_ai_b200.utils import clocks
from warpstate_ai_b200.utils.rules import Rule, enforce, finite, fp32_tensors, matches


# ------------------------------------------------------------------------------------------- rules
def test_enforce_reports_the_first_rule_that_does_not_hold():
    seen = []

    def rule(name, value):
        def holds():
            seen.append(name)
            return value
        return Rule(f"{name} failed", holds)

    enforce([rule("a", True), rule("b", 1)])
    assert seen == ["a", "b"]
    seen.clear()
    with pytest.raises(ValueError, match="^b failed$"):
        enforce([rule("a", True), rule("b", False), rule("c", False)])
    assert seen == ["a", "b"]                                   # later rules are not evaluated

    class Refused(Exception):
        pass

    with pytest.raises(Refused, match="c failed"):
        enforce([rule("c", 0)], Refused)


def test_a_rule_that_cannot_be_evaluated_does_not_hold():
    report = {"status": "ok", "nested": None}
    with pytest.raises(ValueError, match="missing key"):
        enforce([Rule("missing key", lambda: report["absent"] == 1)])
    with pytest.raises(ValueError, match="not a mapping"):
        enforce([Rule("not a mapping", lambda: report["nested"]["x"] == 1)])
    with pytest.raises(ValueError, match="no attribute"):
        enforce([Rule("no attribute", lambda: report.nothing)])
    with pytest.raises(ZeroDivisionError):                     # anything else is a bug in the rule, not a verdict
        enforce([Rule("bug", lambda: 1 / 0)])


def test_finite_and_matches():
    assert finite(0) and finite(-2.5) and finite(10 ** 30)
    assert not any(finite(v) for v in (True, False, None, "1", float("nan"), float("inf"), -math.inf, [1.0]))
    record = {"step": 7, "kind": "sft", "extra": [1]}
    assert matches(record, {"step": 7, "kind": "sft"}) and matches(record, {})
    assert not matches(record, {"step": 7.5}) and not matches(record, {"absent": None})


def test_one_rule_per_floating_point_tensor():
    tensors = {"w": torch.zeros(2), "h": torch.zeros(2, dtype=torch.bfloat16), "i": torch.zeros(2, dtype=torch.int64)}
    rules = fp32_tensors(tensors, "{name} is {dtype}")
    assert [r.message for r in rules] == ["w is torch.float32", "h is torch.bfloat16", "i is torch.int64"]
    assert [bool(r.holds()) for r in rules] == [True, False, True]      # integer tensors are not the rule's business
    with pytest.raises(ValueError, match="h is torch.bfloat16"):
        enforce(rules)


# ------------------------------------------------------------------------------------------- clocks
def line(index, sm, power, *, cap="Not Active", thermal="Not Active", hw="Not Active", max_sm=1965):
    active = "0x0000000000000004" if cap == "Active" else "0x0000000000000000"
    return f"{index}, {sm}, {max_sm}, {power}, {active}, {hw}, Not Active, {thermal}, {cap}"


def test_clock_summary_is_the_median_under_load_with_the_reasons_seen():
    text = "\n".join([
        line(0, 1965, 140.0),                     # idle before the timed region: not "under load"
        line(0, 1410, 980.5, cap="Active"),
        line(0, 1350, 1001.2, cap="Active"),
        line(0, 1290, 995.0, cap="Active"),
        line(1, 1100, 990.0, thermal="Active"),   # another GPU of the box
        "garbage line",
        "x, y, z, 1, 2, 3, 4, 5, 6",
    ])
    mine = clocks.summarise(text, gpu_indices=[0])
    assert mine == {"sm_mhz": 1350, "sm_max_mhz": 1965, "reasons": ["sw_power_cap"], "samples": 4, "power_w_max": 1001.2}
    everyone = clocks.summarise(text)
    assert everyone["samples"] == 5 and everyone["reasons"] == ["sw_power_cap", "sw_thermal_slowdown"]
    assert everyone["sm_mhz"] == 1320                           # median of 1410, 1350, 1290, 1100
    assert clocks.summarise("", [0]) == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    assert clocks.summarise(line(3, 1500, "[N/A]"))["sm_mhz"] == 1500      # no power reading: every sample counts


def test_sampler_without_the_tool_reports_nothing(monkeypatch):
    monkeypatch.setattr(clocks.shutil, "which", lambda name: None)
    sampler = clocks.ClockSampler()
    sampler.start()
    assert sampler.proc is None
    assert sampler.stop([0]) == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


def test_sampler_reads_what_the_tool_printed_and_only_reads(monkeypatch, tmp_path):
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\necho \"$@\" > " + str(tmp_path / "argv") + "\n"
                    "echo '0, 1400, 1965, 900.0, 0x4, Not Active, Not Active, Not Active, Active'\nsleep 30\n")
    fake.chmod(0o755)
    monkeypatch.setenv("PATH", f"{tmp_path}:/usr/bin:/bin")
    sampler = clocks.ClockSampler(period_ms=50)
    sampler.start()
    import time
    for _ in range(100):
        if (tmp_path / "argv").exists():
            break
        time.sleep(0.05)
    time.sleep(0.1)
    summary = sampler.stop([0])
    assert summary["sm_mhz"] == 1400 and summary["reasons"] == ["sw_power_cap"]
    argv = (tmp_path / "argv").read_text().split()
    assert argv == [f"--query-gpu={','.join(clocks.FIELDS)}", "--format=csv,noheader,nounits", "-lms", "50"]   # a query only
    assert sampler.proc.poll() is not None                       # exactly the child it started has been stopped


# ------------------------------------------------------------------------------------------- graph counters
def test_graph_diagnostics_report_the_deltas_of_an_interval():
    class Engine:
        graph_counters = GraphCounters()

    engine = Engine()
    c = engine.graph_counters
    c.capture_calls, c.replay_calls, c.kernels_per_replay = 1, 100, 198
    c.replay_calls_by_batch[64] = 100
    with collect_graph_diagnostics(engine) as diag:
        assert diag.snapshot() == {"capture_calls": 0, "replay_calls": 0, "eager_steps": 0, "invalidations": 0,
                                   "kernels_per_replay": 198, "replay_calls_by_batch": {}}
        c.invalidations += 1
        c.capture_calls += 1
        c.kernels_per_replay = 171
        c.replay_calls += 12
        c.replay_calls_by_batch[16] += 12
        c.eager_steps += 2
        during = diag.snapshot()
    assert during == {"capture_calls": 1, "replay_calls": 12, "eager_steps": 2, "invalidations": 1,
                      "kernels_per_replay": 171, "replay_calls_by_batch": {"16": 12}}
    assert c.as_dict()["replay_calls_by_batch"] == {"16": 12, "64": 100}
    assert GraphCounters().replay_calls_by_batch is not c.replay_calls_by_batch
