"""CPU tests of the benchmark / analysis tools: training benchmark records, run comparison,
communication-overlap analysis on synthetic traces, loss-curve fits on synthetic curves
(reference test_analyze_communication_profile.py, test_compare_communication_benchmarks.py)."""
import json
import math
from pathlib import Path

import numpy as np
import pytest

from warpstate_ai_b200.analysis import loss_forecast as LF
from warpstate_ai_b200.bench import comm_profile as CP
from warpstate_ai_b200.bench import compare_runs as CR
from warpstate_ai_b200.bench import train_bench as TB


def kernel(name, ts, dur, device=0, **args):
    return {"ph": "X", "cat": "kernel", "name": name, "ts": ts, "dur": dur, "args": {"device": device, **args}}


def test_sweep_separates_exposed_and_hidden_communication():
    events = [kernel("gemm2_kernel", 0, 100), kernel("attn_bwd_kernel", 150, 50),
              kernel("ncclDevKernel_AllReduce_Sum_f32", 80, 40, **{"Process Group Name": "0", "Seq": 7,
                     "Collective name": "allreduce", "In msg nelems": 1024, "dtype": "Float"}),
              kernel("ncclDevKernel_AllReduce_Sum_f32", 85, 30, **{"Process Group Name": "0", "Seq": 7,
                     "Collective name": "allreduce", "In msg nelems": 1024, "dtype": "Float"}),
              kernel("ws::grad_reduce_kernel(ws::PeerTable, float*)", 190, 30),
              {"ph": "X", "cat": "gpu_memcpy", "name": "Memcpy HtoD", "ts": 300, "dur": 10, "args": {"device": 0}},
              {"ph": "X", "cat": "gpu_user_annotation", "name": "range", "ts": 0, "dur": 500, "args": {"device": 0}},
              {"ph": "X", "cat": "cpu_op", "name": "c10d::allreduce_", "ts": 1, "dur": 1, "args": {"Input Dims": [[1024]]}}]
    report = CP.summarize_trace({"traceEvents": events, "distributedInfo": {"rank": 1}})
    d = report["devices"][0]
    assert report["rank"] == 1 and report["excluded_gpu_annotation_ranges"] == 1
    # compute: [0,100] [150,200] [300,310]; communication: [80,120] [190,220]
    assert d["compute_communication_overlap_us"] == pytest.approx(20 + 10)
    assert d["communication_only_us"] == pytest.approx(20 + 20)
    assert d["compute_only_us"] == pytest.approx(80 + 40 + 10)
    assert d["idle_within_activity_span_us"] == pytest.approx(30 + 80)
    assert d["activity_span_us"] == pytest.approx(310)
    assert d["communication_overlap_fraction"] == pytest.approx(30 / 70)
    assert d["collective_call_count"] == 1 and d["logical_input_payload_bytes"] == 4096  # two channel kernels, one call
    assert d["own_collective_kernels"] == {"ws::grad_reduce_kernel": 1}
    assert report["cpu_collective_fingerprint"]["call_count"] == 1
    with pytest.raises(ValueError):
        CP.summarize_trace({"traceEvents": [kernel("k", 0, -1)]})


def test_comm_profile_cli_refuses_to_overwrite(tmp_path):
    trace = tmp_path / "profile-rank-3-trace.json"
    trace.write_text(json.dumps({"traceEvents": [kernel("gemm2_kernel", 0, 5)]}))
    out = tmp_path / "report.json"
    assert CP.main([str(trace), "--output", str(out)]) == 0
    assert json.loads(out.read_text())["ranks"][0]["rank"] == 3
    with pytest.raises(SystemExit):
        CP.main([str(trace), "--output", str(out)])


@pytest.fixture(scope="module")
def bench_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("bench")
    common = ["--model", "smoke", "--device", "cpu", "--micro-batch", "2", "--seq-len", "128",
              "--global-tokens-per-update", "512", "--warmup-updates", "1", "--measured-updates", "2"]
    for name in ("a", "b"):
        assert TB.main(common + ["--output-dir", str(root / name)]) == 0
    assert TB.main(common + ["--output-dir", str(root / "profiled"), "--profile", "--diagnose-stalls"]) == 0
    return root


def test_train_bench_records(bench_dirs):
    summary = json.loads((bench_dirs / "a/summary.json").read_text())
    assert summary["format"] == "warpstate-training-benchmark-v1" and len(summary["updates"]) == 2
    rows = [json.loads(l) for l in (bench_dirs / "a/rank-0.jsonl").read_text().splitlines()]
    assert [r["measured"] for r in rows] == [False, True, True]
    assert all(math.isfinite(r["loss"]) and r["tokens_per_second"] > 0 for r in rows)
    prof = json.loads((bench_dirs / "profiled/summary.json").read_text())["profile"]
    assert Path(prof["trace"]).exists() and (bench_dirs / "profiled/profile-rank-0-kernels.tsv").exists()
    stalls = [json.loads(l) for l in (bench_dirs / "profiled/rank-0.jsonl").read_text().splitlines()][-1]
    assert {"forward_backward", "sync_clip_step", "read_back"} <= set(stalls["host_stage_seconds"])


def test_train_bench_records_the_reference_execution_flags_it_ignores(tmp_path):
    common = ["--model", "smoke", "--device", "cpu", "--micro-batch", "2", "--seq-len", "128", "--global-tokens-per-update", "256",
              "--warmup-updates", "0", "--measured-updates", "1"]
    assert TB.main(common + ["--output-dir", str(tmp_path / "a"), "--gradient-mode", "compiled-autograd-overlap", "--compile-cores",
                             "--overlap-memory-budget", "0.1", "--blas-backend", "cublaslt", "--cudagraph-diagnostics",
                             "--no-autocast-cache", "--matmul-plan", "plan.json", "--ddp-bucket-cap-mb", "128", "--bf16-residuals"]) == 0
    summary = json.loads((tmp_path / "a/summary.json").read_text())
    assert summary["reference_execution_flags"] == {
        "--gradient-mode": "compiled-autograd-overlap", "--compile-cores": True, "--overlap-memory-budget": 0.1, "--blas-backend": "cublaslt",
        "--cudagraph-diagnostics": True, "--autocast-cache": False, "--matmul-plan": "plan.json"}
    assert summary["bucket_cap_mb"] == 128 and summary["precision"]["residual_stream"] == "bf16"
    assert TB.main(common + ["--output-dir", str(tmp_path / "b")]) == 0
    plain = json.loads((tmp_path / "b/summary.json").read_text())
    assert plain["reference_execution_flags"] == {} and plain["precision"]["residual_stream"] == "fp32"
    assert plain["updates"][0]["loss"] == pytest.approx(summary["updates"][0]["loss"], rel=1e-5)   # nothing that ran changed (host path)
    for bad in (["--loss-chunk-size", "0"], ["--ddp-bucket-cap-mb", "-1"], ["--overlap-memory-budget", "-0.1"], ["--loss-mode", "fused"]):
        with pytest.raises(SystemExit):
            TB.main(common + ["--output-dir", str(tmp_path / "c"), *bad])


def test_compare_runs_pairs_updates_and_rejects_mismatches(bench_dirs, tmp_path):
    out = tmp_path / "cmp.json"
    assert CR.main(["--control", str(bench_dirs / "a"), "--candidate", str(bench_dirs / "b"), "--output", str(out)]) == 0
    report = json.loads(out.read_text())["comparisons"][0]
    assert report["maximum_absolute_loss_difference"] == 0.0  # same seed, same data: same numbers
    assert report["maximum_relative_grad_norm_difference"] == 0.0
    assert len(report["paired_updates"]) == 2 and report["throughput_ratio"] > 0
    assert [p["update"] for p in report["paired_updates"]] == [2, 3]     # numbered from one; the first was warm-up
    assert report["paired_updates"][0]["ranks"][0]["grad_norm_difference"] == 0.0
    assert len(json.loads(out.read_text())["limitations"]) == 5 and not out.with_name("cmp.json.partial").exists()
    # several candidates after one flag, the flag repeated, and the rules on the report's path
    many = tmp_path / "many.json"
    assert CR.main(["--control", str(bench_dirs / "a"), "--candidate", str(bench_dirs / "b"), str(bench_dirs / "a"),
                    "--candidate", str(bench_dirs / "b"), "--output", str(many)]) == 0
    assert [Path(c["candidate"]["directory"]).name for c in json.loads(many.read_text())["comparisons"]] == ["b", "a", "b"]
    for refused in (many, tmp_path / "report.txt"):
        with pytest.raises(SystemExit):
            CR.main(["--control", str(bench_dirs / "a"), "--candidate", str(bench_dirs / "b"), "--output", str(refused)])
    with pytest.raises(ValueError, match="unprofiled"):
        CR.load_run(bench_dirs / "profiled")
    # a run with another geometry is not comparable
    other = tmp_path / "other"
    TB.main(["--model", "smoke", "--device", "cpu", "--micro-batch", "1", "--seq-len", "128",
             "--global-tokens-per-update", "512", "--warmup-updates", "1", "--measured-updates", "2",
             "--output-dir", str(other)])
    with pytest.raises(ValueError, match="geometry"):
        CR.compare(CR.load_run(bench_dirs / "a"), CR.load_run(other))
    # tampered throughput is caught
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "summary.json").write_text((bench_dirs / "a/summary.json").read_text())
    rows = [json.loads(l) for l in (bench_dirs / "a/rank-0.jsonl").read_text().splitlines()]
    rows[1]["tokens_per_second"] *= 2
    (bad / "rank-0.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    with pytest.raises(ValueError, match="throughput"):
        CR.load_run(bad)


def test_loss_forecast_recovers_a_power_law():
    tokens = np.arange(1.0, 8.01, 0.05) * 1e9
    true = {"floor": 1.7, "amplitude": 1.2, "alpha": 0.35}
    rows = [{"tokens": int(t), "loss": true["floor"] + true["amplitude"] * (t / 1e9) ** -true["alpha"]} for t in tokens]
    raw = "\n".join(json.dumps(r) for r in rows).encode()
    report = LF.analyze(raw)
    free = next(f for f in report["fits"] if f["start_B"] == 1 and f["parameters"]["model"] == "power_free")
    # bin means of a convex curve sit slightly above the curve at the mean token count
    assert free["parameters"]["alpha"] == pytest.approx(true["alpha"], rel=0.05)
    assert free["parameters"]["floor"] == pytest.approx(true["floor"], abs=0.05)
    assert free["parameters"]["rmse"] < 1e-3
    expected_cross = (true["amplitude"] / (2.0 - true["floor"])) ** (1 / true["alpha"])
    assert free["cross_2_tokens_B"] == pytest.approx(expected_cross, rel=0.15)
    log = next(f for f in report["fits"] if f["start_B"] == 1 and f["parameters"]["model"] == "log")
    assert log["parameters"]["slope"] < 0 and log["parameters"]["rmse"] > free["parameters"]["rmse"]
    assert len(report["holdouts"]) == 3 * 7
    best = min((h for h in report["holdouts"] if h["train_end_B"] == 6), key=lambda h: h["rmse"])
    assert best["parameters"]["model"].startswith("power")
    with pytest.raises(ValueError):
        LF.analyze(b'{"tokens": 5, "loss": 1}\n{"tokens": 4, "loss": 1}')


def test_tuner_pairing_policy_and_loader(tmp_path):
    from warpstate_ai_b200.bench import tune_gemm as TG
    from warpstate_ai_b200.ops import gemm as G
    trials = [{"control_before_ms": 1.00, "candidate_ms": 0.90, "control_after_ms": 1.02},
              {"control_before_ms": 1.01, "candidate_ms": 0.99, "control_after_ms": 0.99}]
    m = TG.paired_timing_metrics(trials, minimum_gain=0.02)
    assert m["minimum_trial_gain"] == pytest.approx(1.0 / 0.99 - 1) and m["timing_eligible"] is False
    assert TG.paired_timing_metrics(trials, minimum_gain=0.005)["timing_eligible"] is True
    with pytest.raises(ValueError):
        TG.paired_timing_metrics([{"control_before_ms": 1.0, "candidate_ms": 0.0, "control_after_ms": 1.0}], 0.01)
    case = TG.cases(16384, ["fwd", "dw"])[0]
    rows = [{"case": case, "candidate": {"kernel": "single", "sm_limit": 0}, "status": "ok", "eligible": True,
             "paired_gain": 0.02, "tflops": 1300.0},
            {"case": case, "candidate": {"kernel": "pair", "sm_limit": 0}, "status": "ok", "eligible": True,
             "paired_gain": 0.09, "tflops": 1500.0},
            {"case": case, "candidate": {"kernel": "pair", "sm_limit": 116}, "status": "ok", "eligible": False,
             "paired_gain": 0.5, "tflops": 9999.0}]
    policy = TG.select_policy(rows)
    assert len(policy["entries"]) == 1 and policy["entries"][0]["kernel"] == "pair" and policy["entries"][0]["sm_limit"] == 0
    path = tmp_path / "candidate-policy.json"
    path.write_text(json.dumps(policy))
    assert G.load_policy(path) == 1
    assert G._policy_key(False, False, 16384, 10240, 2048) == policy["entries"][0]["key"]
    G._policy.clear()
    assert TG.main(["--list-cases", "--output-dir", str(tmp_path / "x")]) == 0
    # the SwiGLU screening is one problem, keyed like the launch `linear_swiglu` makes (one output tile per up/gate pair)
    fused = TG.cases(16384, ["fwd", "dx", "dw"], kind="swiglu")
    assert len(fused) == 1 and TG.policy_key(fused[0]) == "fwd:16384x7168x2048"
    assert TG.policy_key(TG.cases(16384, ["fwd"])[2]) == "fwd:16384x14336x2048"
    # candidates: the default sweep, one kernel of it, or exactly what --tile names
    assert len(TG.candidates_of(None, None)) == 4 and {c["kernel"] for c in TG.candidates_of(["single"], None)} == {"single"}
    assert TG.candidates_of(["single"], ["pair,116", "single,0"]) == [{"kernel": "pair", "sm_limit": 116}, {"kernel": "single", "sm_limit": 0}]
    for bad in ("pair", "pair,", "triple,4", "pair,149", "pair,-1", "128,128,64,4,3"):
        with pytest.raises(ValueError):
            TG.candidates_of(None, [bad])
        with pytest.raises(SystemExit):
            TG.main(["--list-cases", "--output-dir", str(tmp_path / "x"), "--tile", bad])


def test_profile_step_idle_gap_arithmetic():
    """Interval union: overlapping kernels count once, gaps are reported longest first."""
    from warpstate_ai_b200.bench.profile_step import idle_gaps
    out = idle_gaps([(0.0, 10.0, "a"), (5.0, 20.0, "b"), (30.0, 40.0, "c"), (41.0, 42.0, "d"), (12.0, 15.0, "e")])
    assert abs(out["span_ms"] - 0.042) < 1e-9 and abs(out["busy_ms"] - 0.031) < 1e-9 and abs(out["idle_ms"] - 0.011) < 1e-9
    assert out["n_gaps"] == 2 and out["gaps"][0]["idle_us"] == 10.0
    assert out["gaps"][0]["after"] == "b" and out["gaps"][0]["before"] == "c"
    assert idle_gaps([])["idle_ms"] == 0.0


def test_decode_bench_combines_replicas():
    """Independent decode replicas: throughputs add, latencies take the slowest rank."""
    from warpstate_ai_b200.bench.decode_bench import combine_ranks
    a = {"tokens_per_second": 100.0, "prefill_tokens_per_second": 1000.0, "p50_latency_seconds": 0.002,
         "prefill_seconds": 0.5, "peak_mem_gib": 30.0, "host_driven_p50_seconds": 0.0021}
    b = {"tokens_per_second": 90.0, "prefill_tokens_per_second": 900.0, "p50_latency_seconds": 0.003,
         "prefill_seconds": 0.6, "peak_mem_gib": 31.0, "host_driven_p50_seconds": 0.0032}
    out = combine_ranks([a, b])
    assert out["tokens_per_second"] == 190.0 and out["prefill_tokens_per_second"] == 1900.0
    assert out["p50_latency_seconds"] == 0.003 and out["prefill_seconds"] == 0.6 and out["peak_mem_gib"] == 31.0
    assert out["host_driven_p50_seconds"] == 0.0032
