"""Differential tests of the analysis and checkpoint tools against the reference's own functions, imported from
``baseline/_ref`` (skipped where it is not installed): chrome-trace overlap analysis, loss-curve fits and the frozen
host snapshot of a training state."""
import copy
import os
from pathlib import Path
import importlib
import json
import random
from collections import OrderedDict

import numpy as np
import pytest
import torch

from test_reference_parity import REF, reference_import_path


@pytest.fixture(scope="module")
def ref():
    if not (REF / "ops" / "analyze_communication_profile.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    with reference_import_path():
        return {name: importlib.import_module(name) for name in
                ("ops.analyze_communication_profile", "ops.loss_curve_forecast", "ops.checkpoint_writer",
                 "ops.compare_communication_benchmarks")}


# ------------------------------------------------------------------------------------------- trace analysis
def synthetic_trace(seed, rank=0):
    rng = random.Random(seed)
    events = []
    clock = 1000.0
    for index in range(120):
        kind = rng.random()
        duration = rng.choice([5.0, 40.0, 250.0, 900.0])
        begin = clock + rng.choice([-30.0, 0.0, 3.0, 60.0])
        if kind < 0.55:
            events.append({"ph": "X", "cat": "kernel", "name": f"gemm_kernel_{index % 5}", "ts": begin, "dur": duration,
                           "args": {"device": 0, "stream": 7}})
        elif kind < 0.8:
            events.append({"ph": "X", "cat": "kernel", "name": "ncclDevKernel_AllReduce_Sum_f32_RING_LL(ncclDevKernelArgsStorage<4096ul>)",
                           "ts": begin, "dur": duration, "args": {"device": 0, "stream": 21}})
        elif kind < 0.9:
            events.append({"ph": "X", "cat": "gpu_memcpy", "name": "Memcpy HtoD", "ts": begin, "dur": duration, "args": {"device": 0, "stream": 9}})
        elif kind < 0.95:
            events.append({"ph": "X", "cat": "gpu_user_annotation", "name": "range", "ts": begin, "dur": duration, "args": {"device": 0}})
        else:
            events.append({"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": begin, "dur": duration})
        clock = begin + duration * rng.choice([0.3, 1.0, 1.0, 1.5])
    events.append({"ph": "i", "name": "marker", "ts": clock})
    events.append({"ph": "X", "cat": "gpu_memset", "name": "Memset", "ts": clock + 5, "dur": 0.0, "args": {"device": 1, "stream": 3}})
    events.append({"ph": "X", "cat": "kernel", "name": "elementwise", "ts": clock + 9, "dur": 12.5, "args": {"device": 1, "stream": 3}})
    return {"traceEvents": events, "distributedInfo": {"rank": rank, "world_size": 2, "backend": "nccl"}}


TIMES = ("activity_span_us", "active_union_us", "idle_within_activity_span_us", "noncommunication_union_us",
         "communication_union_us", "compute_only_us", "compute_communication_overlap_us", "communication_only_us",
         "communication_overlap_fraction", "summed_noncommunication_us", "summed_communication_us")


@pytest.mark.parametrize("seed", range(6))
def test_overlap_analysis_of_a_trace(ref, seed):
    from warpstate_ai_b200.bench import comm_profile as CP
    trace = synthetic_trace(seed, rank=seed % 2)
    mine, theirs = CP.summarize_trace(copy.deepcopy(trace)), ref["ops.analyze_communication_profile"].summarize_trace(trace)
    assert mine["rank"] == theirs["rank"] and mine["distributed_info"] == theirs["distributed_info"]
    assert mine["excluded_gpu_annotation_ranges"] == theirs["excluded_gpu_annotation_ranges"]
    assert [d["device"] for d in mine["devices"]] == [d["device"] for d in theirs["devices"]] == ["0", "1"]
    for a, b in zip(mine["devices"], theirs["devices"]):
        for key in TIMES:
            assert a[key] == pytest.approx(b[key], rel=1e-12, abs=1e-9), (key, a["device"])
        assert a["nccl_kernel_names"] == b["nccl_kernel_names"]
        assert a["nccl_kernel_count"] == b["nccl_kernel_count"]


def test_malformed_activities_are_refused_by_both(ref):
    from warpstate_ai_b200.bench import comm_profile as CP
    for bad in ({"ts": float("nan"), "dur": 1.0}, {"ts": 1.0, "dur": -2.0}, {"ts": "1", "dur": 1.0}, {"ts": 1.0}):
        trace = {"traceEvents": [{"ph": "X", "cat": "kernel", "name": "k", "args": {"device": 0}, **bad}]}
        for function in (CP.summarize_trace, ref["ops.analyze_communication_profile"].summarize_trace):
            with pytest.raises(ValueError):
                function(trace)
    empty = {"traceEvents": []}
    assert CP.summarize_trace(empty)["devices"] == ref["ops.analyze_communication_profile"].summarize_trace(empty)["devices"] == []


# ------------------------------------------------------------------------------------------- loss-curve fits
def test_curve_fits_predictions_and_crossings(ref):
    from warpstate_ai_b200.analysis import loss_forecast as LF
    theirs = ref["ops.loss_curve_forecast"]
    rng = np.random.default_rng(0)
    t = np.linspace(1.0, 9.0, 33)
    curves = [2.0 + 1.3 * t ** -0.4, 1.7 + 0.9 * t ** -0.9 + rng.normal(0, 2e-3, t.size), 3.0 - 0.3 * np.log(t) + rng.normal(0, 1e-3, t.size),
              np.full_like(t, 2.4) + rng.normal(0, 1e-3, t.size)]
    for loss in curves:
        for model in ("log", "power_free", "power_fixed:1.5", "power_fixed:1.9"):
            mine, other = LF.fit(t, loss, model), theirs.fit(t, loss, model)
            assert mine["model"] == other["model"]
            assert mine["rmse"] == pytest.approx(other["rmse"], rel=1e-4, abs=1e-9)                      # same optimum ...
            budgets = [12.0, 40.0, 268.435456]
            assert LF.predict(mine, budgets) == pytest.approx(theirs.predict(other, budgets), rel=2e-3)   # ... same forecast
            for target in (1.0, 2.0, 2.3):
                a, b = LF.crossing(mine, target), theirs.crossing(other, target)
                assert (a is None) == (b is None), (model, target)
                if a is not None and b < 1e6:
                    assert a == pytest.approx(b, rel=0.05)
            if model == "log":
                assert mine["slope"] == pytest.approx(other["slope"], rel=1e-9) and mine["intercept"] == pytest.approx(other["intercept"], rel=1e-9)
    with pytest.raises(ValueError):
        LF.fit(t[:2], curves[0][:2], "log")
    with pytest.raises(ValueError):
        theirs.fit(t[:2], curves[0][:2], "log")


def test_whole_report_on_a_validation_log(ref):
    from warpstate_ai_b200.analysis import loss_forecast as LF
    rows = [{"tokens": int(t * 1e9), "loss": 1.8 + 1.1 * t ** -0.45} for t in np.arange(1.0, 7.31, 0.05)]
    raw = ("\n".join(json.dumps(r) for r in rows) + "\n").encode()
    mine, theirs = LF.analyze(raw), ref["ops.loss_curve_forecast"].analyze(raw)
    assert mine["source_sha256"] == theirs["source_sha256"] and mine["source_rows"] == theirs["source_rows"]
    assert mine["complete_bins_end_B"] == theirs["complete_bins_end_B"] and len(mine["bins"]) == len(theirs["bins"])
    for a, b in zip(mine["bins"], theirs["bins"]):
        assert a["count"] == b["count"] and a["loss"] == pytest.approx(b["loss"], rel=1e-12) and a["tokens_B"] == pytest.approx(b["tokens_B"], rel=1e-12)
    assert [(f["start_B"], f["parameters"]["model"]) for f in mine["fits"]] == [(f["start_B"], f["parameters"]["model"]) for f in theirs["fits"]]
    for a, b in zip(mine["fits"], theirs["fits"]):
        assert a["parameters"]["rmse"] == pytest.approx(b["parameters"]["rmse"], rel=1e-3, abs=1e-9)
        for budget, value in a["endpoint_losses"].items():
            assert value == pytest.approx(b["endpoint_losses"][budget], rel=2e-3)
    assert mine["observed_validation"] == theirs["observed_validation"] and mine["latest_validation"] == theirs["latest_validation"]
    assert len(mine["holdouts"]) == len(theirs["holdouts"])
    for a, b in zip(mine["holdouts"], theirs["holdouts"]):
        assert (a["train_end_B"], a["test_end_B"]) == (b["train_end_B"], b["test_end_B"])
        assert a["actual_mean_loss"] == pytest.approx(b["actual_mean_loss"], rel=1e-12)
        assert a["predicted_mean_loss"] == pytest.approx(b["predicted_mean_loss"], rel=1e-3)


# ------------------------------------------------------------------------------------------- checkpoint snapshots
def test_frozen_snapshot_of_a_training_state(ref, tmp_path):
    from warpstate_ai_b200.ckpt import writer as W
    shared = torch.arange(6.0)
    state = {"model": OrderedDict(a=shared, b=shared, c=torch.ones(2, 2, requires_grad=True)),
             "optimizer": {"state": {0: {"step": torch.tensor(3.0), "exp_avg": torch.zeros(3)}}, "param_groups": [{"lr": 1e-3, "params": [0]}]},
             "rng_numpy": np.random.get_state(), "rng_python": random.getstate(), "history": [("x", 1), ["y", shared]], "step": 3}
    mine, theirs = W.snapshot_to_cpu(state), ref["ops.checkpoint_writer"].snapshot_to_cpu(state)
    for snapshot in (mine, theirs):
        assert snapshot["model"]["a"] is snapshot["model"]["b"] is snapshot["history"][1][1]         # one tensor stays one tensor
        assert snapshot["model"]["a"] is not shared and isinstance(snapshot["model"], OrderedDict)
        assert not snapshot["model"]["c"].requires_grad and snapshot["step"] == 3
    shared.add_(100)
    state["optimizer"]["state"][0]["exp_avg"].fill_(9)
    state["optimizer"]["param_groups"][0]["lr"] = 5.0
    for snapshot in (mine, theirs):
        assert snapshot["model"]["a"].tolist() == [0, 1, 2, 3, 4, 5] and snapshot["optimizer"]["state"][0]["exp_avg"].sum() == 0
        assert snapshot["optimizer"]["param_groups"][0]["lr"] == 1e-3
    W.atomic_torch_save(tmp_path / "mine.pt", mine)
    ref["ops.checkpoint_writer"].atomic_torch_save(tmp_path / "theirs.pt", theirs)
    a, b = (torch.load(tmp_path / name, weights_only=False) for name in ("mine.pt", "theirs.pt"))
    assert list(a) == list(b) and torch.equal(a["model"]["a"], b["model"]["a"]) and a["history"][0] == b["history"][0]
    assert sorted(p.name for p in tmp_path.iterdir()) == ["mine.pt", "theirs.pt"]                      # no staging file left


# ------------------------------------------------------------------------------------------- GEMM benchmark cases
def test_gemm_benchmark_cases_are_the_reference_ones(capsys):
    """The projection GEMMs the isolated benchmark times: same M, N, K and FLOPs per family and operation."""
    from warpstate_ai_b200.bench import gemm_bench as GB
    if not (REF / "ops" / "benchmark_gemm.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    with reference_import_path():
        theirs = importlib.import_module("ops.benchmark_gemm")
    for rows in (8192, 16384):
        mine = GB.projection_cases(["ffn_up_gate", "in_proj", "ffn_down", "out_proj"], rows, ["fwd", "dx", "dw"])
        other = theirs.projection_cases(["ffn_up_gate", "in_proj", "ffn_down", "out_proj"], rows, ["fwd", "dx", "dw"])
        assert [(c["operation"], c["m"], c["n"], c["k"], c["flops"], c["a_shape"], c["b_shape"]) for c in mine] == \
            [(c["operation"], c["m"], c["n"], c["k"], c["flops"], c["a_shape"], c["b_shape"]) for c in other]
    assert GB.main(["--list-shapes", "--families", "in_proj", "--operations", "dw", "--rows", "8192"]) == 0       # no GPU needed
    listed = json.loads(capsys.readouterr().out)
    assert listed == [{"name": "in_proj.dw", "family": "in_proj", "operation": "dw", "m": 10240, "n": 2048, "k": 8192,
                       "a_shape": [10240, 8192], "b_shape": [8192, 2048], "flops": 2 * 10240 * 2048 * 8192}]
    a = GB.arguments(["--tokens", "4096", "--iters", "5"])                       # the earlier spellings still work
    assert (a.rows, a.repeats, a.trials, a.warmup, a.backends) == (4096, 5, 1, 3, ["ours", "cublas"])
    for bad in (["--rows", "0"], ["--trials", "0"], ["--families", "lm_head"], ["--burnin-seconds", "-1"]):
        with pytest.raises(SystemExit):
            GB.arguments(bad)


def test_gradient_accumulation_benchmark_command_line(capsys):
    from warpstate_ai_b200.bench import grad_accum_bench as GA
    assert GA.main(["--list-shapes", "--families", "ffn_down", "in_proj", "--rows", "8192"]) == 0
    assert json.loads(capsys.readouterr().out) == [
        {"family": "down", "rows": 8192, "n": 2048, "k": 7168, "flops": 2 * 8192 * 7168 * 2048},
        {"family": "in_proj", "rows": 8192, "n": 10240, "k": 2048, "flops": 2 * 8192 * 2048 * 10240}]
    a = GA.arguments(["--tokens", "16384", "--iters", "4", "--accumulation-steps", "4"])
    assert (a.rows, a.repeats, a.accumulation_steps) == (16384, 4, 4) and "cublas_fp32_addmm" not in a.variants
    assert "cublas_fp32_addmm" in GA.arguments(["--rows", "4096"]).variants
    assert GA.arguments(["--variants", "grouped_launch"]).variants == ["grouped_launch"]
    for bad in (["--accumulation-steps", "0"], ["--variants", "triton"], ["--rows", "-1"]):
        with pytest.raises(SystemExit):
            GA.arguments(bad)


def test_run_comparison_statistics(ref):
    """Timing statistics and the table of differences of the run comparator, on the same numbers."""
    from warpstate_ai_b200.bench import compare_runs as CR
    theirs = ref["ops.compare_communication_benchmarks"]
    rng = random.Random(11)
    for count in (1, 4, 5, 9, 10, 37):
        seconds = [rng.uniform(0.7, 0.9) for _ in range(count)]
        assert CR.timing_statistics(seconds, 131072) == theirs.timing_statistics(seconds, 131072)
    left = {"a": 1, "b": [1, 2], "c": {"x": 1}, "only_left": None, "same": "s"}
    right = {"a": 2, "b": [1, 2], "c": {"x": 2}, "only_right": 0, "same": "s"}
    assert CR.differences(left, right) == theirs.differences(left, right)
    assert CR.differences(left, left) == theirs.differences(left, left) == {}
    for bad in (float("nan"), float("inf"), True, "1", None):
        with pytest.raises(ValueError):
            CR.finite(bad, "x")
        with pytest.raises(ValueError):
            theirs.finite_number(bad, "x")
    for value in (0, -1.5):
        assert CR.finite(value, "x") == theirs.finite_number(value, "x")
        with pytest.raises(ValueError):
            CR.finite(value, "x", positive=True)
        with pytest.raises(ValueError):
            theirs.finite_number(value, "x", positive=True)


def test_transfer_manifest_and_confinement(tmp_path, monkeypatch):
    """The chunk manifest of a file (what a resumed transfer is checked against) and the rule that confines both
    endpoints to the workspace, against the reference's transfer tool."""
    from warpstate_ai_b200.orchestration import transfer_agent as TA
    if not (REF / "ops" / "transfer_artifacts.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    with reference_import_path():
        theirs = importlib.import_module("ops.transfer_artifacts")
    rng = random.Random(3)
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(tmp_path))
    for size, chunk in ((0, 1024), (1, 1024), (1024, 1024), (1025, 1024), (5 * 1024 * 1024 + 17, 2 * 1024 * 1024), (4096, 4096 * 4)):
        path = tmp_path / f"blob-{size}-{chunk}"
        path.write_bytes(rng.randbytes(size))
        expected, identity = theirs.source_manifest(path, chunk)
        with path.open("rb") as stream:
            assert TA.chunk_manifest(stream, chunk) == expected
        assert TA.file_identity(path.stat()) == list(identity)
        for offset, count in ((0, None), (0, min(size, 7)), (min(size, 1000), None)):
            import hashlib
            data = path.read_bytes()[offset:None if count is None else offset + count]
            assert TA.sha_range(path, offset, count) == hashlib.sha256(data).hexdigest()
    root = tmp_path / "workspace"
    (root / "inside").mkdir(parents=True)
    (root / "inside/file").write_text("x")
    (tmp_path / "outside").mkdir()
    (root / "link").symlink_to(tmp_path / "outside")
    monkeypatch.setattr(theirs, "ROOT", root)
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(root))
    for candidate in (root / "inside/file", root / "inside/new", root, tmp_path / "outside/x", root / "inside/../../outside/x",
                      root / "link/x", root / "link"):
        verdicts = []
        for rule in (theirs.workspace_path, TA.confined):
            try:
                verdicts.append(str(rule(str(candidate))))
            except ValueError:
                verdicts.append("refused")
        assert verdicts[0] == verdicts[1], candidate


# ------------------------------------------------------------------------------------------- launcher
WORKER = """
import os, signal, subprocess, sys, time
mode = os.environ["MODE"]
if len(sys.argv) > 1:                                   # a worker in a session of its own, as torchrun starts them
    signal.signal(signal.SIGTERM, signal.SIG_IGN)
    while True:
        if mode == "graceful" and os.path.exists(os.environ["STOP_FILE"]):
            open(os.environ["MARK"], "w").write("saved")
            sys.exit(0)
        time.sleep(0.05)
open(os.environ["MARK"] + ".started", "w").write("x")
if mode == "exit3":
    sys.exit(3)
worker = subprocess.Popen([sys.executable, __file__, "worker"], start_new_session=True)
open(os.environ["PIDFILE"], "w").write(str(worker.pid))
if mode == "stubborn":
    signal.signal(signal.SIGTERM, signal.SIG_IGN)
sys.exit(worker.wait())
"""


@pytest.fixture
def launchers(tmp_path, monkeypatch):
    from warpstate_ai_b200.orchestration import launcher as mine
    if not (REF / "ops" / "launch_training.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    with reference_import_path():
        theirs = importlib.import_module("ops.launch_training")
    monkeypatch.setattr(theirs, "WORKSPACE", tmp_path.resolve())
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(tmp_path))
    return mine, theirs


@pytest.mark.parametrize("mode", ["exit3", "already-stopped", "graceful", "terminated", "stubborn"])
def test_both_supervisors_end_a_job_the_same_way(launchers, tmp_path, mode):
    """A job that exits by itself, one that is never started because a stop request is pending, one whose workers save
    and leave when asked, one that has to be terminated, and one that has to be killed, workers included."""
    import os
    import signal
    import sys
    import threading
    import time
    from pathlib import Path
    script = tmp_path / "job.py"
    script.write_text(WORKER)
    outcomes = []
    for index, module in enumerate(launchers):
        place = tmp_path / f"run{index}"
        (place / "control").mkdir(parents=True)
        stop = place / "control/training-stop-request"
        environment = dict(os.environ, MODE=mode, STOP_FILE=str(stop), MARK=str(place / "mark"), PIDFILE=str(place / "pid"))
        if mode == "already-stopped":
            stop.write_text("")

        def trigger(place=place):
            for _ in range(200):
                if (place / "pid").exists():
                    break
                time.sleep(0.05)
            time.sleep(0.3)
            os.kill(os.getpid(), signal.SIGUSR1)

        if mode in ("graceful", "terminated", "stubborn"):
            threading.Thread(target=trigger, daemon=True).start()
        code = module.supervise([sys.executable, str(script)], stop, environment, grace_seconds=0.6, terminate_seconds=0.6)
        time.sleep(0.2)
        worker_alive = False
        if (place / "pid").exists():
            pid = int((place / "pid").read_text())
            status = Path(f"/proc/{pid}/stat")
            worker_alive = status.exists() and status.read_text().rsplit(")", 1)[1].split()[0] != "Z"
        outcomes.append({"code": code, "started": (place / "mark.started").exists(), "saved": (place / "mark").exists(),
                         "stop_file": stop.exists(), "worker_alive": worker_alive})
    assert outcomes[0] == outcomes[1], outcomes
    expected = {"exit3": (3, True, False, False), "already-stopped": (0, False, False, True), "graceful": (0, True, True, True),
                "terminated": (-signal.SIGTERM, True, False, True), "stubborn": (-signal.SIGKILL, True, False, True)}[mode]
    assert tuple(outcomes[0][key] for key in ("code", "started", "saved", "stop_file")) == expected
    assert outcomes[0]["worker_alive"] is False


def test_both_launchers_give_the_job_the_same_environment(launchers, tmp_path, monkeypatch):
    mine, theirs = launchers
    monkeypatch.setenv("PIP_CACHE_DIR", "/somewhere/else")
    work = tmp_path / "job/work"
    a, b = mine.training_environment(work), theirs.training_environment(work)
    assert {k: a.get(k) for k in b} == b and a["PIP_CACHE_DIR"] == str(tmp_path / ".cache/pip")
    assert all(Path(a[name]).is_dir() for name in ("TMPDIR", "HF_HOME", "TORCH_EXTENSIONS_DIR", "TRITON_CACHE_DIR"))
    assert mine.process_info(os.getpid()) == theirs.process_info(os.getpid()) and mine.process_info(2 ** 22 + 5) is None
    for place in (tmp_path / "x/../y", tmp_path, "/etc/passwd", tmp_path / ".." / "escape"):
        verdicts = []
        for rule in (mine.workspace_path, theirs.workspace_path):
            try:
                verdicts.append(str(rule(place)))
            except ValueError:
                verdicts.append("refused")
        assert verdicts[0] == verdicts[1], place


def reference_benchmark_directory(root, world=2, warmup=1, measured=3, seed=0, scale=1.0):
    """A benchmark directory in the reference's layout (``summary.json`` with embedded ranks)."""
    rng = random.Random(seed)
    args = {"global_tokens_per_update": 1024 * world, "seq_len": 128, "micro_batch": 2, "warmup_updates": warmup,
            "measured_updates": measured, "seed": 1337, "optimizer_state": "fresh", "bf16_residuals": False, "profile": False,
            "ddp_bucket_cap_mb": 128}
    identity = {"path": "/workspace/WarpState/ckpt.pt", "size": 10, "inode": 3, "mtime_ns": 5}
    config = {"checkpoint": identity, "checkpoint_step": 10, "checkpoint_tokens": 4096, "data": dict(identity, path="/workspace/WarpState/train.bin"),
              "world_size": world, "grad_accum": 4, "parameters": 12345, "parameter_dtype": "float32", "autocast_dtype": "bfloat16",
              "optimizer": "AdamW(fused=True)", "torch": "2.x", "cuda": "12", "gpu": "GPU", "update_timing_includes_gradient_zeroing": True,
              "args": args, "source_sha256": {"run_40b.py": "0" * 64}}
    losses = [5.0 - 0.1 * i for i in range(warmup + measured)]
    ranks = []
    for rank in range(world):
        updates = []
        for index in range(warmup + measured):
            seconds = scale * rng.uniform(0.9, 1.1)
            updates.append({"event": "update", "update": index + 1, "phase": "warmup" if index < warmup else "measured", "rank": rank,
                            "global_tokens": args["global_tokens_per_update"], "profiled": False, "seconds": seconds,
                            "tokens_per_second": args["global_tokens_per_update"] / seconds, "loss": losses[index] + 0.01 * rank,
                            "grad_norm": 1.0 + 0.1 * index, "peak_allocated_gib": 1.5 + rank, "peak_reserved_gib": 2.0 + rank})
        ranks.append({"configuration": dict(config, rank=rank), "updates": updates, "checkpoint_path_identity_after": identity})
    root.mkdir(parents=True)
    summary = {"configuration": dict(config, rank=0), "updates": ranks[0]["updates"], "ranks": ranks,
               "checkpoint_path_identity_after": identity}
    (root / "summary.json").write_text(json.dumps(summary))
    return summary


def test_a_reference_benchmark_directory_is_read_and_paired_with_ours(ref, tmp_path, monkeypatch):
    """The comparator here reads the reference benchmark's own record layout (the fixture is first shown to the
    reference's comparator, which accepts it), reports the same timing figures for it as the reference's comparator does,
    and pairs it with a run recorded in this framework's layout."""
    from warpstate_ai_b200.bench import compare_runs as CR
    theirs = ref["ops.compare_communication_benchmarks"]
    monkeypatch.setattr(theirs, "WORKSPACE", tmp_path.resolve())
    control = reference_benchmark_directory(tmp_path / "control", seed=1)
    reference_benchmark_directory(tmp_path / "candidate", seed=2, scale=0.8)
    expected = theirs.compare_summaries(theirs.load_run(tmp_path / "control")["summary"], theirs.load_run(tmp_path / "candidate")["summary"])
    mine = CR.compare(CR.load_run(tmp_path / "control"), CR.load_run(tmp_path / "candidate"))
    for key in ("control_timing", "candidate_timing", "throughput_ratio", "maximum_absolute_loss_difference",
                "maximum_relative_grad_norm_difference"):
        assert mine[key] == expected[key], key
    for a, b in zip(mine["paired_updates"], expected["paired_updates"]):
        assert {k: a[k] for k in ("update", "control_seconds", "candidate_seconds", "throughput_ratio")} == \
               {k: b[k] for k in ("update", "control_seconds", "candidate_seconds", "throughput_ratio")}
        for x, y in zip(a["ranks"], b["ranks"]):
            assert {k: x[k] for k in x} == {k: y[k] for k in x}
    assert [row["control"]["peak_allocated_bytes"] for row in mine["rank_peak_memory"]] == [int(1.5 * 2 ** 30), int(2.5 * 2 ** 30)]
    # a run in this framework's layout with the same geometry, checkpoint and data
    args = control["configuration"]["args"]
    ours = tmp_path / "ours"
    ours.mkdir()
    rows_by_rank = CR.load_run(tmp_path / "control")["ranks"]
    native = {"format": "warpstate-training-benchmark-v1", "world_size": 2, "model": {"parameters": 12345, "config": {"d_model": 8}},
              "geometry": {"micro_batch": 2, "seq_len": 128, "global_tokens_per_update": args["global_tokens_per_update"], "grad_accum": 4},
              "precision": {"compute": "bf16", "master": "fp32", "grads": "fp32", "residual_stream": "fp32"}, "grad_sync": "fused",
              "optimizer": "replicated", "checkpoint": {"path": "/workspace/WarpState/ckpt.pt", "bytes": 10, "mtime_ns": 5},
              "data": {"path": "/workspace/WarpState/train.bin", "bytes": 10, "mtime_ns": 5}, "optimizer_state": "fresh",
              "warmup_updates": 1, "measured_updates": 3, "profile": None}
    (ours / "summary.json").write_text(json.dumps(native))
    for rank, rows in rows_by_rank.items():
        faster = [dict(row, seconds=row["seconds"] / 2, slowest_rank_seconds=row["seconds"] / 2, tokens_per_second=row["tokens"] / (row["seconds"] / 2))
                  for row in rows]
        (ours / f"rank-{rank}.jsonl").write_text("\n".join(json.dumps(row) for row in faster) + "\n")
    mixed = CR.compare(CR.load_run(tmp_path / "control"), CR.load_run(ours))
    assert mixed["throughput_ratio"] == pytest.approx(2.0) and mixed["maximum_absolute_loss_difference"] == 0.0
    assert {"grad_sync", "optimizer"} <= set(mixed["recorded_differences"])
    (ours / "summary.json").write_text(json.dumps(dict(native, model={"parameters": 999, "config": {}})))
    with pytest.raises(ValueError, match="parameter count"):
        CR.compare(CR.load_run(tmp_path / "control"), CR.load_run(ours))
    # what the reference's comparator refuses in its own layout is refused here too
    for name, damage in (("profiled", lambda s: s["ranks"][1]["updates"][2].update(profiled=True)),
                         ("gap", lambda s: s["ranks"][0]["updates"][1].update(update=7)),
                         ("throughput", lambda s: s["ranks"][1]["updates"][0].update(tokens_per_second=1.0)),
                         ("short", lambda s: s["ranks"][1]["updates"].pop()),
                         ("nan", lambda s: s["ranks"][0]["updates"][0].update(loss=float("nan"))),
                         ("same-rank", lambda s: s["ranks"][1]["configuration"].update(rank=0))):
        summary = json.loads((tmp_path / "control/summary.json").read_text())
        damage(summary)
        summary["updates"] = summary["ranks"][0]["updates"]
        bad = tmp_path / f"bad-{name}"
        bad.mkdir()
        (bad / "summary.json").write_text(json.dumps(summary))
        for load in (theirs.load_run, CR.load_run):
            with pytest.raises(ValueError):
                load(bad)
