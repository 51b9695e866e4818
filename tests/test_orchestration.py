"""Launcher escalation, sealed archives, the handoff state machine with a fake supervisor and a
fake launcher, and the preflight gate on CPU (reference test_training_launcher.py:26-86,
test_posttrain_handoff.py, test_archive_dpo.py, test_posttrain_worker_lock.py)."""
import json
import os
import signal
import subprocess
import sys
import textwrap
import threading
import time
from pathlib import Path

import pytest
import torch

from warpstate_ai_b200.data import prepare as P
from warpstate_ai_b200.data.prepare_posttrain import prepare as prepare_posttrain
from warpstate_ai_b200.orchestration import archive as A
from warpstate_ai_b200.orchestration import handoff as H
from warpstate_ai_b200.orchestration import launcher as L
from warpstate_ai_b200.train import pretrain as T
from warpstate_ai_b200.utils.io import LockHeld, digest, process_lock

ROOT = Path(__file__).resolve().parents[1]
TOK = ROOT / "tokenizer.model"


@pytest.fixture()
def ws(tmp_path, monkeypatch):
    root = tmp_path / "ws"
    root.mkdir()
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(root))
    return root


def worker_script(tmp_path: Path, graceful: bool) -> Path:
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(f"""
        import os, sys, time, subprocess
        # a grandchild in its own session, like a torchrun worker
        if len(sys.argv) > 1 and sys.argv[1] == "leaf":
            stop = os.environ["STOP_FILE"]
            while True:
                if {graceful!r} and os.path.exists(stop):
                    open(os.environ["MARK"], "w").write("saved")
                    sys.exit(0)
                time.sleep(0.05)
        child = subprocess.Popen([sys.executable, __file__, "leaf"], start_new_session=True)
        open(os.environ["PIDFILE"], "w").write(str(child.pid))
        import signal
        signal.signal(signal.SIGTERM, lambda *a: None)
        sys.exit(child.wait())
    """))
    return path


@pytest.mark.parametrize("graceful", [True, False])
def test_launcher_graceful_and_forced_stop(ws, tmp_path, graceful):
    stop = ws / "control/stop"
    stop.parent.mkdir()
    env = dict(os.environ, STOP_FILE=str(stop), MARK=str(tmp_path / "mark"), PIDFILE=str(tmp_path / "pid"))
    script = worker_script(tmp_path, graceful)
    result = {}

    def run():
        result["code"] = L.supervise([sys.executable, str(script)], stop, env, grace_seconds=1.0,
                                     terminate_seconds=0.5, poll_seconds=0.05, scan_seconds=0.1)

    # signal handlers must be installed from the main thread: run supervise here, trigger from a thread
    def trigger():
        for _ in range(100):
            if (tmp_path / "pid").exists():
                break
            time.sleep(0.05)
        time.sleep(0.3)
        os.kill(os.getpid(), signal.SIGUSR1)

    threading.Thread(target=trigger, daemon=True).start()
    run()
    leaf = int((tmp_path / "pid").read_text())
    time.sleep(0.2)
    assert L.process_info(leaf) is None or not Path(f"/proc/{leaf}/cmdline").read_text().count("leaf") \
        or Path(f"/proc/{leaf}/stat").read_text().split()[2] == "Z"
    if graceful:
        assert result["code"] == 0 and (tmp_path / "mark").read_text() == "saved"
    else:
        assert result["code"] != 0 and not (tmp_path / "mark").exists()
    assert stop.exists()


def test_lock_is_inherited_by_children(tmp_path):
    lock = tmp_path / "pipeline.lock"
    with process_lock(lock) as handle:
        child = subprocess.Popen([sys.executable, "-c", "import time; time.sleep(30)"], pass_fds=(handle.fileno(),))
    try:
        with pytest.raises(LockHeld):  # the parent released its context, the orphan still holds the lock
            with process_lock(lock):
                pass
        with pytest.raises(LockHeld):
            with process_lock(lock, shared=True):
                pass
    finally:
        child.kill()
        child.wait()
    with process_lock(lock):
        pass


def train_base(ws: Path) -> tuple[Path, dict]:
    cfg = ws / "cfg.json"
    cfg.write_text(json.dumps(dict(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24,
                                   chunk_size=8, gradient_checkpointing=False, parallel_memory=True)))
    tok = ws / "tokenizer.model"
    tok.write_bytes(TOK.read_bytes())
    base = ws / "base"
    P.write_synthetic_corpus(base, tok, 73, 64, 32768, seed=2)
    T.STOP = False
    T.main(["--from-scratch", "--work-dir", str(base), "--config", str(cfg), "--tokenizer", str(tok), "--stage", "train",
            "--device", "cpu", "--test-small-gpu", "--train-tokens", "73", "--val-tokens", "64", "--seq-len", "8",
            "--micro-batch", "2", "--grad-accum", "2", "--warmup-steps", "1", "--eval-batches", "1",
            "--no-activation-checkpointing", "--dataset", "synthetic/uniform", "--dataset-config", "none",
            "--revision", "0"])
    ckpt = torch.load(base / "run/latest.pt", weights_only=False)
    return tok, {"step": ckpt["step"], "tokens_seen": ckpt["tokens_seen"], "tokenizer_sha256": digest(tok)}


def test_archive_seal_verify_and_tamper(ws):
    tok, boundary = train_base(ws)
    stage = H.SftStage()
    plan = {"base": boundary}
    paths = {"base_work_dir": ws / "base", "tokenizer": tok, "archive_dir": ws / "base/archives/final"}
    meta = stage.make_archive(paths, plan, "rev")
    assert meta["step"] == boundary["step"]
    again = stage.make_archive(paths, plan, "rev")  # idempotent: verifies instead of rewriting
    assert again["snapshot_sha256"] == meta["snapshot_sha256"]
    copy = A.independent_copy(paths["archive_dir"], ws / "sft/initialization", boundary, meta["snapshot_sha256"])
    assert copy.stat().st_ino != (paths["archive_dir"] / "model.pt").stat().st_ino
    with pytest.raises(ValueError):
        A.verify_archive(paths["archive_dir"], dict(boundary, step=boundary["step"] + 1))
    victim = ws / "sft/initialization/ARCHIVE.md"
    os.chmod(victim.parent, 0o755)
    os.chmod(victim, 0o644)
    victim.write_text("tampered")
    os.chmod(victim, 0o444)
    with pytest.raises(ValueError, match="checksum mismatch"):
        A.verify_archive(ws / "sft/initialization", boundary)
    with pytest.raises(OSError):
        A.publish_directory(ws / "cfg.json", paths["archive_dir"])  # never replaces an existing archive


def test_handoff_state_machine_with_fakes(ws, monkeypatch):
    tok, boundary = train_base(ws)
    data = ws / "data"
    rows = [{"messages": [{"role": "user", "content": f"q{i}"}, {"role": "assistant", "content": f"a{i}"}]} for i in range(8)]
    preference = [{"prompt": [{"role": "user", "content": f"Say the number {i}."}],
                   "chosen": [{"role": "assistant", "content": f"{i}"}],
                   "rejected": [{"role": "assistant", "content": f"I will not say {i + 7} today."}]} for i in range(8)]
    prepare_posttrain(data, tok, 64, sft_rows=rows, dpo_rows=preference, val_modulus=3)
    plan = {"format": "warpstate-posttrain-plan-v1", "stage": "sft", "after_completion": "pause_for_evaluation",
            "base": boundary, "training": {"sequence_length": 64, "micro_batch": 2, "grad_accum": 1, "lr": 1e-3,
                                           "eval_every": 1, "save_every": 1, "eval_batches": 1, "workers": 1,
                                           "max_steps": 2},
            "handoff": {"base_work_dir": "base", "supervisor_socket": "supervisor.sock", "archive_dir": "base/archives/final",
                        "work_dir": "sft", "data_dir": "data", "tokenizer": "tokenizer.model", "base_program": "train",
                        "processes": 1, "poll_seconds": 0.01, "preflight": False}}
    config = ws / "plan.json"
    config.write_text(json.dumps(plan))
    monkeypatch.setattr(H, "STOPPED", False)
    states = iter([{"statename": "RUNNING"}, {"statename": "RUNNING"}] + [{"statename": "EXITED", "exitstatus": 0}] * 10)
    calls = []

    def fake_supervise(command, stop_path, environment, pass_fds=()):
        calls.append(command)
        assert len(pass_fds) == 2
        # run the real trainer in-process equivalent: a subprocess on CPU, single rank
        script = next(i for i, word in enumerate(command) if word in (str(L.PACKAGE / "posttrain.py"), str(L.PACKAGE / "dpo.py")))
        env = dict(environment, PYTHONPATH=str(ROOT), WARPSTATE_WORKSPACE=str(ws))
        return subprocess.run([sys.executable, *command[script:], "--device", "cpu"], env=env).returncode

    assert H.run_handoff(config, stage_name="sft", status_fn=lambda s, p: next(states), supervise_fn=fake_supervise) == 0
    state = json.loads((ws / "sft/control/handoff.json").read_text())
    assert state["phase"] == "complete" and state["completion"]["completed"] is True
    assert len(calls) == 1 and (ws / "sft/run/latest.pt").exists() and (ws / "sft/initialization/model.pt").exists()
    A.verify_archive(ws / "base/archives/final", boundary, state["archive_sha256"])
    # a second run is a no-op; a changed plan is refused
    assert H.run_handoff(config, stage_name="sft", status_fn=lambda s, p: {"statename": "EXITED", "exitstatus": 0},
                         supervise_fn=fake_supervise) == 0
    assert len(calls) == 1
    plan["training"]["lr"] = 2e-3
    config.write_text(json.dumps(plan))
    with pytest.raises(ValueError, match="re-arm"):
        H.run_handoff(config, stage_name="sft", status_fn=lambda s, p: {"statename": "EXITED", "exitstatus": 0},
                      supervise_fn=fake_supervise)
    # ---- the second guardian: the completed SFT run is sealed, copied and handed to the DPO trainer
    finished = torch.load(ws / "sft/run/latest.pt", weights_only=False)
    dpo_plan = {"format": "warpstate-dpo-plan-v1", "stage": "dpo", "after_completion": "pause_for_evaluation",
                "sft": {"step": finished["step"], "tokens_seen": finished["tokens_seen"], "tokenizer_sha256": digest(tok)},
                "training": {"sequence_length": 64, "micro_batch": 2, "grad_accum": 1, "lr": 1e-3, "eval_every": 1,
                             "save_every": 1, "eval_batches": 1, "workers": 1, "max_steps": 2, "beta": 0.5,
                             "head_chunk_size": 16},
                "handoff": {"base_work_dir": "base", "sft_work_dir": "sft", "supervisor_socket": "supervisor.sock",
                            "archive_dir": "archives/sft-final", "work_dir": "dpo", "data_dir": "data",
                            "tokenizer": "tokenizer.model", "base_program": "sft-handoff", "processes": 1,
                            "poll_seconds": 0.01, "preflight": False}}
    dpo_config = ws / "dpo-plan.json"
    dpo_config.write_text(json.dumps(dpo_plan))
    assert H.run_handoff(dpo_config, stage_name="dpo", status_fn=lambda s, p: {"statename": "EXITED", "exitstatus": 0},
                         supervise_fn=fake_supervise) == 0
    state = json.loads((ws / "dpo/control/handoff.json").read_text())
    assert state["phase"] == "complete" and state["format"] == "warpstate-dpo-handoff-v1"
    assert "--reference-cache-dir" in calls[-1] and str(ws / "dpo/reference-cache") in calls[-1]
    sealed = torch.load(ws / "archives/sft-final/model.pt", weights_only=False)
    assert sealed["stage"] == "sft" and all(torch.equal(sealed["model"][k], v) for k, v in finished["model"].items())
    assert torch.load(ws / "dpo/run/latest.pt", weights_only=False)["format"] == "warpstate-dpo-v1"
    # the archive keeps the whole finished SFT run; the DPO stage starts from a three-file copy of its own
    archive = ws / "archives/sft-final"
    assert sorted(p.name for p in archive.iterdir()) == sorted((*A.SFT_ARCHIVE_FILES, "SHA256SUMS"))
    assert digest(archive / "checkpoint.pt") == digest(ws / "sft/run/latest.pt")
    assert (archive / "checkpoint.pt").stat().st_ino != (ws / "sft/run/latest.pt").stat().st_ino
    kept = torch.load(archive / "checkpoint.pt", weights_only=False)
    assert kept["optimizer"]["state"] and kept["rng_by_rank"] and kept["format"] == "warpstate-posttrain-v1"
    assert json.loads((archive / "sft-handoff.json").read_text()) == json.loads((ws / "sft/control/handoff.json").read_text())
    assert json.loads((archive / "sft-execution.json").read_text())["plan"]["stage"] == "sft"
    provenance = json.loads((archive / "PROVENANCE.json").read_text())
    assert provenance["format"] == "warpstate-sft-archive-v1" and provenance["source_checkpoint_sha256"] == digest(ws / "sft/run/latest.pt")
    assert provenance["model_sha256"] == digest(archive / "model.pt") and provenance["sft_step"] == finished["step"]
    for name in ("evaluation.json", "completion.json", "settings.json", "metrics.jsonl"):
        assert (archive / name).read_bytes() == (ws / "sft/run" / name).read_bytes()
    assert all(not (p.stat().st_mode & 0o222) for p in archive.iterdir())
    start = ws / "dpo/initialization"
    assert sorted(p.name for p in start.iterdir()) == sorted((*A.INIT_FILES, "SHA256SUMS"))
    assert digest(start / "model.pt") == digest(archive / "model.pt") and (start / "model.pt").stat().st_ino != (archive / "model.pt").stat().st_ino
    A.verify_archive(archive, H.DpoStage().boundary(dpo_plan), files=A.SFT_ARCHIVE_FILES)
    with pytest.raises(ValueError):
        A.verify_archive(archive, H.DpoStage().boundary(dpo_plan))              # not a four-file model archive
    # a parent that stopped one step short is refused by the rule table
    with pytest.raises(ValueError, match="exact planned run"):
        H.DpoStage().validate_parent(dict(finished, step=finished["step"] - 1), dpo_plan, digest(tok))


def test_handoff_rejects_wrong_boundary(ws, monkeypatch):
    tok, boundary = train_base(ws)
    stage = H.SftStage()
    ckpt = torch.load(ws / "base/run/latest.pt", weights_only=False)
    with pytest.raises(ValueError, match="step"):
        stage.validate_parent(ckpt, {"base": dict(boundary, step=boundary["step"] + 1)}, digest(tok))
    ckpt["val_step"] = 0
    with pytest.raises(ValueError, match="final validation"):
        stage.validate_parent(ckpt, {"base": boundary}, digest(tok))


def test_preflight_gate_on_cpu(tmp_path):
    from warpstate_ai_b200.orchestration import preflight
    assert preflight.main(["--stage", "dpo", "--work-dir", str(tmp_path / "pf"), "--processes", "1", "--device", "cpu"]) == 0
    report = json.loads((tmp_path / "pf/report.json").read_text())
    assert report["accepted"] is True and report["frozen_reference_unchanged"] is True
    assert abs(report["initial_validation_loss"] - 0.6931) < 1e-3


def test_launch_scripts_and_supervisor_programs_are_consistent():
    """Every shell launcher parses, points at modules that exist, and every supervisord program
    names an existing launcher with the stop protocol's signal and wait time."""
    import configparser
    launch = ROOT / "launch"
    scripts = sorted(launch.glob("*.sh"))
    assert {"train-b200.sh", "train-8gpu.sh", "benchmark.sh", "posttrain-handoff.sh", "dpo-handoff.sh"} <= {s.name for s in scripts}
    import re
    for script in scripts:
        assert subprocess.run(["bash", "-n", str(script)]).returncode == 0, script
        for module in re.findall(r"-m (warpstate_ai_b200[\w.]+)", script.read_text()):
            assert (ROOT / (module.replace(".", "/") + ".py")).exists(), (script.name, module)
    conf = configparser.RawConfigParser()
    conf.read(launch / "supervisord.conf")
    programs = [s for s in conf.sections() if s.startswith("program:")]
    assert len(programs) >= 4
    for section in programs:
        command = conf.get(section, "command").split()[0]
        assert (launch / Path(command).name).exists(), command
        assert conf.get(section, "autostart") == "false" and conf.get(section, "autorestart") == "false"
        if "benchmark" not in section:
            assert conf.get(section, "stopsignal") == "USR1" and conf.getint(section, "stopwaitsecs") >= 865
    for plan in ("posttrain_plan.json", "dpo_plan.json"):
        data = json.loads((ROOT / "configs" / plan).read_text())
        assert data["after_completion"] == "pause_for_evaluation" and data["handoff"]["processes"] >= 1


def test_ops_entry_points_exist_and_parse_help():
    """The `ops/<name>.py` paths of the original project are thin entry points into the package."""
    names = sorted(p.name for p in (ROOT / "ops").glob("*.py"))
    assert {"launch_training.py", "posttrain_handoff.py", "dpo_handoff.py", "transfer_artifacts.py", "benchmark_training.py",
            "analyze_communication_profile.py", "loss_curve_forecast.py", "archive_dpo.py"} <= set(names)
    for name in ("loss_curve_forecast.py", "transfer_artifacts.py", "compare_communication_benchmarks.py"):
        result = subprocess.run([sys.executable, str(ROOT / "ops" / name), "--help"], capture_output=True, text=True)
        assert result.returncode == 0 and "usage" in result.stdout.lower(), (name, result.stderr[-300:])


def test_process_status_speaks_xmlrpc_over_a_unix_socket(tmp_path):
    """The guardian's supervisord client against a stand-in server on a unix socket: one HTTP/1.0 exchange per
    question, the answer a struct; a non-200 answer is an error, not a status."""
    import socketserver
    import threading
    import xmlrpc.client

    class Handler(socketserver.StreamRequestHandler):
        def handle(self):
            head = b""
            while not head.endswith(b"\r\n\r\n"):
                head += self.rfile.read(1)
            length = int([l.split(b":")[1] for l in head.split(b"\r\n") if l.lower().startswith(b"content-length")][0])
            (program,), method = xmlrpc.client.loads(self.rfile.read(length))
            assert head.startswith(b"POST /RPC2 HTTP/1.0") and method == "supervisor.getProcessInfo"
            if program == "missing":
                self.wfile.write(b"HTTP/1.0 500 Internal Server Error\r\n\r\n")
                return
            body = xmlrpc.client.dumps(({"name": program, "statename": "EXITED", "exitstatus": 0},), methodresponse=True).encode()
            self.wfile.write(b"HTTP/1.0 200 OK\r\nContent-Type: text/xml\r\nContent-Length: %d\r\n\r\n" % len(body) + body)

    path = tmp_path / "supervisor.sock"
    with socketserver.UnixStreamServer(str(path), Handler) as server:
        thread = threading.Thread(target=server.serve_forever, daemon=True)
        thread.start()
        info = H.process_status(path, "train")
        assert info == {"name": "train", "statename": "EXITED", "exitstatus": 0} and H.clean_exit(info)
        with pytest.raises(ConnectionError):
            H.process_status(path, "missing")
        server.shutdown()
    assert not H.clean_exit({"statename": "EXITED", "exitstatus": 1}) and not H.clean_exit({"statename": "RUNNING"})


def test_child_environment_keeps_every_cache_inside_the_workspace(ws):
    work = ws / "work"
    work.mkdir()
    environment = L.training_environment(work)
    inside = {"TMPDIR": ws / "tmp", "XDG_CACHE_HOME": ws / ".cache", "UV_CACHE_DIR": ws / ".cache/uv", "PIP_CACHE_DIR": ws / ".cache/pip",
              "TORCH_HOME": ws / ".cache/torch", "CUDA_CACHE_PATH": ws / ".cache/cuda", "TRITON_CACHE_DIR": ws / ".cache/triton",
              "TORCHINDUCTOR_CACHE_DIR": ws / ".cache/torchinductor", "TORCH_EXTENSIONS_DIR": ws / ".cache/torch-extensions",
              "HF_HOME": work / "hf-cache", "HF_DATASETS_CACHE": work / "hf-cache/datasets", "HF_XET_CACHE": work / "hf-cache/xet"}
    for name, place in inside.items():
        assert environment[name] == str(place) and place.is_dir(), name
    assert environment["PYTHONDONTWRITEBYTECODE"] == "1"
    assert environment["WARPSTATE_STOP_FILE"] == str(work / "control/training-stop-request")
    assert environment["PATH"] == os.environ["PATH"]                        # everything else is inherited
    single = L.build_command(1, Path("run_40b.py"), work, work / "logs", ["--stage", "train"])
    assert single == [sys.executable, "run_40b.py", "--work-dir", str(work), "--stage", "train"]
    many = L.build_command(8, Path("run_40b.py"), work, work / "logs", [])
    assert many[:4] == [sys.executable, "-m", "torch.distributed.run", "--standalone"] and "127.0.0.1" in many
    assert many[many.index("--nproc-per-node") + 1] == "8" and many[-3:] == ["run_40b.py", "--work-dir", str(work)]


def test_preflight_can_prepare_its_fixture_without_launching_anything(ws, capsys, monkeypatch):
    from warpstate_ai_b200.orchestration import preflight
    base = ws / "base"
    base.mkdir()
    monkeypatch.setattr(preflight, "run_trainer", lambda *a, **k: pytest.fail("--prepare-only must not launch training"))
    assert preflight.main(["--stage", "dpo", "--work-dir", str(ws / "dpo/preflight"), "--processes", "2", "--device", "cpu",
                           "--base-work-dir", str(base), "--prepare-only"]) == 0
    said = json.loads(capsys.readouterr().out.splitlines()[-1])
    assert said["prepared"] is True and said["stage"] == "dpo" and said["weights_sha256"] == digest(Path(said["weights"]))
    plan = json.loads(Path(said["plan"]).read_text())
    assert plan["handoff"] == {"base_work_dir": "base"} and plan["format"] == "warpstate-dpo-plan-v1"
    assert (Path(said["data"]) / "manifest.json").is_file() and not (ws / "dpo/preflight/report.json").exists()
    with pytest.raises(SystemExit):
        preflight.main(["--work-dir", str(ws / "x"), "--base-work-dir", str(ws / "absent"), "--prepare-only"])
    with pytest.raises(SystemExit):
        preflight.main(["--work-dir", str(ws / "x"), "--base-work-dir", "/tmp", "--prepare-only"])      # outside the workspace
