"""Guardians that chain the pipeline: base pretraining -> SFT, and SFT -> DPO.

A guardian is an explicitly armed, CUDA-free process (run under supervisord) that

1. polls supervisord (XML-RPC over its unix socket) until the parent job has EXITED with status 0;
2. takes the locks in the fixed order handoff.lock -> training-launcher.lock -> pipeline.lock
   (exclusive), so neither the parent job nor a second guardian can run;
3. validates that the parent's checkpoint sits exactly at the planned boundary (step, tokens,
   final validation at that step, FP32 weights, tokenizer identity);
4. seals an archive of it (`archive.py`), makes an independent physical copy as the child's
   initialisation, waits for and verifies the prepared data;
5. releases pipeline.lock (the child's ranks take it shared), runs the GPU preflight and then
   the child trainer under `launcher.supervise`, passing the lock descriptors down;
6. accepts completion only from the trainer's own ``completion.json`` + final checkpoint +
   evaluation report -- a zero exit status alone may just mean "paused";
7. records every phase in ``control/handoff.json`` and refuses to continue if any source file or
   the plan changed after arming.

Reference behaviour: ops/posttrain_handoff.py:378-531, ops/dpo_handoff.py:366-488.  One state
machine serves both stages here; what differs per stage is a small strategy object.
"""
from __future__ import annotations

import argparse
import contextlib
import http.client
import json
import math
import signal
import socket
import subprocess
import sys
import time
import xmlrpc.client
from pathlib import Path

import torch

from ..utils.io import atomic_json, digest, process_lock, utc_timestamp
from . import archive as A
from .launcher import PACKAGE, supervise, training_environment, workspace_path, workspace_root

STOPPED = False


def request_stop(signum=None, frame=None) -> None:
    global STOPPED
    STOPPED = True


# --------------------------------------------------------------------------- supervisord status
class _UnixConnection(http.client.HTTPConnection):
    def __init__(self, path):
        super().__init__("localhost", timeout=10)
        self._path = str(path)

    def connect(self):
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self.sock.settimeout(self.timeout)
        self.sock.connect(self._path)


class _UnixTransport(xmlrpc.client.Transport):
    def __init__(self, path):
        super().__init__()
        self._path = path

    def make_connection(self, host):
        return _UnixConnection(self._path)


def process_status(socket_path, program: str) -> dict:
    with xmlrpc.client.ServerProxy("http://localhost/RPC2", transport=_UnixTransport(socket_path)) as rpc:
        return rpc.supervisor.getProcessInfo(program)


def clean_exit(info: dict) -> bool:
    return info.get("statename") == "EXITED" and info.get("exitstatus") == 0


def read_json(path):
    return json.loads(Path(path).read_text())


# --------------------------------------------------------------------------- stage strategies
BASE_NOTE = """# KEEP: historical WarpState step {step} weights

Raw model archive created {created} before supervised fine-tuning.
Preserve this directory during cleanup and chat refreshes.

- Completed update: {step:,}; tokens trained: {tokens:,}.
- Validation loss at this step: {val_loss}.
- Original FP32 model tensors; every tensor was compared exactly with the stopped training
  checkpoint before publication.  Model weights only (no optimizer or RNG state); the full
  resume checkpoint stays at `{source}` (SHA256 `{source_sha256}`).
- Independent physical files, all read-only.  Verify with `sha256sum -c SHA256SUMS`.
"""


class SftStage:
    """base pretraining -> SFT."""
    name = "sft"
    plan_format = "warpstate-posttrain-plan-v1"
    handoff_format = "warpstate-posttrain-handoff-v1"
    data_files = ("sft_train.jsonl", "sft_val.jsonl")
    path_keys = ("base_work_dir", "supervisor_socket", "archive_dir", "work_dir", "data_dir", "tokenizer")

    def check_paths(self, plan, paths):
        base, work, archive, data = paths["base_work_dir"], paths["work_dir"], paths["archive_dir"], paths["data_dir"]
        if work == base or work.is_relative_to(base / "run") or work.is_relative_to(base / "archives") \
                or work.is_relative_to(archive):
            raise ValueError("Posttraining must have a separate run directory outside the base run/archive")
        if archive.is_relative_to(work) or data.is_relative_to(work) or work.is_relative_to(data):
            raise ValueError("Archive and prepared data must stay outside the mutable posttraining run")

    def boundary(self, plan):
        return plan["base"]

    def parent_checkpoint(self, paths):
        return paths["base_work_dir"] / "run/latest.pt"

    def validate_parent(self, checkpoint, plan, tokenizer_hash):
        base = plan["base"]
        if checkpoint.get("format") != "warpstate-server-v1":
            raise ValueError("Expected a full base training checkpoint")
        for key in ("step", "tokens_seen"):
            if checkpoint.get(key) != base[key]:
                raise ValueError(f"Base {key} must equal {base[key]}, got {checkpoint.get(key)}")
        if checkpoint.get("val_step") != base["step"] or checkpoint.get("val_tokens") != base["tokens_seen"]:
            raise ValueError("Base checkpoint must contain final validation at the exact stop boundary")
        if not math.isfinite(checkpoint.get("val_loss", float("nan"))):
            raise ValueError("Base validation loss is not finite")
        actual = checkpoint["signature"]["data"]["signature"]["tokenizer_sha256"]
        if actual != tokenizer_hash or actual != base["tokenizer_sha256"]:
            raise ValueError("Base tokenizer identity differs from the pinned posttraining plan")
        if not checkpoint.get("model"):
            raise ValueError("Base checkpoint contains no model tensors")
        for name, tensor in checkpoint["model"].items():
            if tensor.is_floating_point() and tensor.dtype != torch.float32:
                raise ValueError(f"Expected original FP32 model weights: {name}: {tensor.dtype}")

    def make_archive(self, paths, plan, revision):
        base = plan["base"]
        return A.archive_training_checkpoint(
            self.parent_checkpoint(paths), paths["tokenizer"], paths["archive_dir"], base, BASE_NOTE,
            lambda ckpt: self.validate_parent(ckpt, plan, digest(paths["tokenizer"])))

    def trainer_command(self, config, paths, weights, stop_path, processes):
        return [sys.executable, "-B", "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
                "--nnodes", "1", "--nproc-per-node", str(processes), "--log-dir", str(paths["work_dir"] / "logs/torchrun"),
                str(PACKAGE / "posttrain.py"), "--config", str(config), "--work-dir", str(paths["work_dir"] / "run"),
                "--data-dir", str(paths["data_dir"]), "--weights", str(weights), "--tokenizer", str(paths["tokenizer"]),
                "--stop-file", str(stop_path)]

    def preflight_command(self, paths, processes):
        return [sys.executable, "-B", "-m", "warpstate_ai_b200.orchestration.preflight", "--stage", "sft",
                "--work-dir", str(paths["work_dir"] / "preflight"), "--processes", str(processes)]

    def verify_completion(self, run, plan, model_hash):
        completion = read_json(run / "completion.json")
        checkpoint = torch.load(run / "latest.pt", map_location="cpu", weights_only=False, mmap=True)
        report = read_json(run / "evaluation.json")
        step, total = checkpoint["step"], checkpoint["total_steps"]
        if (checkpoint.get("format") != "warpstate-posttrain-v1" or checkpoint.get("completed") is not True
                or step != total or total < 1 or checkpoint.get("val_step") != step
                or not math.isfinite(checkpoint["val_loss"])):
            raise ValueError("SFT completion does not have a durable, fully evaluated final checkpoint")
        if (checkpoint["signature"]["plan"] != plan or checkpoint["signature"]["base_sha256"] != model_hash
                or checkpoint["origin"]["step"] != plan["base"]["step"]):
            raise ValueError("SFT completion belongs to a different plan or initialization")
        if (completion.get("format") != "warpstate-posttrain-completion-v1" or completion.get("stage") != "sft"
                or completion.get("completed") is not True or completion.get("step") != step
                or completion.get("total_steps") != total or completion.get("base_step") != plan["base"]["step"]):
            raise ValueError("SFT completion report differs from its checkpoint")
        if (report.get("stage") != "sft" or report.get("step") != step or report.get("base_sha256") != model_hash
                or report.get("val_loss") != checkpoint["val_loss"]):
            raise ValueError("SFT evaluation report differs from its completed checkpoint")
        return completion

    def tokenizer_hash(self, plan):
        return plan["base"]["tokenizer_sha256"]


class DpoStage(SftStage):
    """SFT -> DPO: the parent is a completed SFT run; its model is exported with ``stage='sft'``."""
    name = "dpo"
    plan_format = "warpstate-dpo-plan-v1"
    handoff_format = "warpstate-dpo-handoff-v1"
    data_files = ("dpo_train.jsonl", "dpo_val.jsonl")
    path_keys = ("base_work_dir", "sft_work_dir", "supervisor_socket", "archive_dir", "work_dir", "data_dir", "tokenizer")

    def check_paths(self, plan, paths):
        work, base, sft, archive, data = (paths[k] for k in ("work_dir", "base_work_dir", "sft_work_dir",
                                                             "archive_dir", "data_dir"))
        for protected in (base / "run", sft, archive, data):
            if work.is_relative_to(protected) or protected.is_relative_to(work):
                raise ValueError(f"DPO outputs overlap protected inputs: {protected}")

    def boundary(self, plan):
        s = plan["sft"]
        return {"step": s["step"], "tokens_seen": s["tokens_seen"], "tokenizer_sha256": s["tokenizer_sha256"]}

    def parent_checkpoint(self, paths):
        return paths["sft_work_dir"] / "run/latest.pt"

    def validate_parent(self, checkpoint, plan, tokenizer_hash):
        expected = plan["sft"]
        if (checkpoint.get("format") != "warpstate-posttrain-v1" or checkpoint.get("completed") is not True
                or checkpoint.get("step") != expected["step"] or checkpoint.get("total_steps") != expected["step"]
                or checkpoint.get("tokens_seen") != expected["tokens_seen"]
                or checkpoint.get("val_step") != expected["step"]):
            raise ValueError("SFT must complete the exact planned run and final validation before DPO")
        if not math.isfinite(checkpoint.get("val_loss", float("nan"))):
            raise ValueError("SFT final validation loss is not finite")
        if checkpoint["signature"]["tokenizer_sha256"] != expected["tokenizer_sha256"] or tokenizer_hash != expected["tokenizer_sha256"]:
            raise ValueError("Completed SFT checkpoint belongs to a different tokenizer")
        if not checkpoint.get("optimizer") or not checkpoint.get("rng_by_rank"):
            raise ValueError("Full SFT optimizer or per-rank resume state is missing")
        for name, tensor in checkpoint["model"].items():
            if tensor.is_floating_point() and tensor.dtype != torch.float32:
                raise ValueError(f"Expected untouched FP32 SFT weights: {name}")

    def make_archive(self, paths, plan, revision):
        """Sealed SFT archive: tensor-exact ``stage='sft'`` model export + tokenizer + the run's
        reports; the complete SFT checkpoint is referenced by hash (it stays in the SFT run)."""
        from ..ckpt.formats import export_chat_snapshot
        import tempfile
        destination = paths["archive_dir"]
        boundary = self.boundary(plan)
        source = self.parent_checkpoint(paths)
        checkpoint = torch.load(source, map_location="cpu", weights_only=False, mmap=True)
        self.validate_parent(checkpoint, plan, digest(paths["tokenizer"]))
        if destination.exists():
            metadata = A.verify_archive(destination, boundary)
            exported = torch.load(destination / "model.pt", map_location="cpu", weights_only=False, mmap=True)
            A.tensors_equal(checkpoint["model"], exported["model"])
            return metadata
        destination.parent.mkdir(parents=True, exist_ok=True)
        staging = Path(tempfile.mkdtemp(prefix=".sft-final-", dir=destination.parent))
        full_hash = digest(source)
        export_chat_snapshot(checkpoint, staging, paths["tokenizer"], {"path": str(source), "sha256": full_hash},
                             stage="sft")
        exported = torch.load(staging / "model.pt", map_location="cpu", weights_only=False, mmap=True)
        A.tensors_equal(checkpoint["model"], exported["model"])
        A.copy_regular(paths["tokenizer"], staging / "tokenizer.model")
        A.write_new(staging / "ARCHIVE.md",
                    f"# KEEP: completed SFT at step {checkpoint['step']}\n\nCreated {utc_timestamp()}.\n"
                    f"Full SFT checkpoint SHA256: `{full_hash}` ({source}).\nFinal full-holdout loss: "
                    f"{checkpoint['val_loss']}.\nRepository revision: `{revision}`.\n")
        A.seal(staging)
        metadata = A.verify_archive(staging, boundary)
        A.publish_directory(staging, destination)
        return metadata

    def trainer_command(self, config, paths, weights, stop_path, processes):
        return [sys.executable, "-B", "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
                "--nnodes", "1", "--nproc-per-node", str(processes), "--log-dir", str(paths["work_dir"] / "logs/torchrun"),
                str(PACKAGE / "dpo.py"), "--config", str(config), "--work-dir", str(paths["work_dir"] / "run"),
                "--data-dir", str(paths["data_dir"]), "--weights", str(weights), "--tokenizer", str(paths["tokenizer"]),
                "--reference-cache-dir", str(paths["work_dir"] / "reference-cache"), "--stop-file", str(stop_path)]

    def preflight_command(self, paths, processes):
        return [sys.executable, "-B", "-m", "warpstate_ai_b200.orchestration.preflight", "--stage", "dpo",
                "--work-dir", str(paths["work_dir"] / "preflight"), "--processes", str(processes)]

    def verify_completion(self, run, plan, model_hash):
        completion = read_json(run / "completion.json")
        checkpoint = torch.load(run / "latest.pt", map_location="cpu", weights_only=False, mmap=True)
        report = read_json(run / "evaluation.json")
        step, total = checkpoint["step"], checkpoint["total_steps"]
        if (checkpoint.get("format") != "warpstate-dpo-v1" or checkpoint.get("completed") is not True or step != total
                or checkpoint.get("val_step") != step or not math.isfinite(checkpoint["val_loss"])):
            raise ValueError("DPO completion does not have a durable, fully evaluated final checkpoint")
        if checkpoint["signature"]["plan"] != plan or checkpoint["signature"]["base_sha256"] != model_hash:
            raise ValueError("DPO completion belongs to a different plan or initialization")
        if (completion.get("format") != "warpstate-dpo-completion-v1" or completion.get("completed") is not True
                or completion.get("step") != step or report.get("step") != step
                or report.get("val_loss") != checkpoint["val_loss"]):
            raise ValueError("DPO completion/evaluation reports differ from the checkpoint")
        return completion

    def tokenizer_hash(self, plan):
        return plan["sft"]["tokenizer_sha256"]


STAGES = {"sft": SftStage(), "dpo": DpoStage()}


# --------------------------------------------------------------------------- plan / data
def load_plan(path, stage):
    plan = read_json(path)
    if (plan.get("format") != stage.plan_format or plan.get("stage") != stage.name
            or plan.get("after_completion") != "pause_for_evaluation"):
        raise ValueError(f"This handoff supports {stage.name} followed by an evaluation pause only")
    options = plan["handoff"]
    root = workspace_root()
    paths = {key: workspace_path(root / options[key]) for key in stage.path_keys}
    stage.check_paths(plan, paths)
    if not 1 <= options["processes"] <= 8 or not 0.01 <= options["poll_seconds"] <= 60:
        raise ValueError("Invalid process count or polling interval")
    return plan, paths


def data_readiness(folder: Path, plan, stage, *, verify: bool = False):
    path = folder / "manifest.json"
    if not path.is_file():
        return False, "waiting for data manifest"
    manifest = read_json(path)
    if manifest.get("format") != "warpstate-posttrain-data-v1" or not manifest.get("complete"):
        return False, "data preparation is incomplete"
    if manifest.get("tokenizer_sha256") != stage.tokenizer_hash(plan):
        raise ValueError("Prepared data uses a different tokenizer")
    if manifest.get("max_length") != plan["training"]["sequence_length"]:
        raise ValueError("Prepared data context length differs from the plan")
    expected_manifest = plan["handoff"].get("data_manifest_sha256")
    if expected_manifest is not None and digest(path) != expected_manifest:
        raise ValueError("Prepared data differs from the authorized plan")
    for name in stage.data_files:
        entry = manifest["outputs"].get(name, {})
        if entry.get("rows", 0) < 1 or not (folder / name).is_file():
            raise ValueError(f"Prepared split is empty or missing: {name}")
        if verify and digest(folder / name) != entry.get("sha256"):
            raise ValueError(f"Prepared file checksum mismatch: {name}")
    return True, "data manifest complete" if not verify else "data hashes verified"


def source_identity(config: Path) -> dict:
    """Hashes of the plan and of every source file that defines what the child stage runs."""
    package = PACKAGE / "warpstate_ai_b200"
    files = [config, PACKAGE / "posttrain.py", PACKAGE / "dpo.py", PACKAGE / "run_40b.py", PACKAGE / "chat.py",
             *sorted((package / "train").glob("*.py")), *sorted((package / "data").glob("*.py")),
             *sorted((package / "orchestration").glob("*.py")), package / "models/warpstate.py", package / "config.py",
             package / "ckpt/writer.py", package / "ckpt/formats.py"]
    return {str(p): digest(p) for p in files if p.is_file()}


def git_revision() -> str:
    try:
        return subprocess.check_output(["git", "rev-parse", "HEAD"], cwd=PACKAGE, text=True,
                                       stderr=subprocess.DEVNULL).strip()
    except (OSError, subprocess.CalledProcessError):
        return "unknown"


def verify_preflight(path: Path, stage, processes: int) -> dict:
    report = read_json(path)
    if (report.get("format") != f"warpstate-{'posttrain' if stage.name == 'sft' else 'dpo'}-preflight-v1"
            or report.get("accepted") is not True or report.get("processes") != processes
            or report.get("bf16_compute") is not True or report.get("fp32_parameters_and_adam") is not True):
        raise ValueError("GPU preflight report is missing, failed, or belongs to different sources")
    return report


# --------------------------------------------------------------------------- the state machine
def run_handoff(config, *, stage_name: str = "sft", check: bool = False, status_fn=process_status,
                supervise_fn=supervise) -> int:
    global STOPPED
    stage = STAGES[stage_name]
    config = Path(config)
    plan, paths = load_plan(config, stage)
    options = plan["handoff"]
    boundary = stage.boundary(plan)
    work, base_work = paths["work_dir"], paths["base_work_dir"]
    state_path = work / "control/handoff.json"

    def status():
        return status_fn(paths["supervisor_socket"], options["parent_program"] if "parent_program" in options
                         else options["base_program"])

    if check:
        ready, reason = data_readiness(paths["data_dir"], plan, stage)
        print(json.dumps(dict(parent_process=status(), target=boundary, data_ready=ready, data_status=reason,
                              state_path=str(state_path),
                              handoff=read_json(state_path) if state_path.exists() else None), indent=2))
        return 0
    state_path.parent.mkdir(parents=True, exist_ok=True)
    with process_lock(work / "control/handoff.lock") as handoff_file:
        identity = source_identity(config)
        if state_path.exists():
            state = read_json(state_path)
            if state["source_sha256"] != identity:
                raise ValueError("Armed handoff source/config changed; inspect and explicitly re-arm")
            if state.get("phase") == "complete":
                print(f"{stage.name} already completed; remaining paused for evaluation.", flush=True)
                return 0
        else:
            state = dict(format=stage.handoff_format, armed_at=utc_timestamp(), source_sha256=identity,
                         git_revision=git_revision(), target=boundary, archive_dir=str(paths["archive_dir"]),
                         work_dir=str(work))

        def record(phase, message, **extra):
            changed = state.get("phase") != phase or state.get("message") != message
            state.update(phase=phase, message=message, updated_at=utc_timestamp(), **extra)
            atomic_json(state_path, state)
            if changed:
                print(f"[{utc_timestamp()}] {phase}: {message}", flush=True)

        stop_path = work / "control/training-stop-request"
        for sig in (signal.SIGINT, signal.SIGTERM, signal.SIGUSR1):
            with contextlib.suppress(ValueError):
                signal.signal(sig, request_stop)
        try:
            while not STOPPED:
                info = status()
                ready, reason = data_readiness(paths["data_dir"], plan, stage)
                if not clean_exit(info):
                    record("waiting_for_parent", f"Parent {info.get('statename')}; {reason}", data_ready=ready)
                    time.sleep(options["poll_seconds"])
                    continue
                # outer -> inner lock order of the base launcher; surviving child ranks hold the
                # pipeline lock shared, so a retry while they live fails closed
                launcher_ctx = process_lock(base_work / "control/training-launcher.lock")
                try:
                    launcher_file = launcher_ctx.__enter__()
                except Exception as error:
                    if type(error).__name__ != "LockHeld":
                        raise
                    record("waiting_for_locks", "Base launcher is still occupied")
                    time.sleep(options["poll_seconds"])
                    continue
                try:
                    with process_lock(base_work / "pipeline.lock"):
                        if not clean_exit(status()):
                            continue
                        parent_path = stage.parent_checkpoint(paths)
                        raw = torch.load(parent_path, map_location="cpu", weights_only=False, mmap=True)
                        if raw.get("step", -1) < boundary["step"]:
                            record("waiting_for_parent", f"Parent exited early at step {raw.get('step')}")
                            del raw
                            time.sleep(options["poll_seconds"])
                            continue
                        stage.validate_parent(raw, plan, digest(paths["tokenizer"]))
                        del raw
                        if source_identity(config) != identity:
                            raise ValueError("Armed source/config changed before handoff")
                        record("archiving", "Sealing the parent's original FP32 weights at the exact final step")
                        metadata = stage.make_archive(paths, plan, state["git_revision"])
                        model_hash = metadata["snapshot_sha256"]
                        record("copying_initialization", "Creating/verifying the independent initialization",
                               archive_sha256=model_hash)
                        weights = A.independent_copy(paths["archive_dir"], work / "initialization", boundary, model_hash)
                        while not STOPPED:
                            ready, reason = data_readiness(paths["data_dir"], plan, stage)
                            if ready:
                                break
                            record("waiting_for_data", reason)
                            time.sleep(options["poll_seconds"])
                        if STOPPED:
                            break
                        data_readiness(paths["data_dir"], plan, stage, verify=True)
                        if source_identity(config) != identity:
                            raise ValueError("Armed source/config changed before launch")
                        stop_path.unlink(missing_ok=True)  # no surviving worker can still need it
                        atomic_json(work / "control/execution.json", dict(
                            plan=plan, source_sha256=identity, git_revision=state["git_revision"],
                            archive_sha256=model_hash,
                            data_manifest_sha256=digest(paths["data_dir"] / "manifest.json")))
                    if STOPPED:
                        break
                    # pipeline.lock (exclusive) is released here; launcher lock + handoff lock stay
                    # held and are passed to the children so that the guardian's death cannot
                    # lead to a duplicate launch
                    environment = training_environment(work)
                    fds = (handoff_file.fileno(), launcher_file.fileno())
                    processes = options["processes"]
                    if options.get("preflight", True):
                        record("gpu_preflight", "Checking BF16 training, masked tails and checkpoint resume")
                        result = supervise_fn(stage.preflight_command(paths, processes), stop_path, environment,
                                              pass_fds=fds)
                        if result:
                            raise RuntimeError(f"GPU preflight exited with status {result}; training was not started")
                        if stop_path.exists() or STOPPED:
                            record("paused", "Handoff stopped during GPU preflight; training was not started")
                            return 0
                        state["preflight"] = verify_preflight(work / "preflight/report.json", stage, processes)
                    command = stage.trainer_command(config, paths, weights, stop_path, processes)
                    record(stage.name, f"Starting/resuming {stage.name}; fresh optimizer on first start", command=command)
                    result = supervise_fn(command, stop_path, environment, pass_fds=fds)
                    if result:
                        raise RuntimeError(f"{stage.name} child exited with status {result}; checkpoints preserved")
                    if (work / "run/completion.json").is_file():
                        completed = stage.verify_completion(work / "run", plan, model_hash)
                        A.verify_archive(paths["archive_dir"], boundary, model_hash)
                        if digest(weights) != model_hash:
                            raise ValueError("Initialization changed during training")
                        record("complete", f"{stage.name} finished; paused for evaluation.", completion=completed)
                    else:
                        record("paused", f"{stage.name} stopped before completion; its resume checkpoint is retained")
                    return 0
                finally:
                    launcher_ctx.__exit__(None, None, None)
            record("paused", "Handoff paused by request; no further training will start automatically")
            return 0
        except BaseException as error:
            record("failed", f"{type(error).__name__}: {error}")
            raise


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--config", type=Path, required=True)
    parser.add_argument("--stage", choices=sorted(STAGES), default="sft")
    parser.add_argument("--check", action="store_true", help="read-only status; do not arm or launch")
    args = parser.parse_args(argv)
    return run_handoff(workspace_path(args.config), stage_name=args.stage, check=args.check)


if __name__ == "__main__":
    sys.exit(main())
