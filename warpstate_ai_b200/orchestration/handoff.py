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

Reference behaviour: ops/posttrain_handoff.py:378-531, ops/dpo_handoff.py:366-488.  Here one `Guardian`
serves both stages.  What a stage demands of its parent checkpoint and of its own completion is a table of
`Rule`s (message, predicate) that `enforce` walks; the journal file, the lock ladder and the child launches are
methods of the guardian, one per phase, and a phase that cannot proceed yet returns `RETRY`.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import signal
import socket
import subprocess
import sys
import tempfile
import time
import xmlrpc.client
from pathlib import Path

import torch

from ..utils.io import LockHeld, atomic_json, digest, process_lock, utc_timestamp
from ..utils.rules import Rule, enforce, finite, fp32_tensors
from . import archive as A
from .launcher import PACKAGE, supervise, training_environment, workspace_path, workspace_root

STOPPED = False
RETRY = object()          # a phase's answer when the world is not ready: sleep one poll interval, start over


def request_stop(signum=None, frame=None) -> None:
    global STOPPED
    STOPPED = True


# --------------------------------------------------------------------------- supervisord status
def process_status(socket_path, program: str) -> dict:
    """``supervisor.getProcessInfo(program)`` as one HTTP/1.0 exchange over supervisord's unix socket."""
    call = xmlrpc.client.dumps((program,), "supervisor.getProcessInfo").encode()
    request = (b"POST /RPC2 HTTP/1.0\r\nHost: localhost\r\nContent-Type: text/xml\r\nContent-Length: "
               + str(len(call)).encode() + b"\r\n\r\n" + call)
    with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as link:
        link.settimeout(10)
        link.connect(str(socket_path))
        link.sendall(request)
        answer = b"".join(iter(lambda: link.recv(1 << 16), b""))
    head, separator, body = answer.partition(b"\r\n\r\n")
    status_line = head.split(b"\r\n", 1)[0].split()
    if not separator or len(status_line) < 2 or status_line[1] != b"200":
        raise ConnectionError(f"supervisord answered {head[:80]!r}")
    (info,), _ = xmlrpc.client.loads(body)
    return info


def clean_exit(info: dict) -> bool:
    return (info.get("statename"), info.get("exitstatus")) == ("EXITED", 0)


def read_json(path):
    with open(path, encoding="utf-8") as handle:
        return json.load(handle)


def load_checkpoint(path):
    return torch.load(path, map_location="cpu", weights_only=False, mmap=True)


def fp32_weights(model: dict, what: str):
    return fp32_tensors(model, "Expected " + what + " FP32 model weights: {name}: {dtype}")


def overlaps(a: Path, b: Path) -> bool:
    return a.is_relative_to(b) or b.is_relative_to(a)


# --------------------------------------------------------------------------- stages
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


class Stage:
    """What differs between the two hand-offs.  Subclasses fill the class attributes and the rule tables."""
    name = plan_format = handoff_format = preflight_format = trainer = checkpoint_format = completion_format = ""
    parent_key = parent_dir_key = ""
    data_files: tuple = ()
    path_keys: tuple = ()
    trainer_extras: tuple = ()
    archive_files: tuple = A.ARCHIVE_FILES      # what the sealed archive of the parent holds
    init_files = None                           # what the new stage copies from it (None: all of it)

    def check_paths(self, plan, paths) -> None:
        raise NotImplementedError

    def parent_rules(self, checkpoint, plan, tokenizer_hash) -> list:
        raise NotImplementedError

    def make_archive(self, paths, plan, revision) -> dict:
        raise NotImplementedError

    def completion_rules(self, checkpoint, completion, report, plan, model_hash) -> list:
        raise NotImplementedError

    # ---- shared behaviour
    def boundary(self, plan) -> dict:
        parent = plan[self.parent_key]
        return {key: parent[key] for key in ("step", "tokens_seen", "tokenizer_sha256")}

    def tokenizer_hash(self, plan) -> str:
        return plan[self.parent_key]["tokenizer_sha256"]

    def parent_checkpoint(self, paths) -> Path:
        return paths[self.parent_dir_key] / "run/latest.pt"

    def validate_parent(self, checkpoint, plan, tokenizer_hash) -> None:
        enforce(self.parent_rules(checkpoint, plan, tokenizer_hash))

    def verify_completion(self, run: Path, plan, model_hash) -> dict:
        completion, report = read_json(run / "completion.json"), read_json(run / "evaluation.json")
        enforce(self.completion_rules(load_checkpoint(run / "latest.pt"), completion, report, plan, model_hash))
        return completion

    def torchrun(self, paths, processes: int) -> list:
        return [sys.executable, "-B", "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
                "--nnodes", "1", "--nproc-per-node", str(processes), "--log-dir", str(paths["work_dir"] / "logs/torchrun")]

    def trainer_command(self, config, paths, weights, stop_path, processes) -> list:
        work = paths["work_dir"]
        flags = {"--config": config, "--work-dir": work / "run", "--data-dir": paths["data_dir"], "--weights": weights,
                 "--tokenizer": paths["tokenizer"]}
        flags.update({flag: work / leaf for flag, leaf in self.trainer_extras})
        flags["--stop-file"] = stop_path
        return [*self.torchrun(paths, processes), str(PACKAGE / self.trainer),
                *(text for flag, value in flags.items() for text in (flag, str(value)))]

    def preflight_command(self, paths, processes) -> list:
        return [sys.executable, "-B", "-m", "warpstate_ai_b200.orchestration.preflight", "--stage", self.name,
                "--work-dir", str(paths["work_dir"] / "preflight"), "--processes", str(processes)]


class SftStage(Stage):
    """base pretraining -> SFT."""
    name, trainer = "sft", "posttrain.py"
    plan_format, handoff_format = "warpstate-posttrain-plan-v1", "warpstate-posttrain-handoff-v1"
    preflight_format = "warpstate-posttrain-preflight-v1"
    checkpoint_format, completion_format = "warpstate-posttrain-v1", "warpstate-posttrain-completion-v1"
    parent_key, parent_dir_key = "base", "base_work_dir"
    data_files = ("sft_train.jsonl", "sft_val.jsonl")
    path_keys = ("base_work_dir", "supervisor_socket", "archive_dir", "work_dir", "data_dir", "tokenizer")

    def check_paths(self, plan, paths):
        work, base = paths["work_dir"], paths["base_work_dir"]
        inside = [base / "run", base / "archives", paths["archive_dir"]]
        enforce([Rule("Posttraining must have a separate run directory outside the base run/archive",
                      lambda: work != base and not any(work.is_relative_to(p) for p in inside)),
                 Rule("Archive and prepared data must stay outside the mutable posttraining run",
                      lambda: not paths["archive_dir"].is_relative_to(work) and not overlaps(paths["data_dir"], work))])

    def parent_rules(self, checkpoint, plan, tokenizer_hash):
        want = plan["base"]
        recorded = lambda: checkpoint["signature"]["data"]["signature"]["tokenizer_sha256"]   # noqa: E731
        return [Rule("Expected a full base training checkpoint", lambda: checkpoint["format"] == "warpstate-server-v1"),
                *(Rule(f"Base {key} must equal {want[key]}, got {checkpoint.get(key)}",
                       lambda key=key: checkpoint[key] == want[key]) for key in ("step", "tokens_seen")),
                Rule("Base checkpoint must contain final validation at the exact stop boundary",
                     lambda: (checkpoint["val_step"], checkpoint["val_tokens"]) == (want["step"], want["tokens_seen"])),
                Rule("Base validation loss is not finite", lambda: finite(checkpoint["val_loss"])),
                Rule("Base tokenizer identity differs from the pinned posttraining plan",
                     lambda: recorded() == tokenizer_hash == want["tokenizer_sha256"]),
                Rule("Base checkpoint contains no model tensors", lambda: len(checkpoint["model"]) > 0),
                *fp32_weights(checkpoint.get("model") or {}, "original")]

    def make_archive(self, paths, plan, revision):
        identity = digest(paths["tokenizer"])
        return A.archive_training_checkpoint(self.parent_checkpoint(paths), paths["tokenizer"], paths["archive_dir"],
                                             plan["base"], BASE_NOTE,
                                             lambda loaded: self.validate_parent(loaded, plan, identity))

    def completion_rules(self, checkpoint, completion, report, plan, model_hash):
        step, origin = checkpoint["step"], plan["base"]["step"]
        return [Rule("SFT completion does not have a durable, fully evaluated final checkpoint",
                     lambda: (checkpoint["format"] == self.checkpoint_format and checkpoint["completed"] is True
                              and 1 <= checkpoint["total_steps"] == step == checkpoint["val_step"]
                              and finite(checkpoint["val_loss"]))),
                Rule("SFT completion belongs to a different plan or initialization",
                     lambda: (checkpoint["signature"]["plan"] == plan and checkpoint["signature"]["base_sha256"] == model_hash
                              and checkpoint["origin"]["step"] == origin)),
                Rule("SFT completion report differs from its checkpoint",
                     lambda: ({k: completion[k] for k in ("format", "stage", "completed", "step", "total_steps", "base_step")}
                              == {"format": self.completion_format, "stage": "sft", "completed": True, "step": step,
                                  "total_steps": checkpoint["total_steps"], "base_step": origin})),
                Rule("SFT evaluation report differs from its completed checkpoint",
                     lambda: ({k: report[k] for k in ("stage", "step", "base_sha256", "val_loss")}
                              == {"stage": "sft", "step": step, "base_sha256": model_hash, "val_loss": checkpoint["val_loss"]}))]


class DpoStage(Stage):
    """SFT -> DPO: the parent is a completed SFT run; its model is exported with ``stage='sft'``."""
    name, trainer = "dpo", "dpo.py"
    plan_format, handoff_format = "warpstate-dpo-plan-v1", "warpstate-dpo-handoff-v1"
    preflight_format = "warpstate-dpo-preflight-v1"
    checkpoint_format, completion_format = "warpstate-dpo-v1", "warpstate-dpo-completion-v1"
    parent_key, parent_dir_key = "sft", "sft_work_dir"
    data_files = ("dpo_train.jsonl", "dpo_val.jsonl")
    path_keys = ("base_work_dir", "sft_work_dir", "supervisor_socket", "archive_dir", "work_dir", "data_dir", "tokenizer")
    trainer_extras = (("--reference-cache-dir", "reference-cache"),)
    archive_files, init_files = A.SFT_ARCHIVE_FILES, A.INIT_FILES

    def check_paths(self, plan, paths):
        work = paths["work_dir"]
        base = paths["base_work_dir"]
        protected = [base / "run", base / "archives", paths["sft_work_dir"], paths["archive_dir"], paths["data_dir"]]
        enforce(Rule(f"DPO outputs overlap protected inputs: {p}", lambda p=p: not overlaps(work, p)) for p in protected)
        named = plan["handoff"].get("sft_plan")
        if named is not None:                # the SFT plan on file must describe the parent that the DPO plan pins
            original = read_json(workspace_path(workspace_root() / named))["base"]
            enforce([Rule("SFT parent identity differs from the DPO plan",
                          lambda: (original["step"], original["tokens_seen"], original["tokenizer_sha256"])
                          == (plan["sft"]["base_step"], plan["sft"]["base_tokens_seen"], plan["sft"]["tokenizer_sha256"]))])

    def parent_rules(self, checkpoint, plan, tokenizer_hash):
        want = plan["sft"]
        return [Rule("SFT must complete the exact planned run and final validation before DPO",
                     lambda: (checkpoint["format"] == "warpstate-posttrain-v1" and checkpoint["completed"] is True
                              and checkpoint["step"] == checkpoint["total_steps"] == checkpoint["val_step"] == want["step"]
                              and checkpoint["tokens_seen"] == want["tokens_seen"])),
                Rule("SFT final validation loss is not finite", lambda: finite(checkpoint["val_loss"])),
                Rule("Completed SFT checkpoint belongs to a different tokenizer",
                     lambda: checkpoint["signature"]["tokenizer_sha256"] == tokenizer_hash == want["tokenizer_sha256"]),
                Rule("Full SFT optimizer or per-rank resume state is missing",
                     lambda: bool(checkpoint["optimizer"]) and bool(checkpoint["rng_by_rank"])),
                *fp32_weights(checkpoint.get("model") or {}, "untouched SFT")]

    def make_archive(self, paths, plan, revision):
        """Sealed archive of the whole finished SFT run: the byte-identical checkpoint (FP32 model, Adam moments, per-rank
        RNG, cursors, signatures), a tensor-exact ``stage='sft'`` model export, the tokenizer, the run's reports, what the
        SFT guardian recorded, provenance and a note.  An existing archive is verified instead."""
        from ..ckpt.formats import export_chat_snapshot
        destination, boundary, source = paths["archive_dir"], self.boundary(plan), self.parent_checkpoint(paths)
        run, sft_work = source.parent, source.parent.parent
        seen_first = source.stat()
        checkpoint = load_checkpoint(source)
        self.validate_parent(checkpoint, plan, digest(paths["tokenizer"]))
        whole = digest(source)

        def intact(folder):
            A.tensors_equal(checkpoint["model"], load_checkpoint(folder / "model.pt")["model"])
            if digest(folder / "checkpoint.pt") != whole:
                raise ValueError("the archived SFT checkpoint is not the run's final checkpoint")

        if destination.exists():
            metadata = A.verify_archive(destination, boundary, files=self.archive_files)
            intact(destination)
            return metadata
        destination.parent.mkdir(parents=True, exist_ok=True)
        staging = Path(tempfile.mkdtemp(prefix=".sft-final-", dir=destination.parent))
        A.copy_regular(source, staging / "checkpoint.pt")
        export_chat_snapshot(checkpoint, staging, paths["tokenizer"], {"path": str(source), "sha256": whole}, stage="sft")
        A.copy_regular(paths["tokenizer"], staging / "tokenizer.model")
        for name in ("settings.json", "evaluation.json", "completion.json", "metrics.jsonl"):
            A.copy_regular(run / name, staging / name)
        for name, leaf in (("sft-execution.json", "control/execution.json"), ("sft-handoff.json", "control/handoff.json")):
            if (sft_work / leaf).is_file():
                A.copy_regular(sft_work / leaf, staging / name)
            else:                                   # an SFT run that no guardian started: same layout, and it says so
                A.write_new(staging / name, json.dumps({"recorded": False, "reason": "the SFT run was not started by a "
                                                        "hand-off guardian; nothing was recorded here"}, indent=2) + "\n")
        model_hash = digest(staging / "model.pt")
        A.write_new(staging / "PROVENANCE.json", json.dumps({
            "format": "warpstate-sft-archive-v1", "repository_revision": revision, "source_checkpoint_sha256": whole,
            "model_sha256": model_hash, "sft_step": checkpoint["step"], "sft_input_tokens": checkpoint["tokens_seen"],
            "sft_assistant_tokens": checkpoint.get("assistant_tokens_seen"), "base": checkpoint.get("origin"),
            "data_sha256": checkpoint["signature"].get("data_sha256"), "tokenizer_sha256": boundary["tokenizer_sha256"],
            "sft_signature": checkpoint["signature"]}, indent=2, default=str) + "\n")
        A.write_new(staging / "ARCHIVE.md", "\n".join([
            f"# KEEP: completed SFT at step {checkpoint['step']}", "", f"Created {utc_timestamp()}.",
            f"`checkpoint.pt` is the untouched final SFT checkpoint (SHA256 `{whole}`, from {source}): FP32 model, Adam "
            "moments, per-rank RNG, cursors and signatures.",
            "`model.pt` is a tensor-exact FP32 model-only export; DPO starts from an independent copy of it with a fresh "
            "optimizer, and its fixed reference stays at this model.",
            f"Final full-holdout loss: {checkpoint['val_loss']}.", f"Repository revision: `{revision}`.",
            "Independent physical files, all read-only. Verify with `sha256sum -c SHA256SUMS`.", ""]))
        now = source.stat()
        if (seen_first.st_ino, seen_first.st_size, seen_first.st_mtime_ns) != (now.st_ino, now.st_size, now.st_mtime_ns):
            raise RuntimeError("the SFT checkpoint changed while it was being archived")
        A.seal(staging, self.archive_files)
        metadata = A.verify_archive(staging, boundary, files=self.archive_files)
        intact(staging)
        A.publish_directory(staging, destination)
        return metadata

    def completion_rules(self, checkpoint, completion, report, plan, model_hash):
        step = checkpoint["step"]
        return [Rule("DPO completion does not have a durable, fully evaluated final checkpoint",
                     lambda: (checkpoint["format"] == self.checkpoint_format and checkpoint["completed"] is True
                              and checkpoint["total_steps"] == step == checkpoint["val_step"]
                              and finite(checkpoint["val_loss"]))),
                Rule("DPO completion belongs to a different plan or initialization",
                     lambda: checkpoint["signature"]["plan"] == plan and checkpoint["signature"]["base_sha256"] == model_hash),
                Rule("DPO completion/evaluation reports differ from the checkpoint",
                     lambda: (completion["format"] == self.completion_format and completion["completed"] is True
                              and completion["step"] == step == report["step"]
                              and report["val_loss"] == checkpoint["val_loss"]))]


STAGES = {"sft": SftStage(), "dpo": DpoStage()}


# --------------------------------------------------------------------------- plan / data / identity
def load_plan(path, stage):
    plan = read_json(path)
    enforce([Rule(f"This handoff supports {stage.name} followed by an evaluation pause only",
                  lambda: (plan["format"], plan["stage"], plan["after_completion"])
                  == (stage.plan_format, stage.name, "pause_for_evaluation"))])
    options, root = plan["handoff"], workspace_root()
    paths = {key: workspace_path(root / options[key]) for key in stage.path_keys}
    stage.check_paths(plan, paths)
    enforce([Rule("Invalid process count or polling interval",
                  lambda: 1 <= options["processes"] <= 8 and 0.01 <= options["poll_seconds"] <= 60)])
    return plan, paths


def data_readiness(folder: Path, plan, stage, *, verify: bool = False):
    """(ready, why).  Not ready is an answer; prepared data that contradicts the plan is an error."""
    listing = folder / "manifest.json"
    if not listing.is_file():
        return False, "waiting for data manifest"
    manifest = read_json(listing)
    if (manifest.get("format"), bool(manifest.get("complete"))) != ("warpstate-posttrain-data-v1", True):
        return False, "data preparation is incomplete"
    pinned = plan["handoff"].get("data_manifest_sha256")
    outputs = manifest.get("outputs", {})
    enforce([Rule("Prepared data uses a different tokenizer", lambda: manifest["tokenizer_sha256"] == stage.tokenizer_hash(plan)),
             Rule("Prepared data context length differs from the plan",
                  lambda: manifest["max_length"] == plan["training"]["sequence_length"]),
             Rule("Prepared data differs from the authorized plan", lambda: pinned is None or digest(listing) == pinned),
             *(Rule(f"Prepared split is empty or missing: {name}",
                    lambda name=name: outputs[name]["rows"] >= 1 and (folder / name).is_file()) for name in stage.data_files)])
    if not verify:
        return True, "data manifest complete"
    enforce(Rule(f"Prepared file checksum mismatch: {name}", lambda name=name: digest(folder / name) == outputs[name]["sha256"])
            for name in stage.data_files)
    return True, "data hashes verified"


def source_identity(config: Path) -> dict:
    """Hashes of the plan and of every source file that defines what the child stage runs."""
    package = PACKAGE / "warpstate_ai_b200"
    entry_points = [PACKAGE / name for name in ("posttrain.py", "dpo.py", "run_40b.py", "chat.py")]
    folders = [sorted((package / sub).glob("*.py")) for sub in ("train", "data", "orchestration")]
    single = [package / leaf for leaf in ("models/warpstate.py", "config.py", "ckpt/writer.py", "ckpt/formats.py")]
    return {str(p): digest(p) for p in (config, *entry_points, *(f for group in folders for f in group), *single) if p.is_file()}


def git_revision() -> str:
    done = subprocess.run(["git", "rev-parse", "HEAD"], cwd=PACKAGE, text=True, capture_output=True, check=False)
    return done.stdout.strip() if done.returncode == 0 and done.stdout.strip() else "unknown"


def verify_preflight(path: Path, stage, processes: int) -> dict:
    report = read_json(path)
    wanted = {"format": stage.preflight_format, "accepted": True, "processes": processes, "bf16_compute": True,
              "fp32_parameters_and_adam": True}
    enforce([Rule("GPU preflight report is missing, failed, or belongs to different sources",
                  lambda: {key: report[key] for key in wanted} == wanted)])
    return report


# --------------------------------------------------------------------------- the guardian
class Journal:
    """``control/handoff.json``: who armed the hand-off against which sources, and the phase it is in."""

    def __init__(self, path: Path, stage, identity: dict, boundary: dict, paths: dict):
        self.path = path
        if path.exists():
            self.state = read_json(path)
            if self.state["source_sha256"] != identity:
                raise ValueError("Armed handoff source/config changed; inspect and explicitly re-arm")
        else:
            self.state = {"format": stage.handoff_format, "armed_at": utc_timestamp(), "source_sha256": identity,
                          "git_revision": git_revision(), "target": boundary, "archive_dir": str(paths["archive_dir"]),
                          "work_dir": str(paths["work_dir"])}

    @property
    def complete(self) -> bool:
        return self.state.get("phase") == "complete"

    def note(self, phase: str, message: str, **extra) -> None:
        fresh = (self.state.get("phase"), self.state.get("message")) != (phase, message)
        self.state.update(extra, phase=phase, message=message, updated_at=utc_timestamp())
        atomic_json(self.path, self.state)
        if fresh:
            print(f"[{utc_timestamp()}] {phase}: {message}", flush=True)


class Guardian:
    def __init__(self, config: Path, stage, status_fn, supervise_fn):
        self.config, self.stage, self.supervise_fn = Path(config), stage, supervise_fn
        self.plan, self.paths = load_plan(self.config, stage)
        self.options = self.plan["handoff"]
        self.boundary = stage.boundary(self.plan)
        self.work, self.base_work = self.paths["work_dir"], self.paths["base_work_dir"]
        self.state_path = self.work / "control/handoff.json"
        self.stop_path = self.work / "control/training-stop-request"
        program = self.options["parent_program"] if "parent_program" in self.options else self.options["base_program"]
        self.parent_status = lambda: status_fn(self.paths["supervisor_socket"], program)

    # ---- read-only report
    def describe(self) -> dict:
        ready, reason = data_readiness(self.paths["data_dir"], self.plan, self.stage)
        return {"parent_process": self.parent_status(), "target": self.boundary, "data_ready": ready, "data_status": reason,
                "state_path": str(self.state_path),
                "handoff": read_json(self.state_path) if self.state_path.exists() else None}

    # ---- helpers
    def nap(self):
        time.sleep(self.options["poll_seconds"])

    def unchanged(self, when: str) -> None:
        if source_identity(self.config) != self.identity:
            raise ValueError(f"Armed source/config changed before {when}")

    # ---- phases (each returns RETRY when it has to wait)
    def parent_finished(self):
        info = self.parent_status()
        if clean_exit(info):
            return True
        ready, reason = data_readiness(self.paths["data_dir"], self.plan, self.stage)
        self.journal.note("waiting_for_parent", f"Parent {info.get('statename')}; {reason}", data_ready=ready)
        return RETRY

    def seal_and_stage(self):
        """Under the exclusive pipeline lock: validate, archive, copy, wait for data, write execution.json.
        -> (weights path, archive hash), RETRY, or None when a stop arrived while waiting for data."""
        if not clean_exit(self.parent_status()):
            return RETRY
        reached = load_checkpoint(self.stage.parent_checkpoint(self.paths))
        if reached.get("step", -1) < self.boundary["step"]:
            self.journal.note("waiting_for_parent", f"Parent exited early at step {reached.get('step')}")
            return RETRY
        self.stage.validate_parent(reached, self.plan, digest(self.paths["tokenizer"]))
        del reached
        self.unchanged("handoff")
        self.journal.note("archiving", "Sealing the parent's original FP32 weights at the exact final step")
        model_hash = self.stage.make_archive(self.paths, self.plan, self.journal.state["git_revision"])["snapshot_sha256"]
        self.journal.note("copying_initialization", "Creating/verifying the independent initialization",
                          archive_sha256=model_hash)
        weights = A.independent_copy(self.paths["archive_dir"], self.work / "initialization", self.boundary, model_hash,
                                     files=self.stage.archive_files, only=self.stage.init_files)
        while True:
            if STOPPED:
                return None
            ready, reason = data_readiness(self.paths["data_dir"], self.plan, self.stage)
            if ready:
                break
            self.journal.note("waiting_for_data", reason)
            self.nap()
        data_readiness(self.paths["data_dir"], self.plan, self.stage, verify=True)
        self.unchanged("launch")
        self.stop_path.unlink(missing_ok=True)        # no surviving worker can still need it
        atomic_json(self.work / "control/execution.json", {
            "plan": self.plan, "source_sha256": self.identity, "git_revision": self.journal.state["git_revision"],
            "archive_sha256": model_hash, "data_manifest_sha256": digest(self.paths["data_dir"] / "manifest.json")})
        return weights, model_hash

    def run_children(self, weights: Path, model_hash: str, descriptors: tuple) -> None:
        """Preflight, then the trainer; both inherit the guardian's lock descriptors so that its death cannot lead to
        a duplicate launch."""
        environment, processes = training_environment(self.work), self.options["processes"]
        if self.options.get("preflight", True):
            self.journal.note("gpu_preflight", "Checking BF16 training, masked tails and checkpoint resume")
            code = self.supervise_fn(self.stage.preflight_command(self.paths, processes), self.stop_path, environment,
                                     pass_fds=descriptors)
            if code:
                raise RuntimeError(f"GPU preflight exited with status {code}; training was not started")
            if STOPPED or self.stop_path.exists():
                self.journal.note("paused", "Handoff stopped during GPU preflight; training was not started")
                return
            self.journal.state["preflight"] = verify_preflight(self.work / "preflight/report.json", self.stage, processes)
        command = self.stage.trainer_command(self.config, self.paths, weights, self.stop_path, processes)
        name = self.stage.name
        self.journal.note(name, f"Starting/resuming {name}; fresh optimizer on first start", command=command)
        code = self.supervise_fn(command, self.stop_path, environment, pass_fds=descriptors)
        if code:
            raise RuntimeError(f"{name} child exited with status {code}; checkpoints preserved")
        if not (self.work / "run/completion.json").is_file():
            self.journal.note("paused", f"{name} stopped before completion; its resume checkpoint is retained")
            return
        completion = self.stage.verify_completion(self.work / "run", self.plan, model_hash)
        A.verify_archive(self.paths["archive_dir"], self.boundary, model_hash, files=self.stage.archive_files)
        if digest(weights) != model_hash:
            raise ValueError("Initialization changed during training")
        self.journal.note("complete", f"{name} finished; paused for evaluation.", completion=completion)

    def attempt(self, handoff_file):
        """One pass down the lock ladder.  True when the hand-off has run its course (completed or paused)."""
        if self.parent_finished() is RETRY:
            return RETRY
        with contextlib.ExitStack() as held:
            # outer -> inner order of the base launcher; surviving child ranks hold the pipeline lock shared, so a
            # retry while they live fails closed
            try:
                launcher_file = held.enter_context(process_lock(self.base_work / "control/training-launcher.lock"))
            except LockHeld:
                self.journal.note("waiting_for_locks", "Base launcher is still occupied")
                return RETRY
            with process_lock(self.base_work / "pipeline.lock"):
                staged = self.seal_and_stage()
            # the exclusive pipeline lock is released; the launcher and hand-off locks stay held
            if staged is RETRY:
                return RETRY
            if staged is None or STOPPED:
                return None
            self.run_children(*staged, (handoff_file.fileno(), launcher_file.fileno()))
            return True

    def run(self) -> int:
        self.state_path.parent.mkdir(parents=True, exist_ok=True)
        with process_lock(self.work / "control/handoff.lock") as handoff_file:
            self.identity = source_identity(self.config)
            self.journal = Journal(self.state_path, self.stage, self.identity, self.boundary, self.paths)
            if self.journal.complete:
                print(f"{self.stage.name} already completed; remaining paused for evaluation.", flush=True)
                return 0
            for number in (signal.SIGINT, signal.SIGTERM, signal.SIGUSR1):
                with contextlib.suppress(ValueError):      # not the main thread (tests)
                    signal.signal(number, request_stop)
            try:
                while not STOPPED:
                    outcome = self.attempt(handoff_file)
                    if outcome is True:
                        return 0
                    if outcome is RETRY:
                        self.nap()
                self.journal.note("paused", "Handoff paused by request; no further training will start automatically")
                return 0
            except BaseException as error:
                self.journal.note("failed", f"{type(error).__name__}: {error}")
                raise


def run_handoff(config, *, stage_name: str = "sft", check: bool = False, status_fn=process_status,
                supervise_fn=supervise) -> int:
    guardian = Guardian(config, STAGES[stage_name], status_fn, supervise_fn)
    if check:
        print(json.dumps(guardian.describe(), indent=2))
        return 0
    return guardian.run()


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--config", required=True, type=Path, help="the stage's plan file")
    parser.add_argument("--stage", default="sft", choices=sorted(STAGES))
    parser.add_argument("--check", action="store_true", help="print the read-only status; do not arm or launch")
    options = parser.parse_args(argv)
    return run_handoff(workspace_path(options.config), stage_name=options.stage, check=options.check)


if __name__ == "__main__":
    sys.exit(main())
