"""The run shared by the post-training stages (SFT, DPO): one template, two sets of hooks.

What a stage run is (the behaviour of the reference's two runners, reference posttrain.py:199-543 and
dpo.py:388-647, which repeat it): every input and output lives inside one workspace root and outputs are
kept apart from inputs; a JSON plan resolves to settings; the run initialises from a sealed model export
or resumes from its own ``latest.pt`` when the stored signature equals the current one; updates draw a
deterministic global batch per step from a resumable sample cursor; rank 0 validates (whole hold-out set
before the first update and at the end, a subset in between) and appends JSON-lines events to
``metrics.jsonl``; checkpoints go through the distributed asynchronous writer; ``completion.json``
appears when the last step is done; a stop request (signal or file) pauses between updates.

`StageRun.execute` is that sequence once.  A stage supplies: how to read its data, what a valid source
export looks like, its signature fields, one update, one validation, and the extra fields of its
records.  The file formats (event keys, checkpoint keys, settings / evaluation / completion files) are
the reference's.
"""
from __future__ import annotations

import contextlib
import json
import math
import os
import random
import time
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from ..ckpt.formats import capture_rng, clean_state_dict, restore_rng
from ..utils.io import atomic_json, digest, process_lock


# ----------------------------------------------------------------------------------- workspace rules
def workspace() -> Path:
    """Root that confines every path of a post-training job (``WARPSTATE_WORKSPACE``)."""
    return Path(os.environ.get("WARPSTATE_WORKSPACE", "/workspace/WarpState")).resolve()


def _within(path: Path, parent: Path) -> bool:
    return path == parent or path.is_relative_to(parent)


def validate_paths(work_dir, data_dir, weights, tokenizer, config):
    """Resolved ``[work, data, weights, tokenizer, plan]`` after checking confinement and separation."""
    root = workspace()
    work, data, source, tok, plan = (Path(p).resolve() for p in (work_dir, data_dir, weights, tokenizer, config))
    for path in (work, data, source, tok, plan):
        if not path.is_relative_to(root):
            raise ValueError(f"{path} is not inside the workspace {root}")
    if work == root:
        raise ValueError("the output directory cannot be the workspace root itself")
    for path in (data, source, tok, plan):
        if _within(path, work):
            raise ValueError(f"input {path} lies in the output directory {work}; keep outputs separate from inputs")
    if work.is_relative_to(data) or work.is_relative_to(source.parent):
        raise ValueError(f"the output directory {work} must not be inside data or source-weight directories")
    for path in (source, tok, plan):
        if not path.is_file():
            raise ValueError(f"required input file is missing: {path}")
    if not data.is_dir():
        raise ValueError(f"prepared data directory is missing: {data}")
    return [work, data, source, tok, plan]


@contextlib.contextmanager
def shared_pipeline_lock(path):
    """Every post-training rank holds the base job's ``pipeline.lock`` shared, so pretraining
    cannot start while any of them -- even an orphan -- is alive."""
    from ..utils.io import LockHeld
    path = Path(path).resolve()
    if not path.is_relative_to(workspace()):
        raise ValueError("the pipeline lock must be a file inside the workspace")
    try:
        with process_lock(path, shared=True):
            yield
    except LockHeld as held:
        raise RuntimeError("pipeline.lock is held exclusively: pretraining or its hand-off is still running") from held


@contextlib.contextmanager
def base_pipeline_lock(plan: dict):
    """The shared lock on the pretraining job named by ``plan['handoff']['base_work_dir']``, if any."""
    relative = plan.get("handoff", {}).get("base_work_dir")
    if relative is None:
        yield
        return
    root = workspace()
    base = (root / relative).resolve()
    if base == root or not base.is_relative_to(root) or not base.is_dir():
        raise ValueError("handoff.base_work_dir must name an existing directory inside the workspace")
    with shared_pipeline_lock(base / "pipeline.lock"):
        yield


# ----------------------------------------------------------------------------------- schedule
def warmup_steps(total_steps: int, ratio: float) -> int:
    return min(math.ceil(ratio * total_steps), max(0, total_steps - 1))


def schedule_position(step: int, total_steps: int, ratio: float):
    """``("warmup", number of warm-up steps)`` or ``("decay", progress in [0, 1])`` for a 0-based step; during
    warm-up the rate is ``peak * (step + 1) / warm-up steps``."""
    warm = warmup_steps(total_steps, ratio)
    if step < warm:
        return "warmup", warm
    return "decay", min(1.0, (step - warm) / max(1, total_steps - warm - 1))


@dataclass
class Progress:
    step: int = 0
    sample_cursor: int = 0
    tokens_seen: int = 0
    scored_tokens: int = 0      # assistant tokens (SFT) / response tokens (DPO)


class StageRun:
    """Template of one post-training run.  Subclasses set the class attributes and implement the hooks."""

    stage = ""                       # "sft" | "dpo"
    checkpoint_format = ""
    completion_format = ""
    scored_key = ""                  # name of `Progress.scored_tokens` in events and checkpoints
    schema = None                    # PlanSchema

    def __init__(self, args, stop_flag):
        self.args, self.stop_flag = args, stop_flag
        self.work, self.data_dir, self.weights, self.tokenizer_path, self.plan_path = validate_paths(
            args.work_dir, args.data_dir, args.weights, args.tokenizer, args.config)
        self.plan, self.s = self.schema.read(self.plan_path)
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.control = None
        self.progress = Progress()
        self.last_validation = None
        self.last_validation_step = None

    # ------------------------------------------------------------------ hooks
    def load_data(self):
        """-> (train records, validation records, manifest, manifest hash)"""
        raise NotImplementedError

    def check_source(self, export: dict) -> None:
        """Raise ValueError unless ``export`` is a valid initialisation for this stage."""
        raise NotImplementedError

    def signature_fields(self) -> dict:
        return {}

    def before_training(self) -> bool:
        """Stage work between joining the process group and building the trainer; False ends the run."""
        return True

    def after_trainer(self) -> None:
        pass

    def run_update(self, indices, lr: float) -> dict:
        """One optimizer update over the global sample ids; returns the fields of the ``train`` event."""
        raise NotImplementedError

    def count_tokens(self, indices) -> tuple[int, int]:
        """(all tokens, scored tokens) of the samples of one update."""
        raise NotImplementedError

    def validate(self, full: bool) -> dict:
        """Fields of a ``validation`` event (must contain ``val_loss``); runs on rank 0 only."""
        raise NotImplementedError

    def learning_rate(self, step: int) -> float:
        raise NotImplementedError

    def event_fields(self) -> dict:
        return {}

    def evaluation_fields(self, values: dict) -> dict:
        return {}

    def checkpoint_fields(self) -> dict:
        return {}

    def completion_fields(self) -> dict:
        return {}

    def after_training(self) -> None:
        pass

    # ------------------------------------------------------------------ fixed parts
    def open_environment(self) -> None:
        import sentencepiece as spm
        local = int(os.environ.get("LOCAL_RANK", "0"))
        self.device = torch.device("cuda", local) if self.args.device == "cuda" else torch.device("cpu")
        if self.device.type == "cuda":
            if not torch.cuda.is_available() or not torch.cuda.is_bf16_supported():
                raise RuntimeError("a CUDA GPU with BF16 support is required")
            torch.cuda.set_device(self.device)
        torch.set_num_threads(self.s["workers"])
        seed = self.s["seed"] + self.rank
        random.seed(seed)
        np.random.seed(seed)
        torch.manual_seed(seed)
        self.tokenizer_hash = digest(self.tokenizer_path)
        self.base_hash = digest(self.weights)
        self.sp = spm.SentencePieceProcessor(model_file=str(self.tokenizer_path))
        self.pad_id = self.sp.pad_id() if self.sp.pad_id() >= 0 else self.sp.eos_id()

    def join_process_group(self) -> None:
        if self.world > 1:
            from ..ckpt.writer import host_control_group
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if self.device.type == "cuda":
                dist.init_process_group("nccl", device_id=self.device)
            else:
                dist.init_process_group("gloo")
            self.control = host_control_group()

    def stop_requested(self) -> bool:
        wanted = bool(self.stop_flag()) or bool(self.args.stop_file and Path(self.args.stop_file).exists())
        if self.world > 1:
            vote = torch.tensor([int(wanted)])
            dist.all_reduce(vote, op=dist.ReduceOp.MAX, group=self.control)
            wanted = bool(vote.item())
        return wanted

    def origin_of(self, export: dict) -> dict:
        origin = {key: value for key, value in export.items() if key != "model"}
        origin["weights_sha256"], origin["weights_path"] = self.base_hash, str(self.weights)
        return origin

    def build_model(self, checkpoint: dict, dtype=torch.float32):
        from ..config import WarpStateConfig
        from ..models.warpstate import WarpStateLM
        cfg = WarpStateConfig(**checkpoint["config"])
        cfg.gradient_checkpointing = self.s["gradient_checkpointing"]
        self.adjust_config(cfg)
        cfg.validate()
        if cfg.vocab_size != self.sp.vocab_size() or self.s["sequence_length"] % cfg.chunk_size:
            raise ValueError("the model does not fit the tokenizer's vocabulary, or sequence_length is not a whole "
                             "number of chunks")
        with torch.device("meta"):
            model = WarpStateLM(cfg)
        model.load_state_dict(checkpoint["model"], strict=True, assign=True)
        model = model.to(device=self.device, dtype=dtype)
        if self.device.type == "cpu":
            for p in model.parameters():        # memory-mapped checkpoint tensors must not alias training state
                p.data = p.data.clone()
        model.bf16_residuals = bool(self.s["bf16_residuals"])
        return model, cfg

    def adjust_config(self, cfg) -> None:
        pass

    def build_trainer(self) -> None:
        from ..ckpt.formats import load_checkpoint
        from .engine import Trainer
        s = self.s
        self.signature = dict(plan=self.plan, settings=s, data_sha256=self.manifest_hash,
                              tokenizer_sha256=self.tokenizer_hash, **self.signature_fields(), world_size=self.world,
                              device_type=self.device.type, torch_version=torch.__version__)
        self.latest = self.work / "latest.pt"
        self.resuming = self.latest.exists()
        saved = load_checkpoint(self.latest if self.resuming else self.weights)
        if self.resuming:
            if saved.get("format") != self.checkpoint_format or saved.get("signature") != self.signature:
                raise ValueError(f"{self.latest} was written by a run with another signature; "
                                 "resume with the same inputs or use a new output directory")
            if len(saved.get("rng_by_rank", [])) != self.world:
                raise ValueError(f"{self.latest} does not carry one RNG state per rank of this launch")
            self.origin = saved["origin"]
        self.model, self.cfg = self.build_model(saved)
        self.model.requires_grad_(True)
        self.trainer = Trainer(self.model, device=self.device, rank=self.rank, world_size=self.world, lr=s["lr"],
                               weight_decay=s["weight_decay"], max_grad_norm=s["clip_grad_norm"])
        if self.resuming:
            self.trainer.optimizer.load_state_dict(saved["optimizer"])
            self.progress = Progress(saved["step"], saved["sample_cursor"], saved["tokens_seen"], saved[self.scored_key])
            restore_rng(saved["rng_by_rank"][self.rank], self.device)
        del saved
        self.global_batch = s["micro_batch"] * s["grad_accum"] * self.world
        self.total_steps = math.ceil(len(self.train_data) / self.global_batch) * s["epochs"]
        if s["max_steps"] is not None:
            self.total_steps = min(self.total_steps, s["max_steps"])
        self.end_step = self.total_steps
        if self.args.max_steps is not None:
            self.end_step = min(self.total_steps, self.progress.step + self.args.max_steps)
        self.work.mkdir(parents=True, exist_ok=True)
        if self.rank == 0:
            record = dict(signature=self.signature, origin=self.origin, total_steps=self.total_steps,
                          train_rows=len(self.train_data), val_rows=len(self.val_data))
            (self.work / "settings.json").write_text(json.dumps(record, indent=2, default=str) + "\n")
            if self.progress.step < self.total_steps:
                (self.work / "completion.json").unlink(missing_ok=True)

    # ------------------------------------------------------------------ records
    def emit(self, event: str, **fields) -> None:
        if self.rank != 0:
            return
        p = self.progress
        record = dict(event=event, **fields, timestamp=time.time(), stage=self.stage, step=p.step,
                      tokens_seen=p.tokens_seen, sample_cursor=p.sample_cursor, **self.event_fields())
        record[self.scored_key] = p.scored_tokens
        line = json.dumps(record, allow_nan=False)
        with (self.work / "metrics.jsonl").open("a") as stream:
            stream.write(line + "\n")
        if event == "validation":
            atomic_json(self.work / "evaluation.json",
                        dict(record, data_sha256=self.manifest_hash, base_sha256=self.base_hash,
                             tokenizer_sha256=self.tokenizer_hash, available_validation_samples=len(self.val_data),
                             **self.evaluation_fields(record)))
        print(line, flush=True)

    def run_validation(self, full: bool) -> None:
        box = [self.validate(full) if self.rank == 0 else None]
        if self.world > 1:
            dist.broadcast_object_list(box, src=0, group=self.control)
        self.last_validation = box[0]
        self.last_validation_step = self.progress.step
        self.emit("validation", full_holdout=full, **self.last_validation)

    def submit_checkpoint(self, writer) -> None:
        mine = capture_rng(self.device)
        every = [mine]
        if self.world > 1:
            every = [None] * self.world
            dist.all_gather_object(every, mine, group=self.control)
        p = self.progress
        done = p.step >= self.total_steps

        def state():
            record = dict(format=self.checkpoint_format, signature=self.signature, origin=self.origin,
                          config=vars(self.cfg).copy(), model=clean_state_dict(self.model),
                          optimizer=self.trainer.optimizer.state_dict(), step=p.step, sample_cursor=p.sample_cursor,
                          tokens_seen=p.tokens_seen, val_loss=self.last_validation["val_loss"],
                          val_step=self.last_validation_step, rng_by_rank=every, completed=done,
                          total_steps=self.total_steps, **self.checkpoint_fields())
            record[self.scored_key] = p.scored_tokens
            return record

        writer.submit(state_factory=state)

    # ------------------------------------------------------------------ the sequence
    def execute(self) -> None:
        from ..ckpt.formats import load_checkpoint
        from ..ckpt.writer import DistributedCheckpointWriter
        from ..data.sft import update_indices
        self.open_environment()
        self.train_data, self.val_data, self.manifest, self.manifest_hash = self.load_data()
        export = load_checkpoint(self.weights)
        self.check_source(export)
        self.origin = self.origin_of(export)
        del export
        self.join_process_group()
        try:
            if not self.before_training():
                return
            self.build_trainer()
            self.after_trainer()
            s, p = self.s, self.progress
            with DistributedCheckpointWriter(self.latest, rank=self.rank, device=self.device,
                                             distributed=self.world > 1, control_group=self.control) as writer:
                self.run_validation(full=True)
                saved_at = p.step if self.resuming else -1
                self.model.train()
                while p.step < self.end_step and not self.stop_requested():
                    writer.check()
                    indices, cursor = update_indices(len(self.train_data), s["seed"], p.sample_cursor, s["epochs"],
                                                     self.global_batch)
                    if not indices:
                        break
                    lr = self.learning_rate(p.step)
                    began = time.perf_counter()
                    fields = self.run_update(indices, lr)
                    seconds = time.perf_counter() - began
                    tokens, scored = self.count_tokens(indices)
                    p.step += 1
                    p.sample_cursor = cursor
                    p.tokens_seen += tokens
                    p.scored_tokens += scored
                    self.emit("train", **fields, lr=lr, update_seconds=seconds, tokens_per_second=tokens / seconds,
                              update_samples=len(indices), **self.rate_fields(indices, scored, seconds))
                    if p.step % s["eval_every"] == 0 or p.step == self.end_step:
                        self.run_validation(full=p.step >= self.total_steps)
                    if p.step % s["save_every"] == 0 or p.step == self.end_step:
                        self.submit_checkpoint(writer)
                        saved_at = p.step
                if saved_at != p.step:
                    self.submit_checkpoint(writer)
                writer.flush()
                finished = p.step >= self.total_steps
                if self.rank == 0 and finished:
                    record = dict(format=self.completion_format, stage=self.stage, completed=True,
                                  paused_for_evaluation=True, step=p.step, total_steps=self.total_steps,
                                  tokens_seen=p.tokens_seen, val_loss=self.last_validation["val_loss"],
                                  evaluation_file=str(self.work / "evaluation.json"), checkpoint=str(self.latest),
                                  timestamp=time.time(), **self.completion_fields())
                    record[self.scored_key] = p.scored_tokens
                    atomic_json(self.work / "completion.json", record)
                self.emit("complete" if finished else "paused", total_steps=self.total_steps, checkpoint=str(self.latest))
            self.after_training()
        finally:
            if self.world > 1 and dist.is_initialized():
                dist.destroy_process_group()

    def rate_fields(self, indices, scored: int, seconds: float) -> dict:
        return {}

    def lock_directories(self) -> list:
        """Directories in which this rank takes its ``rank-<r>.lock``."""
        return [self.work]


def run_stage_cli(stage_class, module, argv, description: str, extra_dirs=(), extra_flags=(), signals=()):
    """Command line shared by the stage entry points: path flags, pause controls, signal handlers, per-rank
    lock files.  ``module.STOP`` is the process-wide stop flag (set by the handlers, read between updates)."""
    import argparse
    import signal as _signal
    parser = argparse.ArgumentParser(description=description)
    for name in ("config", "work-dir", "data-dir", "weights", "tokenizer", *extra_dirs):
        parser.add_argument("--" + name, type=Path, required=True)
    parser.add_argument("--max-steps", type=int, help="pause after this many more updates (the schedule is unchanged)")
    parser.add_argument("--stop-file", type=Path, help="default: <work-dir>/control/training-stop-request")
    parser.add_argument("--device", choices=("cuda", "cpu"), default="cuda")
    for flag in extra_flags:
        parser.add_argument(flag, action="store_true")
    args = parser.parse_args(argv)
    if args.max_steps is not None and args.max_steps < 1:
        parser.error("--max-steps must be at least 1")
    if args.stop_file is None:
        args.stop_file = args.work_dir / "control/training-stop-request"
    if not args.stop_file.resolve().is_relative_to(workspace()):
        parser.error("--stop-file must be inside the workspace")

    def request_stop(signum, frame):
        module.STOP = True

    for signum in (_signal.SIGTERM, _signal.SIGINT, *signals):
        _signal.signal(signum, request_stop)
    run = stage_class(args, lambda: module.STOP)
    rank = int(os.environ.get("RANK", "0"))
    with contextlib.ExitStack() as held:
        # one lock file per rank and directory: a second launch of the same rank is refused, ranks do not queue
        for directory in run.lock_directories():
            directory.mkdir(parents=True, exist_ok=True)
            held.enter_context(process_lock(directory / f"rank-{rank}.lock"))
        held.enter_context(base_pipeline_lock(run.plan))
        run.execute()
