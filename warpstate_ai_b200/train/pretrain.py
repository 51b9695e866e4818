"""Pretraining runner (the engine behind ``run_40b.py``).

Command-line surface, defaults, cross-validation of flags, resume semantics, metrics files and
stop protocol follow the reference runner (run_40b.py:25-165 flags, :459-796 training,
:805-840 preflight, :843-885 main).  Flags that select the reference's Inductor / Triton
execution experiments are accepted and recorded in the resume signature so that its command
lines and checkpoints keep working; here the hot path is always the hand-written sm_100a
kernels on CUDA (or plain PyTorch with ``--device cpu``), so those flags do not change what
runs (`train.flags` holds both flag tables).  Additional flags of this framework: ``--device``,
``--grad-sync``, ``--kernels``, ``--shard-optimizer``, ``--shard-params``; ``--ddp-bucket-cap-mb`` sizes the
ranges of the in-kernel gradient reduction.

Host-side control traffic (stop agreement, validation-loss broadcast, RNG gathering, checkpoint
status) goes over a gloo group, never through the training stream.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import math
import os
import random
import shutil
import signal
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
STOP = False


def request_stop(signum=None, frame=None) -> None:
    """Signal handler: the run stops at its next safe point (a preparation commit or the end of an update)."""
    global STOP
    STOP = True
    print("Stop requested: the current preparation batch or optimizer update will be the last one.", flush=True)


def arguments(argv=None):
    """Parsed, checked and resolved command line (flag tables: `train.flags`)."""
    from .flags import build_parser, check, inert_settings
    parser = build_parser()
    a = parser.parse_args(argv)
    check(parser, a)
    a.rank = int(os.environ.get("RANK", "0"))
    a.world_size = int(os.environ.get("WORLD_SIZE", "1"))
    a.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if a.world_size > 1 and a.stage != "train":
        parser.error("a multi-process launch runs --stage train only; prepare the corpus beforehand in one process")
    for name in ("work_dir", "tokenizer", "config", "weights", "matmul_plan"):
        if getattr(a, name) is not None:
            setattr(a, name, getattr(a, name).expanduser().resolve())
    a.kernels = "sm100a" if (a.kernels and a.device == "cuda") else "pytorch"
    if a.world_size == 1:
        a.shard_optimizer = False
    if a.rank == 0:
        for name, value, native in inert_settings(a):
            print(f"note: {name} {value} has no effect here: {native}.", flush=True)
    return a


def bootstrap(a) -> None:
    """With ``--bootstrap``: a virtual environment next to the sources with the pinned dependencies, then the same
    command line re-executed inside it (what the reference does unless told not to, reference run_40b.py:168-190).
    Off by default: machines without network access run in the interpreter they were started with."""
    import subprocess
    import sys
    if not a.bootstrap:
        return
    if sys.platform != "linux":
        raise RuntimeError("--bootstrap supports Linux only")
    env_dir = ROOT / ".server-venv"
    python = env_dir / "bin/python"
    if not python.exists():
        subprocess.run([sys.executable, "-m", "venv", str(env_dir)], check=True)
    stamp = env_dir / "warpstate-deps-v1.json"
    if not stamp.exists():
        pip = [str(python), "-m", "pip"]
        subprocess.run(pip + ["install", "--upgrade", "pip"], check=True)
        subprocess.run(pip + ["install", "-r", str(ROOT / "launch/requirements-training.txt")], check=True)
        subprocess.run(pip + ["check"], check=True)
        (env_dir / "requirements-resolved.txt").write_text(subprocess.check_output(pip + ["freeze"], text=True))
        stamp.write_text(json.dumps({"installed": time.time()}))
    forwarded = [arg for arg in sys.argv[1:] if arg != "--bootstrap"]
    os.execv(str(python), [str(python), "-u", str(ROOT / "run_40b.py"), *forwarded, "--no-bootstrap"])


# start-up pieces (where the run begins, device requirements, allocator cap, preflight) live in train.startup
from .startup import cap_device_memory as configure_memory  # noqa: E402,F401
from .startup import preflight  # noqa: E402,F401


# --------------------------------------------------------------------------- the run
class _FrozenState:
    """An already materialised ``state_dict()`` behind the optimizer interface `server_state` expects."""

    def __init__(self, state: dict):
        self._state = state

    def state_dict(self) -> dict:
        return self._state


class PretrainRun:
    """State of one training process between `setup()` and the end of `loop()`."""

    def __init__(self, a):
        self.a = a

    # ---- setup
    def setup(self) -> None:
        import numpy as np
        import torch
        import torch.distributed as dist
        from ..ckpt.formats import restore_rng, seed_everything
        from ..ckpt.writer import host_control_group
        from ..data.prepare import check_manifest
        from ..optim import cosine_lr
        from .engine import Trainer
        from .signature import check_resume_signature, train_signature
        from .startup import StartPoint, check_fit, require_device

        a = self.a
        self.torch, self.np, self.dist = torch, np, dist
        self.manifest = check_manifest(a)
        a.matmul_metadata = None
        a.backward_layout_metadata = None
        if a.matmul_plan is not None:
            plan = json.loads(a.matmul_plan.read_text())
            a.matmul_metadata = {"format": plan.get("format"), "sha256": __import__("hashlib").sha256(
                a.matmul_plan.read_bytes()).hexdigest()}
        if a.backward_layout != "baseline":
            a.backward_layout_metadata = {"mode": a.backward_layout, "implementation": "fused attention backward"}
        self.distributed = a.world_size > 1
        self.device, self.gpu_name, self.gpu_bytes = require_device(a)
        torch.set_num_threads(min(a.workers, 8))
        seed_everything(a.seed, a.rank, self.device)
        self.control = host_control_group() if self.distributed else None
        self.run_dir = a.work_dir / "run"
        self.run_dir.mkdir(exist_ok=True)
        self.latest = self.run_dir / "latest.pt"
        start = StartPoint.resolve(a)
        resuming = start.kind == "resume"
        source, checkpoint = start.source, start.checkpoint
        cfg = start.config(a)
        check_fit(cfg, a)
        self.signature = train_signature(a, self.manifest)
        changed = resuming and check_resume_signature(checkpoint["signature"], self.signature, a.reconfigure)
        model = start.build_model(cfg, a.seed).to(device=self.device, dtype=torch.float32).requires_grad_(True)
        masters = start.legacy_masters()
        if masters is not None:
            with torch.no_grad():      # the legacy CPU-offload layout keeps unrounded FP32 masters: prefer them
                for parameter, master in zip(model.parameters(), masters, strict=True):
                    parameter.copy_(master)
        cfg.gradient_checkpointing = a.activation_checkpointing
        model.loss_chunk_size = a.loss_chunk_size
        model.bf16_residuals = bool(a.bf16_residuals)
        model.train()
        self.cfg, self.model = cfg, model
        self.parameters = model.num_parameters()      # before any sharding re-homes the parameters
        sync = None
        if self.distributed:
            from ..parallel.grad_sync import make_grad_sync
            kind = {"auto": "auto", "fused": "fused", "nccl": "collective"}[a.grad_sync]
            sync = make_grad_sync(self.device, a.world_size, a.rank, None, kind=kind,
                                  bucket_cap_bytes=int(a.ddp_bucket_cap_mb * 2 ** 20))
        if a.device == "cuda" and a.kernels != "sm100a":
            from ..ops import fused
            fused._enabled = False
        self.trainer = Trainer(model, device=self.device, rank=a.rank, world_size=a.world_size, lr=a.lr,
                               weight_decay=a.weight_decay, grad_sync=sync,
                               shard_optimizer=getattr(a, "shard_optimizer", False),
                               shard_params=None if a.shard_params == "off" else a.shard_params,
                               bucket_cap_bytes=int(a.ddp_bucket_cap_mb * 2 ** 20))
        self.seen, self.step = 0, 0
        if resuming:
            self.trainer.optimizer.load_state_dict(checkpoint["optimizer"])
            self.seen, self.step = checkpoint["tokens_seen"], checkpoint["step"]
            rank_states = checkpoint.get("rng_by_rank")
            if rank_states is None:
                rank_states = [{"torch": checkpoint["rng_torch"], "cuda": checkpoint["rng_cuda"][0],
                                "numpy": checkpoint["rng_numpy"], "python": checkpoint["rng_python"]}]
            if a.rank < len(rank_states):
                restore_rng(rank_states[a.rank], self.device)
            else:  # a rank added by --reconfigure gets a reproducible stream of its own
                seed_everything(a.seed + a.rank, 0, self.device)
        fresh_origin = {"initialization": "random", "seed": a.seed, "previous_training_tokens": 0}
        self.origin = checkpoint.get("origin", fresh_origin if (not resuming and a.from_scratch) else
                                     {"path": str(source), "previous_training_tokens": checkpoint.get("tokens_seen")})
        self.history = list(checkpoint.get("execution_history", []))
        if changed:
            self.history.append({"step": self.step, "tokens": self.seen, "timestamp": time.time(),
                                 "from": checkpoint["signature"]["settings"], "to": self.signature["settings"]})
            if a.rank == 0:
                print(f"Reconfiguring execution at step {self.step}, tokens={self.seen:,}; preserving model, "
                      "optimizer and schedule.", flush=True)
        self.last_val = checkpoint.get("val_loss") if resuming else None
        del checkpoint, start
        if shutil.disk_usage(self.run_dir).free < self.parameters * 28:
            raise RuntimeError("Need free space for checkpoint plus atomic replacement")
        self.train_data = np.memmap(a.work_dir / "data/train.bin", dtype="<u2", mode="r")
        self.val_data = np.memmap(a.work_dir / "data/val.bin", dtype="<u2", mode="r")
        self.batch_tokens = a.micro_batch * a.seq_len
        self.update_tokens = self.batch_tokens * a.grad_accum * a.world_size
        self.total_steps = math.ceil(a.train_tokens / self.update_tokens)
        self.end_step = self.total_steps
        if a.max_steps is not None:
            self.end_step = min(self.end_step, self.step + a.max_steps)
        if a.stop_at_step is not None:
            self.end_step = min(self.end_step, a.stop_at_step)
        self.lr_at = lambda step: cosine_lr(step, lr=a.lr, min_lr=a.min_lr, warmup_steps=a.warmup_steps,
                                            total_steps=self.total_steps)
        if a.rank == 0:
            print(f"{a.world_size} x {self.gpu_name}: {self.gpu_bytes / 1024 ** 3:.1f} GiB/device; "
                  f"{self.parameters:,} parameters; FP32 master/grad/AdamW + BF16 compute ({a.kernels}); "
                  f"start tokens={self.seen:,}", flush=True)
            if self.end_step < self.total_steps:
                print(f"Pause boundary: optimizer step {self.end_step}; loaded step {self.step}; "
                      f"learning-rate schedule remains {self.total_steps} steps.", flush=True)
                if self.step >= self.end_step:
                    print("Pause boundary already reached; no further optimizer updates.", flush=True)
            self.write_settings()

    def write_settings(self) -> None:
        a, torch = self.a, self.torch
        runtime = {k: getattr(a, k) for k in (
            "stop_at_step", "max_steps", "vram_limit_gib", "vram_headroom_gib", "autocast_cache", "eval_micro_batch",
            "eval_every", "save_every", "async_checkpoint", "bf16_residuals", "activation_mode", "gradient_mode",
            "overlap_swap_collectives", "overlap_runtime_estimates", "overlap_memory_budget",
            "overlap_producer_schedule", "cache_core_weight_casts", "ddp_bucket_cap_mb", "ddp_batched_grad_copy",
            "kernels", "grad_sync", "device")}
        runtime.update(end_step=self.end_step, matmul_execution=a.matmul_metadata,
                       backward_layout_execution=a.backward_layout_metadata,
                       cuda_visible_devices=os.getenv("CUDA_VISIBLE_DEVICES"))
        (self.run_dir / "settings.json").write_text(json.dumps({
            "signature": self.signature, "gpu": self.gpu_name, "torch": torch.__version__, "cuda": torch.version.cuda,
            "parameters": self.parameters, "origin": self.origin, "execution_history": self.history,
            "runtime": runtime}, indent=2, default=str))

    # ---- host-side collectives
    def agree_max(self, value: int) -> int:
        if not self.distributed:
            return value
        t = self.torch.tensor([value], dtype=self.torch.int64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX, group=self.control)
        return int(t.item())

    def stop_requested(self) -> bool:
        stop_file = os.environ.get("WARPSTATE_STOP_FILE")
        requested = STOP or bool(stop_file and Path(stop_file).is_file())
        return bool(self.agree_max(int(requested)))

    # ---- evaluation: rank 0 only, fixed evenly spaced windows of the validation file
    def evaluate(self) -> float:
        a, np = self.a, self.np
        value = 0.0
        if a.rank == 0:
            window = a.eval_micro_batch * a.seq_len
            cursors = np.linspace(0, max(0, len(self.val_data) - window - 1), a.eval_batches, dtype=np.int64)
            value = self.trainer.evaluate_tokens(self.val_data, cursors, a.eval_micro_batch, a.seq_len)
        if self.distributed:
            box = [value]
            self.dist.broadcast_object_list(box, src=0, group=self.control)
            value = box[0]
        if not math.isfinite(value):
            raise RuntimeError("Non-finite validation loss")
        return value

    # ---- checkpoint
    def save(self, validation: float) -> None:
        from ..ckpt.formats import capture_rng, server_state
        from ..ckpt.writer import atomic_torch_save
        a = self.a
        state = capture_rng(self.device)
        rank_states = [state]
        if self.distributed:
            rank_states = [None] * a.world_size
            self.dist.all_gather_object(rank_states, state, group=self.control)

        optimizer = self.trainer.optimizer
        model_state = None
        if self.trainer.sharded is not None or hasattr(optimizer, "gather_master"):
            # sharded state: assembling the unsharded checkpoint is collective, so every rank does it now
            model_state = self.trainer.model_state_dict()
            optimizer = _FrozenState(optimizer.state_dict())

        def build_state():
            print("Staging full CPU checkpoint..." if a.async_checkpoint else "Saving full checkpoint...", flush=True)
            return server_state(signature=self.signature, origin=self.origin, history=self.history, cfg=self.cfg,
                                model=self.model, model_state=model_state, optimizer=optimizer, step=self.step,
                                tokens_seen=self.seen, val_loss=validation, val_step=self.last_val_step,
                                val_tokens=self.last_val_tokens, rng_by_rank=rank_states)

        if self.writer is not None:
            seconds = self.writer.submit(state_factory=build_state)
            if a.rank == 0:
                print(f"Staged step {self.step}, tokens={self.seen:,} for asynchronous checkpoint; "
                      f"synchronous CPU staging {seconds:.2f}s.", flush=True)
        else:
            if a.rank == 0:
                atomic_torch_save(self.latest, build_state())
                print("Saved " + str(self.latest), flush=True)
            if self.distributed:
                self.dist.barrier(group=self.control)

    # ---- the loop
    def loop(self) -> None:
        from ..ckpt.writer import DistributedCheckpointWriter
        from ..data.tokens import HostBatcher
        from ..utils.io import append_jsonl
        a, torch = self.a, self.torch
        self.writer = None
        if a.async_checkpoint:
            self.writer = DistributedCheckpointWriter(self.latest, rank=a.rank, device=self.device,
                                                      distributed=self.distributed, control_group=self.control)
        batcher = HostBatcher(a.micro_batch, a.seq_len, self.device)
        with self.writer if self.writer is not None else contextlib.nullcontext():
            self.last_val = self.evaluate()
            self.last_val_step, self.last_val_tokens = self.step, self.seen
            if a.rank == 0:
                print(f"initial validation loss: {self.last_val:.5f}", flush=True)
            while self.seen < a.train_tokens and self.step < self.end_step:
                if self.writer is not None:
                    self.writer.check()
                if self.stop_requested():
                    self.save(self.last_val)
                    break
                target = min(self.update_tokens, a.train_tokens - self.seen)
                rate = self.lr_at(self.step)
                result = self.trainer.pretrain_update(self.train_data, self.seen, target, a.micro_batch, a.seq_len,
                                                      rate, batcher)
                elapsed = result.seconds
                stats = self.memory_stats(elapsed)
                gpu_stats = [stats]
                if self.distributed:
                    gpu_stats = [None] * a.world_size
                    self.dist.all_gather_object(gpu_stats, stats, group=self.control)
                    elapsed = max(item["seconds"] for item in gpu_stats)
                self.seen += target
                self.step += 1
                record = {"step": self.step, "tokens": self.seen, "loss": result.loss, "lr": rate,
                          "grad_norm": result.grad_norm, "tokens_per_second": target / elapsed, "seconds": elapsed,
                          "timestamp": time.time(), "world_size": a.world_size, "gpu_memory": gpu_stats,
                          "peak_vram_gib": max(i["allocated"] for i in gpu_stats),
                          "peak_reserved_vram_gib": max(i["reserved"] for i in gpu_stats),
                          "device_free_vram_gib": min(i["free"] for i in gpu_stats)}
                if self.device.type == "cuda":
                    torch.cuda.reset_peak_memory_stats()
                ending = self.stop_requested() or self.seen == a.train_tokens or self.step >= self.end_step
                if self.step % a.eval_every == 0 or ending:
                    self.last_val = self.evaluate()
                    self.last_val_step, self.last_val_tokens = self.step, self.seen
                    if a.rank == 0:
                        append_jsonl(self.run_dir / "validation.jsonl",
                                     {"step": self.step, "tokens": self.seen, "loss": self.last_val})
                record.update(val_loss=self.last_val, val_step=self.last_val_step, val_tokens=self.last_val_tokens)
                if a.rank == 0:
                    val = f"val {self.last_val:.5f} (step {self.last_val_step}) | " if self.last_val_step == self.step else ""
                    print(f"step {self.step}/{self.total_steps} | {self.seen:,}/{a.train_tokens:,} tokens | "
                          f"loss {record['loss']:.4f} | {val}{record['tokens_per_second']:,.0f} tok/s | "
                          f"peak {record['peak_vram_gib']:.2f} GiB allocated / "
                          f"{record['peak_reserved_vram_gib']:.2f} GiB reserved | "
                          f"free {record['device_free_vram_gib']:.2f} GiB", flush=True)
                    append_jsonl(self.run_dir / "metrics.jsonl", record)
                if self.step % a.save_every == 0 or ending:
                    self.save(self.last_val)
                if ending:
                    break

    def memory_stats(self, seconds: float) -> dict:
        torch = self.torch
        if self.device.type != "cuda":
            return {"allocated": 0.0, "reserved": 0.0, "free": 0.0, "seconds": seconds}
        return {"allocated": torch.cuda.max_memory_allocated(self.device) / 1024 ** 3,
                "reserved": torch.cuda.max_memory_reserved(self.device) / 1024 ** 3,
                "free": torch.cuda.mem_get_info(self.device)[0] / 1024 ** 3, "seconds": seconds}


def train(a) -> None:
    run = PretrainRun(a)
    run.setup()
    run.loop()


@contextlib.contextmanager
def process_group(a):
    """The training process group of a multi-process launch (NCCL on GPUs, gloo on CPU); nothing for one process."""
    if a.world_size == 1 or a.stage == "prepare":
        yield None
        return
    import torch
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if a.device == "cuda":
        dist.init_process_group("nccl", device_id=torch.device("cuda", a.local_rank))
    else:
        dist.init_process_group("gloo")
    try:
        yield dist
    finally:
        dist.destroy_process_group()


def main(argv=None) -> None:
    from ..utils.io import process_lock
    a = arguments(argv)
    bootstrap(a)
    if not a.tokenizer.is_file():
        raise FileNotFoundError(a.tokenizer)
    training = a.stage != "prepare"
    has_start = (a.work_dir / "run/latest.pt").exists() or a.from_scratch or (a.weights is not None and a.weights.is_file())
    if training and not has_start:
        raise ValueError("nothing to start from: pass --weights <checkpoint.pt>, or --from-scratch for a fresh model")
    a.work_dir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("HF_HOME", str(a.work_dir / "hf-cache"))
    for name in ("SIGINT", "SIGTERM", "SIGUSR1"):
        if hasattr(signal, name):
            signal.signal(getattr(signal, name), request_stop)
    if training and a.device == "cuda":
        import torch
        torch.cuda.set_device(a.local_rank)
        configure_memory(a)
    with process_group(a) as dist, contextlib.ExitStack() as held:
        if a.rank == 0:
            # one pretraining job per work directory; post-training ranks hold the same file shared
            held.enter_context(process_lock(a.work_dir / "pipeline.lock"))
        if dist is not None:
            dist.barrier()
        if training:
            preflight(a)
        if a.stage in ("all", "prepare"):
            from ..data.prepare import prepare
            if not prepare(a, stop_requested=lambda: STOP):
                return                      # stopped after a commit; the next launch continues
        if training:
            train(a)


if __name__ == "__main__":
    main()
