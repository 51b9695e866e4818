"""Pretraining runner (the engine behind ``run_40b.py``).

Command-line surface, defaults, cross-validation of flags, resume semantics, metrics files and
stop protocol follow the reference runner (run_40b.py:25-165 flags, :459-796 training,
:805-840 preflight, :843-885 main).  Flags that select the reference's Inductor / Triton
execution experiments are accepted and recorded in the resume signature so that its command
lines and checkpoints keep working; here the hot path is always the hand-written sm_100a
kernels on CUDA (or plain PyTorch with ``--device cpu``), so those flags do not change what
runs.  Additional flags of this framework: ``--device``, ``--grad-sync``, ``--kernels``.

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
    global STOP
    STOP = True
    print("Stop requested; committing preparation or finishing the current optimizer update.", flush=True)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="WarpState pretraining on B200 (prepare + train)")
    init = p.add_mutually_exclusive_group()
    init.add_argument("--weights", type=Path, help="existing trusted WarpState checkpoint used to initialise a new run")
    init.add_argument("--from-scratch", action="store_true", help="initialise a new model from --config and --seed")
    p.add_argument("--work-dir", type=Path, default=ROOT / "work")
    p.add_argument("--tokenizer", type=Path, default=ROOT / "tokenizer.model")
    p.add_argument("--config", type=Path, default=ROOT / "configs/warpstate_2b.json")
    p.add_argument("--stage", choices=["all", "prepare", "train"], default="all")
    p.add_argument("--verify-data", action="store_true")
    p.add_argument("--dataset", default="HuggingFaceFW/fineweb-edu")
    p.add_argument("--dataset-config", default="sample-100BT")
    p.add_argument("--revision", default="main")
    p.add_argument("--train-tokens", type=int, default=40_000_000_000)
    p.add_argument("--val-tokens", type=int, default=1_048_576)
    p.add_argument("--workers", type=int, default=min(16, os.cpu_count() or 4))
    p.add_argument("--documents-per-batch", type=int, default=256)
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--micro-batch", type=int, default=8)
    p.add_argument("--grad-accum", type=int, default=8)
    p.add_argument("--lr", type=float, default=1.5e-4)
    p.add_argument("--min-lr", type=float, default=1.5e-5)
    p.add_argument("--warmup-steps", type=int, default=1000)
    p.add_argument("--weight-decay", type=float, default=0.1)
    p.add_argument("--activation-checkpointing", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--autocast-cache", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--vram-limit-gib", type=float)
    p.add_argument("--vram-headroom-gib", type=float, default=3.0)
    p.add_argument("--loss-chunk-size", type=int, default=1024)
    p.add_argument("--loss-mode", choices=["checkpointed", "full", "compiled-full"], default="checkpointed")
    p.add_argument("--bf16-residuals", action=argparse.BooleanOptionalAction, default=False)
    p.add_argument("--activation-mode", choices=["baseline", "swiglu", "rmsnorm", "all"], default="baseline")
    p.add_argument("--matmul-plan", type=Path)
    p.add_argument("--gradient-mode", choices=["eager", "compiled-autograd", "compiled-autograd-overlap"],
                   default="eager")
    p.add_argument("--backward-layout", choices=["baseline", "inspect", "paired"], default="baseline")
    p.add_argument("--overlap-swap-collectives", action="store_true")
    p.add_argument("--overlap-runtime-estimates", action="store_true")
    p.add_argument("--overlap-producer-schedule", action="store_true")
    p.add_argument("--overlap-memory-budget", type=float, default=0.0)
    p.add_argument("--cache-core-weight-casts", action=argparse.BooleanOptionalAction, default=False)
    p.add_argument("--ddp-bucket-cap-mb", type=float, default=128)
    p.add_argument("--ddp-batched-grad-copy", action=argparse.BooleanOptionalAction, default=False)
    p.add_argument("--compile", action="store_true")
    p.add_argument("--compile-core", action="store_true")
    p.add_argument("--compile-mode", choices=["default", "reduce-overhead", "max-autotune-no-cudagraphs"],
                   default="default")
    p.add_argument("--reconfigure", action="store_true")
    p.add_argument("--eval-every", type=int, default=500)
    p.add_argument("--eval-batches", type=int, default=8)
    p.add_argument("--eval-micro-batch", type=int, default=1)
    p.add_argument("--save-every", type=int, default=1000)
    p.add_argument("--async-checkpoint", action=argparse.BooleanOptionalAction, default=False)
    p.add_argument("--max-steps", type=int)
    p.add_argument("--stop-at-step", type=int)
    p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--no-bootstrap", action="store_true", help="accepted for compatibility; nothing is installed")
    p.add_argument("--test-small-gpu", action="store_true", help="tests only: bypass the 80 GiB device requirement")
    # this framework
    p.add_argument("--device", choices=["cuda", "cpu"], default="cuda", help="cpu runs the plain-PyTorch path (tests)")
    p.add_argument("--grad-sync", choices=["auto", "fused", "nccl"], default="auto",
                   help="multi-GPU gradient path: in-kernel all-reduce over NVLink peer memory, or NCCL")
    p.add_argument("--shard-optimizer", action="store_true",
                   help="multi-GPU: each rank keeps AdamW state for 1/world of every bucket and broadcasts its "
                        "updated BF16 weights from the update kernel (checkpoints stay unsharded)")
    p.add_argument("--kernels", action=argparse.BooleanOptionalAction, default=True,
                   help="use the sm_100a kernel library on CUDA")
    return p


def validate(p: argparse.ArgumentParser, a) -> None:
    positive = ("train_tokens", "val_tokens", "workers", "documents_per_batch", "seq_len", "micro_batch",
                "grad_accum", "loss_chunk_size", "eval_every", "eval_batches", "eval_micro_batch", "save_every",
                "warmup_steps")
    for key in positive:
        if getattr(a, key) < 1:
            p.error(key + " must be positive")
    if a.max_steps is not None and a.max_steps < 1:
        p.error("--max-steps must be positive")
    if a.stop_at_step is not None and a.stop_at_step < 1:
        p.error("--stop-at-step must be positive")
    if a.vram_limit_gib is not None and (not math.isfinite(a.vram_limit_gib) or a.vram_limit_gib <= 0):
        p.error("--vram-limit-gib must be finite and positive")
    if not math.isfinite(a.vram_headroom_gib) or a.vram_headroom_gib < 0:
        p.error("--vram-headroom-gib must be finite and nonnegative")
    if not 0 < a.min_lr <= a.lr or a.weight_decay < 0:
        p.error("Invalid learning rate or weight decay")
    if a.train_tokens < 2 or a.val_tokens <= a.seq_len:
        p.error("Need at least 2 training tokens and more validation tokens than seq-len")
    if a.compile and a.compile_core:
        p.error("Choose --compile or --compile-core")
    if a.compile_mode != "default" and not (a.compile or a.compile_core):
        p.error("A nondefault --compile-mode requires --compile-core or --compile")
    if not math.isfinite(a.ddp_bucket_cap_mb) or a.ddp_bucket_cap_mb * 1024 ** 2 < 1:
        p.error("--ddp-bucket-cap-mb must be finite and at least one byte in MiB")
    if not math.isfinite(a.overlap_memory_budget) or not 0 <= a.overlap_memory_budget <= 0.25:
        p.error("--overlap-memory-budget must be finite and between 0 and 0.25")
    overlap_options = (a.overlap_swap_collectives or a.overlap_runtime_estimates or a.overlap_memory_budget
                       or a.overlap_producer_schedule)
    if a.gradient_mode != "compiled-autograd-overlap" and overlap_options:
        p.error("Overlap scheduling options require --gradient-mode compiled-autograd-overlap")
    if a.overlap_producer_schedule and (a.overlap_swap_collectives or a.overlap_runtime_estimates
                                        or a.overlap_memory_budget):
        p.error("--overlap-producer-schedule must be tested separately from other overlap scheduling options")
    if a.gradient_mode != "eager" and a.ddp_batched_grad_copy:
        p.error("--ddp-batched-grad-copy uses the C++ reducer and cannot be combined with compiled autograd")
    if a.backward_layout != "baseline":
        ok = (a.gradient_mode == "compiled-autograd-overlap" and a.compile_core and not a.activation_checkpointing
              and a.bf16_residuals and a.micro_batch == 4 and a.seq_len == 2048 and a.activation_mode == "baseline"
              and a.matmul_plan is None and a.compile_mode == "default")
        if not ok:
            p.error("--backward-layout requires compiled-autograd-overlap, --compile-core, "
                    "--no-activation-checkpointing, --bf16-residuals, microbatch 4, sequence 2048, "
                    "default compile mode, baseline activations and no matmul plan")
    if a.gradient_mode != "eager" and a.activation_mode != "baseline":
        p.error("Standalone activation modes require eager gradients; use baseline activations "
                "for compiled autograd, including matmul-plan epilogues")
    if a.cache_core_weight_casts and a.activation_checkpointing:
        p.error("--cache-core-weight-casts requires --no-activation-checkpointing")
    if a.cache_core_weight_casts and a.gradient_mode != "eager":
        p.error("Core weight cast caching and compiled autograd must be tested separately")
    if a.compile_mode == "reduce-overhead" and (a.cache_core_weight_casts or a.gradient_mode != "eager"):
        p.error("Weight cast caching and compiled autograd require a compile mode without CUDA graphs")
    if a.matmul_plan is not None and a.cache_core_weight_casts:
        p.error("--matmul-plan cannot be combined with external core weight cast caching")
    if a.matmul_plan is not None and a.compile_mode == "reduce-overhead":
        p.error("--matmul-plan currently requires a compile mode without CUDA graphs")
    if a.matmul_plan is not None and a.gradient_mode != "eager" and a.activation_checkpointing:
        p.error("--matmul-plan with compiled autograd requires --no-activation-checkpointing")


def arguments(argv=None):
    p = build_parser()
    a = p.parse_args(argv)
    validate(p, a)
    a.rank = int(os.environ.get("RANK", "0"))
    a.world_size = int(os.environ.get("WORLD_SIZE", "1"))
    a.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if a.world_size > 1 and a.stage != "train":
        p.error("torchrun supports --stage train only; prepare the corpus once beforehand")
    for name in ("work_dir", "tokenizer", "config", "weights", "matmul_plan"):
        if getattr(a, name) is not None:
            setattr(a, name, getattr(a, name).expanduser().resolve())
    a.kernels = "sm100a" if (a.kernels and a.device == "cuda") else "pytorch"
    a.shard_optimizer = False
    return a


# --------------------------------------------------------------------------- device / memory
def configure_memory(a) -> None:
    """Cap the caching allocator before anything is allocated (reference run_40b.py:442-456)."""
    if a.vram_limit_gib is None or a.device != "cuda":
        return
    import torch
    device = torch.device("cuda", a.local_rank)
    free, total = torch.cuda.mem_get_info(device)
    limit = int(a.vram_limit_gib * 1024 ** 3)
    required = limit + int(a.vram_headroom_gib * 1024 ** 3)
    if limit > total or free < required:
        raise RuntimeError(f"Only {free / 1024 ** 3:.2f} GiB free; need {required / 1024 ** 3:.2f} GiB "
                           "for the requested allocator cap and headroom")
    torch.cuda.set_per_process_memory_fraction(limit / total, device)
    print(f"CUDA allocator cap {a.vram_limit_gib:.2f} GiB; free before model {free / 1024 ** 3:.2f} GiB", flush=True)


def tokenizer_vocab(path: Path) -> int:
    import sentencepiece as spm
    return spm.SentencePieceProcessor(model_file=str(path)).vocab_size()


def preflight(a) -> None:
    """Reject incompatible weights / hardware before a long preparation or run."""
    import torch
    from ..ckpt.formats import SERVER_FORMAT, load_checkpoint
    from ..config import WarpStateConfig
    from ..models.warpstate import WarpStateLM
    if a.device == "cuda":
        if not torch.cuda.is_available() or not torch.cuda.is_bf16_supported():
            raise RuntimeError("BF16 CUDA GPU required")
        if not a.test_small_gpu and torch.cuda.get_device_properties(a.local_rank).total_memory < 80 * 1024 ** 3:
            raise RuntimeError("The normal preset requires a GPU with at least 80 GiB")
    latest = a.work_dir / "run/latest.pt"
    source = latest if latest.exists() else a.weights
    fresh = not latest.exists() and a.from_scratch
    checkpoint = {} if fresh else load_checkpoint(source)
    if not fresh and "model" not in checkpoint:
        raise ValueError("Expected a WarpState checkpoint with a model state dictionary, not arbitrary model weights")
    cfg = WarpStateConfig(**checkpoint.get("config", json.loads(a.config.read_text()) if fresh or "config" not in checkpoint else {}))
    cfg.validate()
    if cfg.vocab_size != tokenizer_vocab(a.tokenizer):
        raise ValueError("Tokenizer/model vocabulary mismatch")
    if a.seq_len % cfg.chunk_size:
        raise ValueError("Sequence length must be divisible by the local tile size")
    with torch.device("meta"):
        probe = WarpStateLM(cfg)
    if not fresh:
        probe.load_state_dict(checkpoint["model"], assign=True, strict=True)
    if not a.test_small_gpu and not 2_000_000_000 <= probe.num_parameters() <= 2_020_000_000:
        raise ValueError("This package expects the approximately 2B WarpState architecture")
    optimizer_state = checkpoint.get("optimizer", {})
    if optimizer_state.get("kind") == "cpu_offload_adamw":
        for parameter, master in zip(probe.parameters(), optimizer_state["masters"], strict=True):
            if parameter.shape != master.shape:
                raise ValueError("FP32 master weight shape mismatch")
    if latest.exists() and checkpoint.get("format") != SERVER_FORMAT:
        raise ValueError("Use --weights to initialize a new run; work/run/latest.pt is not a server checkpoint")
    what = "configuration for fresh initialization" if fresh else "weights"
    print(f"Preflight: compatible WarpState {what} ({probe.num_parameters():,} parameters).", flush=True)


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
        from ..ckpt.formats import SERVER_FORMAT, load_checkpoint, restore_rng, seed_everything
        from ..ckpt.writer import host_control_group
        from ..config import WarpStateConfig
        from ..data.prepare import check_manifest
        from ..models.warpstate import WarpStateLM
        from ..optim import cosine_lr
        from .engine import Trainer
        from .signature import check_resume_signature, train_signature

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
        if a.device == "cuda":
            if not torch.cuda.is_available() or not torch.cuda.is_bf16_supported():
                raise RuntimeError("BF16 CUDA GPU required")
            self.device = torch.device("cuda", a.local_rank)
            props = torch.cuda.get_device_properties(self.device)
            if not a.test_small_gpu and props.total_memory < 80 * 1024 ** 3:
                raise RuntimeError("This preset requires a GPU with at least 80 GiB; use --test-small-gpu for tests")
            self.gpu_name, self.gpu_bytes = props.name, props.total_memory
        else:
            self.device = torch.device("cpu")
            self.gpu_name, self.gpu_bytes = "cpu", 0
        torch.set_num_threads(min(a.workers, 8))
        seed_everything(a.seed, a.rank, self.device)
        self.control = host_control_group() if self.distributed else None
        self.run_dir = a.work_dir / "run"
        self.run_dir.mkdir(exist_ok=True)
        self.latest = self.run_dir / "latest.pt"
        resuming = self.latest.exists()
        source = self.latest if resuming else a.weights
        if not resuming and a.from_scratch:
            checkpoint = {}
        elif source is None or not source.is_file():
            raise ValueError("First launch requires --weights /path/to/your/checkpoint.pt")
        else:
            checkpoint = load_checkpoint(source)
        cfg = WarpStateConfig(**checkpoint.get("config", json.loads(a.config.read_text()) if "config" not in checkpoint else {}))
        cfg.validate()
        if a.seq_len % cfg.chunk_size:
            raise ValueError("seq-len must be divisible by model chunk_size")
        if cfg.vocab_size != tokenizer_vocab(a.tokenizer):
            raise ValueError("Tokenizer/model vocabulary mismatch; use the exact original tokenizer")
        self.signature = train_signature(a, self.manifest)
        changed = False
        if resuming:
            if checkpoint.get("format") != SERVER_FORMAT:
                raise ValueError("Resume settings/data differ; unsupported checkpoint format")
            changed = check_resume_signature(checkpoint["signature"], self.signature, a.reconfigure)
        if not resuming and a.from_scratch:
            print(f"Initializing fresh FP32 weights with seed {a.seed}.", flush=True)
            model = WarpStateLM(cfg)
        else:
            with torch.device("meta"):
                model = WarpStateLM(cfg)
            model.load_state_dict(checkpoint["model"], assign=True)
        model = model.to(device=self.device, dtype=torch.float32).requires_grad_(True)
        old_opt = checkpoint.get("optimizer", {})
        if not resuming and old_opt.get("kind") == "cpu_offload_adamw":
            with torch.no_grad():  # prefer unrounded FP32 masters of the legacy CPU-offload layout
                for parameter, master in zip(model.parameters(), old_opt["masters"], strict=True):
                    if parameter.shape != master.shape:
                        raise ValueError("Master weight shape mismatch")
                    parameter.copy_(master)
        cfg.gradient_checkpointing = a.activation_checkpointing
        model.loss_chunk_size = a.loss_chunk_size
        model.train()
        self.cfg, self.model = cfg, model
        sync = None
        if self.distributed:
            from ..parallel.grad_sync import make_grad_sync
            kind = {"auto": "auto", "fused": "fused", "nccl": "collective"}[a.grad_sync]
            sync = make_grad_sync(self.device, a.world_size, a.rank, None, kind=kind)
        if a.device == "cuda" and a.kernels != "sm100a":
            from ..ops import fused
            fused._enabled = False
        self.trainer = Trainer(model, device=self.device, rank=a.rank, world_size=a.world_size, lr=a.lr,
                               weight_decay=a.weight_decay, grad_sync=sync,
                               shard_optimizer=getattr(a, "shard_optimizer", False))
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
        del checkpoint, old_opt
        self.parameters = model.num_parameters()
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
        if hasattr(optimizer, "gather_master"):
            # sharded optimizer: assembling the unsharded state is collective, so every rank does it now
            self.trainer.gather_for_checkpoint()
            optimizer = _FrozenState(optimizer.state_dict())

        def build_state():
            print("Staging full CPU checkpoint..." if a.async_checkpoint else "Saving full checkpoint...", flush=True)
            return server_state(signature=self.signature, origin=self.origin, history=self.history, cfg=self.cfg,
                                model=self.model, optimizer=optimizer, step=self.step,
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


def main(argv=None) -> None:
    from ..utils.io import process_lock
    a = arguments(argv)
    if not a.tokenizer.is_file():
        raise FileNotFoundError(a.tokenizer)
    if (a.stage != "prepare" and not (a.work_dir / "run/latest.pt").exists() and not a.from_scratch
            and (a.weights is None or not a.weights.is_file())):
        raise ValueError("Supply --weights or explicitly choose --from-scratch before training")
    a.work_dir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("HF_HOME", str(a.work_dir / "hf-cache"))
    for sig in (signal.SIGINT, signal.SIGTERM, getattr(signal, "SIGUSR1", None)):
        if sig is not None:
            signal.signal(sig, request_stop)
    distributed = a.world_size > 1
    dist = None
    if a.stage != "prepare":
        import torch
        if a.device == "cuda":
            torch.cuda.set_device(a.local_rank)
            configure_memory(a)
        if distributed:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if a.device == "cuda":
                dist.init_process_group("nccl", device_id=torch.device("cuda", a.local_rank))
            else:
                dist.init_process_group("gloo")
    try:
        with contextlib.ExitStack() as stack:
            if a.rank == 0:
                stack.enter_context(process_lock(a.work_dir / "pipeline.lock"))
            if distributed:
                dist.barrier()
            if a.stage != "prepare":
                preflight(a)
            if a.stage in ("all", "prepare"):
                from ..data.prepare import prepare
                if not prepare(a, stop_requested=lambda: STOP):
                    return
            if a.stage in ("all", "train"):
                train(a)
    finally:
        if distributed:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
