"""Where a pretraining run starts from, and what the machine must offer before it starts.

Three ways to begin (the reference's rules, reference run_40b.py:459-520, 805-840): resume from the run's own
``run/latest.pt`` (a ``warpstate-server-v1`` checkpoint); initialise a new run from ``--weights`` (any WarpState
checkpoint with a model state dict, including the legacy CPU-offload layout whose unrounded FP32 masters are
preferred over its model tensors); or ``--from-scratch`` from ``--config`` and ``--seed``.  `StartPoint`
resolves that once; the preflight check and the run's set-up both read it, so they cannot disagree.

`require_device` and `cap_device_memory` are the hardware side: BF16-capable CUDA device of at least 80 GiB
for the normal preset, and an optional hard cap on the caching allocator (with headroom for what lives outside
it) installed before anything is allocated, for GPUs shared with other jobs.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path

GIB = 1 << 30
FULL_SIZE = range(2_000_000_000, 2_020_000_001)      # parameter count of the architecture this package trains


@dataclass
class StartPoint:
    kind: str                      # "resume" | "weights" | "scratch"
    source: Path | None
    checkpoint: dict = field(repr=False, default_factory=dict)

    @classmethod
    def resolve(cls, a) -> "StartPoint":
        from ..ckpt.formats import SERVER_FORMAT, load_checkpoint
        latest = a.work_dir / "run/latest.pt"
        if latest.exists():
            checkpoint = load_checkpoint(latest)
            if checkpoint.get("format") != SERVER_FORMAT:
                raise ValueError(f"{latest} is not a {SERVER_FORMAT} checkpoint; start a new run with --weights "
                                 "in another work directory")
            return cls("resume", latest, checkpoint)
        if a.from_scratch:
            return cls("scratch", None)
        if a.weights is None or not a.weights.is_file():
            raise ValueError("the first launch of a run needs --weights <checkpoint.pt> (or --from-scratch)")
        checkpoint = load_checkpoint(a.weights)
        if "model" not in checkpoint:
            raise ValueError(f"{a.weights} holds no WarpState model state dict")
        return cls("weights", a.weights, checkpoint)

    def config(self, a):
        """The model configuration: the checkpoint's, or ``--config`` when it has none / for a fresh model."""
        from ..config import WarpStateConfig
        values = self.checkpoint.get("config")
        if values is None:
            values = json.loads(a.config.read_text())
        cfg = WarpStateConfig(**values)
        cfg.validate()
        return cfg

    def legacy_masters(self):
        """FP32 master tensors of a legacy CPU-offload optimizer state (only when initialising from weights)."""
        state = self.checkpoint.get("optimizer", {})
        if self.kind == "weights" and state.get("kind") == "cpu_offload_adamw":
            return state["masters"]
        return None

    def build_model(self, cfg, seed: int):
        """FP32 model on the CPU/meta side, filled from the checkpoint (or freshly initialised)."""
        import torch
        from ..models.warpstate import WarpStateLM
        if self.kind == "scratch":
            print(f"Initialising fresh FP32 weights from seed {seed}.", flush=True)
            return WarpStateLM(cfg)
        with torch.device("meta"):
            model = WarpStateLM(cfg)
        model.load_state_dict(self.checkpoint["model"], assign=True)
        return model


def check_fit(cfg, a) -> None:
    """Model against tokenizer and sequence length."""
    import sentencepiece as spm
    vocabulary = spm.SentencePieceProcessor(model_file=str(a.tokenizer)).vocab_size()
    if cfg.vocab_size != vocabulary:
        raise ValueError(f"the model has {cfg.vocab_size} vocabulary rows, the tokenizer {vocabulary}: use the tokenizer "
                         "the weights were trained with")
    if a.seq_len % cfg.chunk_size:
        raise ValueError(f"--seq-len {a.seq_len} is not a multiple of the model's chunk size {cfg.chunk_size}")


def require_device(a):
    """The training device and its (name, bytes); raises when the machine cannot run the preset."""
    import torch
    if a.device != "cuda":
        return torch.device("cpu"), "cpu", 0
    if not torch.cuda.is_available() or not torch.cuda.is_bf16_supported():
        raise RuntimeError("a CUDA GPU with BF16 support is required (or --device cpu for tests)")
    device = torch.device("cuda", a.local_rank)
    properties = torch.cuda.get_device_properties(device)
    if properties.total_memory < 80 * GIB and not a.test_small_gpu:
        raise RuntimeError(f"{properties.name} has {properties.total_memory / GIB:.0f} GiB; the training preset needs "
                           "80 GiB or more")
    return device, properties.name, properties.total_memory


def cap_device_memory(a) -> None:
    """``--vram-limit-gib``: hard cap of this process's caching allocator (reference run_40b.py:442-456)."""
    if a.device != "cuda" or a.vram_limit_gib is None:
        return
    import torch
    device = torch.device("cuda", a.local_rank)
    free, total = torch.cuda.mem_get_info(device)
    cap = int(a.vram_limit_gib * GIB)
    needed = cap + int(a.vram_headroom_gib * GIB)
    if cap > total or needed > free:
        raise RuntimeError(f"the allocator cap plus headroom needs {needed / GIB:.2f} GiB but the device has "
                           f"{free / GIB:.2f} GiB free of {total / GIB:.2f}")
    torch.cuda.set_per_process_memory_fraction(cap / total, device)
    print(f"CUDA allocator capped at {a.vram_limit_gib:.2f} GiB ({free / GIB:.2f} GiB were free).", flush=True)


def preflight(a) -> None:
    """Reject weights, tokenizer or hardware that cannot work -- before a long preparation or run."""
    import torch
    from ..models.warpstate import WarpStateLM
    require_device(a)
    start = StartPoint.resolve(a)
    cfg = start.config(a)
    check_fit(cfg, a)
    with torch.device("meta"):
        probe = WarpStateLM(cfg)
    if start.kind != "scratch":
        probe.load_state_dict(start.checkpoint["model"], assign=True, strict=True)
    count = probe.num_parameters()
    if count not in FULL_SIZE and not a.test_small_gpu:
        raise ValueError(f"{count:,} parameters: this package trains the ~2.005 B WarpState architecture")
    masters = start.legacy_masters()
    if masters is not None:
        shapes = [tuple(p.shape) for p in probe.parameters()]
        if len(masters) != len(shapes) or any(tuple(m.shape) != s for m, s in zip(masters, shapes)):
            raise ValueError("the FP32 masters of the legacy optimizer state do not match the model's parameters")
    described = {"scratch": "configuration for a fresh model", "weights": "initial weights", "resume": "checkpoint"}
    print(f"Preflight: usable {described[start.kind]} ({count:,} parameters).", flush=True)
