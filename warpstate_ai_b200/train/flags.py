"""The pretraining command line as data.

Two tables:

* `RUN_FLAGS` -- everything that changes what this framework does: data, schedule, checkpointing,
  evaluation, memory cap, device, gradient path, sharding, activation checkpointing, residual dtype,
  gradient bucket size.  Names and defaults are the reference's where the reference has the flag
  (reference run_40b.py:25-110), so its launch scripts keep working.
* `REFERENCE_EXECUTION_FLAGS` -- switches of the reference's Inductor / Triton / compiled-autograd
  execution experiments (reference run_40b.py:57-93).  This framework has one native execution path that
  already does what each of them tried to buy, so they are accepted, stored in the resume signature (a
  reference checkpoint carries them, and `--reconfigure` compares them) and otherwise have no effect; a
  non-default value is reported once at start-up together with what the native path does instead.
  None of the reference's rules about which experiments may be combined applies here.

`build_parser` and `check` are generic over the tables.
"""
from __future__ import annotations

import argparse
import math
import os
from dataclasses import dataclass
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]


@dataclass(frozen=True)
class Flag:
    name: str                    # "--seq-len"
    kind: object = str           # int | float | str | Path | "switch" | "toggle"
    default: object = None
    rule: str = ""               # "" | ">=1" | "opt>=1" | ">0" | ">=0" | "opt>0"
    choices: tuple = ()
    help: str = ""
    native: str = ""             # reference-execution flags: what this framework does instead

    @property
    def dest(self) -> str:
        return self.name[2:].replace("-", "_")

    def add_to(self, parser) -> None:
        options = {"help": self.help or self.native or None}
        if self.kind == "switch":
            parser.add_argument(self.name, action="store_true", **options)
        elif self.kind == "toggle":
            parser.add_argument(self.name, action=argparse.BooleanOptionalAction, default=self.default, **options)
        else:
            if self.choices:
                options["choices"] = list(self.choices)
            parser.add_argument(self.name, type=self.kind, default=self.default, **options)

    def problem(self, value) -> str | None:
        optional = self.rule.startswith("opt")
        rule = self.rule[3:] if optional else self.rule
        if not rule or (optional and value is None):
            return None
        if not isinstance(value, (int, float)) or not math.isfinite(value):
            return f"{self.name} must be a finite number"
        ok = {">=1": value >= 1, ">0": value > 0, ">=0": value >= 0}[rule]
        return None if ok else f"{self.name} must be {rule.replace('>=', 'at least ').replace('>', 'greater than ')}"


RUN_FLAGS = (
    # initialisation and layout
    Flag("--work-dir", Path, ROOT / "work"), Flag("--tokenizer", Path, ROOT / "tokenizer.model"),
    Flag("--config", Path, ROOT / "configs/warpstate_2b.json"),
    Flag("--stage", str, "all", choices=("all", "prepare", "train")),
    Flag("--seed", int, 1337),
    # corpus
    Flag("--dataset", str, "HuggingFaceFW/fineweb-edu"), Flag("--dataset-config", str, "sample-100BT"),
    Flag("--revision", str, "main"), Flag("--verify-data", "switch", help="re-hash the token files against the manifest"),
    Flag("--train-tokens", int, 40_000_000_000, ">=1"), Flag("--val-tokens", int, 1_048_576, ">=1"),
    Flag("--workers", int, min(16, os.cpu_count() or 4), ">=1"), Flag("--documents-per-batch", int, 256, ">=1"),
    # objective and schedule
    Flag("--seq-len", int, 2048, ">=1"), Flag("--micro-batch", int, 8, ">=1"), Flag("--grad-accum", int, 8, ">=1"),
    Flag("--lr", float, 1.5e-4, ">0"), Flag("--min-lr", float, 1.5e-5, ">0"), Flag("--warmup-steps", int, 1000, ">=1"),
    Flag("--weight-decay", float, 0.1, ">=0"), Flag("--loss-chunk-size", int, 1024, ">=1"),
    # memory
    Flag("--activation-checkpointing", "toggle", True,
         help="keep only each core's input and recompute the core in its backward"),
    Flag("--bf16-residuals", "toggle", False, help="BF16 residual stream (FP32 by default)"),
    Flag("--vram-limit-gib", float, None, "opt>0"), Flag("--vram-headroom-gib", float, 3.0, ">=0"),
    # evaluation, checkpoints, pauses
    Flag("--eval-every", int, 500, ">=1"), Flag("--eval-batches", int, 8, ">=1"), Flag("--eval-micro-batch", int, 1, ">=1"),
    Flag("--save-every", int, 1000, ">=1"), Flag("--async-checkpoint", "toggle", False),
    Flag("--max-steps", int, None, "opt>=1"), Flag("--stop-at-step", int, None, "opt>=1"),
    Flag("--reconfigure", "switch", help="accept execution-only changes against the checkpoint's signature"),
    # environment
    Flag("--bootstrap", "switch", help="create a virtual environment with pinned dependencies and re-execute in it "
                                       "(needs network access; off by default)"),
    Flag("--no-bootstrap", "switch", help="never install anything (the default here; kept for the reference's scripts)"),
    Flag("--test-small-gpu", "switch", help="tests only: waive the 80 GiB device and 2 B parameter checks"),
    # this framework
    Flag("--device", str, "cuda", choices=("cuda", "cpu"), help="cpu runs the plain-PyTorch definition (tests)"),
    Flag("--kernels", "toggle", True, help="use the sm_100a kernel library on CUDA"),
    Flag("--grad-sync", str, "auto", choices=("auto", "fused", "nccl"),
         help="multi-GPU gradient path: in-kernel reduction over NVLink peer memory, or NCCL"),
    Flag("--shard-optimizer", "switch",
         help="multi-GPU: AdamW state for 1/world of every bucket per rank, updated weights broadcast from the update "
              "kernel (checkpoints stay unsharded)"),
    Flag("--shard-params", str, "off", choices=("off", "stream", "resident"),
         help="multi-GPU: parameters, gradients and optimizer state of the core projections sharded over the ranks; "
              "stream re-gathers BF16 weights for every use, resident once per update"),
    Flag("--ddp-bucket-cap-mb", float, 0.0, ">=0",
         help="largest gradient range reduced by one launch, in MiB of FP32 gradients: larger buckets are split, "
              "consecutive cores are merged up to it; 0 = one bucket per core"),
)

REFERENCE_EXECUTION_FLAGS = (
    Flag("--compile", "switch", native="no tracing compiler: every core is one autograd node over hand-written kernels"),
    Flag("--compile-core", "switch", native="no tracing compiler: every core is one autograd node over hand-written kernels"),
    Flag("--compile-mode", str, "default", choices=("default", "reduce-overhead", "max-autotune-no-cudagraphs"),
         native="kernel tile shapes are fixed at build time; bench/tune_gemm.py chooses between the two GEMM kernels"),
    Flag("--autocast-cache", "toggle", True, native="BF16 weights are a persistent mirror refreshed by the AdamW kernel"),
    Flag("--cache-core-weight-casts", "toggle", False,
         native="BF16 weights are a persistent mirror refreshed by the AdamW kernel"),
    Flag("--loss-mode", str, "checkpointed", choices=("checkpointed", "full", "compiled-full"),
         native="one fused LM-head cross-entropy that never materialises the logits"),
    Flag("--activation-mode", str, "baseline", choices=("baseline", "swiglu", "rmsnorm", "all"),
         native="SwiGLU lives in the up/gate GEMM epilogue, RMSNorm is one kernel with the depth modulation folded in"),
    Flag("--matmul-plan", Path, None, native="GEMMs are the tcgen05 kernels; a policy from bench/tune_gemm.py is loaded with "
                                             "ops.gemm.load_policy"),
    Flag("--gradient-mode", str, "eager", choices=("eager", "compiled-autograd", "compiled-autograd-overlap"),
         native="weight gradients accumulate in FP32 from the dW epilogue and buckets reduce under the remaining backward"),
    Flag("--backward-layout", str, "baseline", choices=("baseline", "inspect", "paired"),
         native="the attention backward kernel stores the packed [tokens, 5d] gradient directly"),
    Flag("--overlap-swap-collectives", "switch", native="bucket reductions are launched from the core-gradient hook"),
    Flag("--overlap-runtime-estimates", "switch", native="bucket reductions are launched from the core-gradient hook"),
    Flag("--overlap-producer-schedule", "switch", native="bucket reductions are launched from the core-gradient hook"),
    Flag("--overlap-memory-budget", float, 0.0, ">=0", native="bucket reductions are launched from the core-gradient hook"),
    Flag("--ddp-batched-grad-copy", "toggle", False,
         native="there is no gradient copy: the dW epilogue writes into the bucket that is reduced"),
)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="WarpState pretraining on B200 (prepare + train)")
    start = parser.add_mutually_exclusive_group()
    start.add_argument("--weights", type=Path, help="a trusted WarpState checkpoint that initialises a new run")
    start.add_argument("--from-scratch", action="store_true", help="initialise a new model from --config and --seed")
    for flag in RUN_FLAGS:
        flag.add_to(parser)
    compat = parser.add_argument_group(
        "reference execution experiments", "accepted and recorded in the resume signature; no effect on what runs here")
    for flag in REFERENCE_EXECUTION_FLAGS:
        flag.add_to(compat)
    return parser


def check(parser: argparse.ArgumentParser, a) -> None:
    for flag in RUN_FLAGS + REFERENCE_EXECUTION_FLAGS:
        complaint = flag.problem(getattr(a, flag.dest))
        if complaint:
            parser.error(complaint)
    if a.min_lr > a.lr:
        parser.error("--min-lr must not exceed --lr")
    if a.train_tokens < 2:
        parser.error("--train-tokens must be at least 2")
    if a.val_tokens <= a.seq_len:
        parser.error("--val-tokens must exceed --seq-len (one evaluation window)")
    if a.shard_params != "off" and a.shard_optimizer:
        parser.error("--shard-params already shards the optimizer state; drop --shard-optimizer")
    if a.bootstrap and a.no_bootstrap:
        parser.error("choose --bootstrap or --no-bootstrap")


def inert_settings(a) -> list[tuple[str, object, str]]:
    """(flag, value, what the native path does instead) for every reference-execution flag that was changed."""
    return [(flag.name, getattr(a, flag.dest), flag.native) for flag in REFERENCE_EXECUTION_FLAGS
            if getattr(a, flag.dest) != (False if flag.kind == "switch" else flag.default)]
