"""Post-training plan files as declarative schemas.

A plan is a JSON document ``{"format": ..., "stage": ..., "training": {...}, ...}``; its ``training``
section overrides the defaults of the stage.  The plan formats and every key and default below are the
reference's (reference posttrain.py:34-97 for ``warpstate-posttrain-plan-v1``, reference dpo.py:38-80
for ``warpstate-dpo-plan-v1``); they are data here, not code: one `Setting` per key with a kind that
knows how to check a value, plus the few relations between keys.

``reference_mode`` is this framework's addition to the DPO plan (score the frozen reference from a cache,
or keep it resident on the GPU).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path


def _is_number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(v)


KINDS = {
    "count": (lambda v, s: type(v) is int and v >= 1, "a positive integer"),
    "optional_count": (lambda v, s: v is None or (type(v) is int and v >= 1), "null or a positive integer"),
    "amount": (lambda v, s: _is_number(v) and v >= 0, "a finite number >= 0"),
    "positive": (lambda v, s: _is_number(v) and v > 0, "a finite number > 0"),
    "ratio": (lambda v, s: _is_number(v) and 0 <= v < 1, "a number in [0, 1)"),
    "flag": (lambda v, s: type(v) is bool, "true or false"),
    "seed": (lambda v, s: type(v) is int and v >= 0, "an integer >= 0"),
    "choice": (lambda v, s: v in s.choices, "one of the listed choices"),
}


@dataclass(frozen=True)
class Setting:
    name: str
    default: object
    kind: str
    choices: tuple = ()

    def check(self, value) -> None:
        accepts, wording = KINDS[self.kind]
        if not accepts(value, self):
            extra = f" {list(self.choices)}" if self.choices else ""
            raise ValueError(f"training.{self.name} must be {wording}{extra}; got {value!r}")


@dataclass(frozen=True)
class Relation:
    holds: object      # callable(settings) -> bool
    message: str


class PlanSchema:
    def __init__(self, plan_format: str, stage: str, settings: tuple, relations: tuple = ()):
        self.plan_format, self.stage, self.settings, self.relations = plan_format, stage, settings, relations

    @property
    def defaults(self) -> dict:
        return {s.name: s.default for s in self.settings}

    def resolve(self, plan: dict) -> dict:
        """The effective settings of a parsed plan (defaults overridden by its ``training`` section)."""
        if plan.get("format") != self.plan_format or plan.get("stage") != self.stage:
            raise ValueError(f"expected a {self.plan_format} plan for stage '{self.stage}'")
        given = plan.get("training", {})
        known = {s.name for s in self.settings}
        strangers = sorted(set(given) - known)
        if strangers:
            raise ValueError(f"unknown training settings in the plan: {strangers}")
        merged = {**self.defaults, **given}
        for setting in self.settings:
            setting.check(merged[setting.name])
        for relation in self.relations:
            if not relation.holds(merged):
                raise ValueError(relation.message)
        return merged

    def read(self, path):
        plan = json.loads(Path(path).read_text())
        return plan, self.resolve(plan)


_COMMON = (
    Setting("sequence_length", 2048, "count"), Setting("epochs", 1, "count"), Setting("max_steps", None, "optional_count"),
    Setting("weight_decay", 0.0, "amount"), Setting("seed", 42, "seed"), Setting("eval_every", 100, "count"),
    Setting("save_every", 100, "count"), Setting("eval_batches", 32, "count"), Setting("compile_core", True, "flag"),
    Setting("bf16_residuals", True, "flag"), Setting("gradient_checkpointing", False, "flag"),
    Setting("workers", 4, "count"), Setting("deterministic", True, "flag"), Setting("clip_grad_norm", 1.0, "positive"),
    Setting("min_lr", 0.0, "amount"),
)
_LR_ORDER = Relation(lambda s: s["min_lr"] <= s["lr"], "training.min_lr must not exceed training.lr")

SFT_PLAN = PlanSchema("warpstate-posttrain-plan-v1", "sft", _COMMON + (
    Setting("micro_batch", 4, "count"), Setting("grad_accum", 4, "count"), Setting("lr", 5e-6, "positive"),
    Setting("warmup_ratio", 0.03, "ratio"),
    Setting("loss_mode", "compiled-full", "choice", ("full", "compiled-full", "checkpointed")),
), (_LR_ORDER,))

DPO_PLAN = PlanSchema("warpstate-dpo-plan-v1", "dpo", _COMMON + (
    Setting("micro_batch", 2, "count"), Setting("grad_accum", 8, "count"), Setting("lr", 5e-7, "positive"),
    Setting("warmup_ratio", 0.1, "ratio"), Setting("beta", 5.0, "positive"),
    Setting("objective", "length-normalized-dpo", "choice", ("length-normalized-dpo", "summed-dpo")),
    Setting("head_chunk_size", 256, "count"), Setting("reference_mode", "cached", "choice", ("cached", "resident")),
), (_LR_ORDER,))
