"""Declarative consistency checks: a check is a list of `Rule`s (message, predicate); `enforce` raises the message
of the first one that does not hold.  The pipeline's guardians and archives state what must be true of a
checkpoint, a report or a directory as such tables instead of ladders of ``if ...: raise``."""
from __future__ import annotations

import math
from typing import Callable, NamedTuple

import torch


class Rule(NamedTuple):
    message: str
    holds: Callable[[], bool]


def enforce(rules, error=ValueError) -> None:
    """A rule that cannot even be evaluated (a missing key, a ``None`` where a mapping was expected) does not hold."""
    for rule in rules:
        try:
            fine = bool(rule.holds())
        except (KeyError, TypeError, AttributeError):
            fine = False
        if not fine:
            raise error(rule.message)


def finite(value) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)


def matches(record, wanted: dict) -> bool:
    """``record`` carries every key of ``wanted`` with exactly that value."""
    return all(key in record and record[key] == value for key, value in wanted.items())


def fp32_tensors(tensors: dict, message: str) -> list:
    """One rule per floating-point tensor: it must still be FP32.  ``message`` is formatted with name and dtype."""
    return [Rule(message.format(name=name, dtype=tensor.dtype),
                 lambda t=tensor: not t.is_floating_point() or t.dtype == torch.float32) for name, tensor in tensors.items()]
