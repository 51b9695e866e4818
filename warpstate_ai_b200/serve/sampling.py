"""Token sampling: repetition penalty -> banned n-grams -> greedy / top-k / top-p.

Semantics follow the reference probe (chat.py:154-193): the penalty lowers both positive and
negative scores of tokens already generated in this reply; an n-gram ban blocks the token that
would complete an n-gram already present in the reply; ``temperature == 0`` is greedy; top-p
keeps the token that crosses the cumulative threshold; ``None`` is returned when every token is
masked.  Sampling uses the caller's generator so that replies are reproducible.
"""
from __future__ import annotations

import math

import torch


def banned_ngram_tokens(tokens, size: int) -> set:
    """Tokens that would complete an n-gram of length ``size`` already present in ``tokens``."""
    if size == 0 or len(tokens) + 1 < size:
        return set()
    prefix = tuple(tokens[-(size - 1):]) if size > 1 else ()
    return {tokens[i + size - 1] for i in range(len(tokens) - size + 1)
            if tuple(tokens[i:i + size - 1]) == prefix}


def sample_token(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, generator, *,
                 previous_tokens=(), repetition_penalty: float = 1.0, banned_tokens=()):
    logits = logits.float().clone()
    if not torch.isfinite(logits).all():
        raise ValueError("Non-finite generation logits")
    if not math.isfinite(temperature) or temperature < 0 or not 0 < top_p <= 1 or top_k < 0:
        raise ValueError("Invalid sampling settings")
    if not math.isfinite(repetition_penalty) or repetition_penalty < 1:
        raise ValueError("Require a finite repetition-penalty >= 1")
    if previous_tokens and repetition_penalty != 1:
        seen = list(set(previous_tokens))
        scores = logits[seen]
        logits[seen] = torch.where(scores < 0, scores * repetition_penalty, scores / repetition_penalty)
    if banned_tokens:
        logits[list(banned_tokens)] = -torch.inf
    if not torch.isfinite(logits).any():
        return None
    if temperature == 0:
        return int(logits.argmax())
    values = logits / temperature
    if top_k:
        threshold = values.topk(min(top_k, values.numel())).values[-1]
        values = values.masked_fill(values < threshold, -torch.inf)
    ordered, indices = values.sort(descending=True)
    probability = ordered.softmax(dim=-1)
    ordered = ordered.masked_fill(probability.cumsum(-1) - probability > top_p, -torch.inf)
    picked = torch.multinomial(ordered.softmax(dim=-1), 1, generator=generator)
    return int(indices[picked].item())
