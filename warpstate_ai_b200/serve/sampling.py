"""Next-token selection for the chat entry points.

Behaviour (what the reference probe does in chat.py:154-193, restated): a repetition penalty
pushes the score of every token already in the reply towards "less likely" (positive scores are
divided, negative ones multiplied); a no-repeat rule forbids the token that would complete an
n-gram the reply already contains; temperature 0 means arg-max; otherwise top-k (ties at the
cut kept) and nucleus filtering (the token that crosses the mass threshold is kept) precede one
multinomial draw over the candidates in descending order, from the caller's generator, so that a
seeded reply can be reproduced.  ``None`` means that nothing is left to choose from.

`Sampler` validates its settings once and is then called per token; `ReplyHistory` keeps the
reply's tokens together with an index from every (n-1)-gram to the tokens that followed it, so the
ban list is a dictionary lookup instead of a rescan of the reply.  `sample_token` and
`banned_ngram_tokens` are the stateless forms.
"""
from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class SamplingSettings:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    no_repeat_ngram: int = 0

    def __post_init__(self):
        problems = []
        if not (math.isfinite(self.temperature) and self.temperature >= 0):
            problems.append("temperature must be finite and >= 0")
        if self.top_k < 0:
            problems.append("top-k must be >= 0")
        if not 0 < self.top_p <= 1:
            problems.append("top-p must lie in (0, 1]")
        if not (math.isfinite(self.repetition_penalty) and self.repetition_penalty >= 1):
            problems.append("repetition penalty must be finite and >= 1")
        if not isinstance(self.no_repeat_ngram, int) or self.no_repeat_ngram < 0:
            problems.append("no-repeat n-gram size must be an integer >= 0")
        if problems:
            raise ValueError("Invalid sampling settings: " + "; ".join(problems))


class ReplyHistory:
    """Tokens of the reply so far, with the follower index the no-repeat rule needs."""

    def __init__(self, ngram: int = 0, tokens=()):
        self.ngram = int(ngram)
        self.tokens: list[int] = []
        self.distinct: set[int] = set()
        self._followers: dict[tuple, set] = defaultdict(set)
        for token in tokens:
            self.push(token)

    def push(self, token: int) -> None:
        self.tokens.append(int(token))
        self.distinct.add(int(token))
        n = self.ngram
        if n and len(self.tokens) >= n:
            self._followers[tuple(self.tokens[-n:-1])].add(self.tokens[-1])

    def blocked(self) -> set:
        """Tokens that would repeat an n-gram of the reply if they came next."""
        n = self.ngram
        if n == 0 or len(self.tokens) + 1 < n:
            return set()
        context = tuple(self.tokens[len(self.tokens) - (n - 1):]) if n > 1 else ()
        return set(self._followers.get(context, ()))


class Sampler:
    def __init__(self, settings: SamplingSettings, generator: torch.Generator | None = None):
        self.settings = settings
        self.generator = generator

    def pick(self, logits: torch.Tensor, seen=(), blocked=()) -> int | None:
        s = self.settings
        scores = logits.detach().to(torch.float32).clone()
        if bool(torch.isfinite(scores).logical_not().any()):
            raise ValueError("Non-finite generation logits")
        if s.repetition_penalty != 1 and len(seen):
            where = torch.tensor(sorted(set(seen)), dtype=torch.long)
            old = scores.index_select(0, where)
            scores[where] = torch.where(old >= 0, old / s.repetition_penalty, old * s.repetition_penalty)
        if len(blocked):
            scores[torch.tensor(sorted(blocked), dtype=torch.long)] = float("-inf")
        if not bool(torch.isfinite(scores).any()):
            return None
        if s.temperature == 0:
            return int(torch.argmax(scores))
        return self._draw(scores / s.temperature)

    def _draw(self, scores: torch.Tensor) -> int:
        s = self.settings
        order = torch.argsort(scores, descending=True, stable=True)
        ranked = scores[order]
        alive = torch.isfinite(ranked)
        if s.top_k:
            cut = ranked[min(s.top_k, ranked.numel()) - 1]
            alive &= ranked >= cut
        mass = torch.softmax(ranked.masked_fill(~alive, float("-inf")), dim=-1)
        alive &= (torch.cumsum(mass, dim=-1) - mass) <= s.top_p        # mass strictly before the token
        final = torch.softmax(ranked.masked_fill(~alive, float("-inf")), dim=-1)
        slot = torch.multinomial(final, 1, generator=self.generator)
        return int(order[slot])

    def next(self, logits: torch.Tensor, history: ReplyHistory) -> int | None:
        """Choose the next token given the reply so far (does not push it)."""
        return self.pick(logits, history.distinct, history.blocked())


# ----------------------------------------------------------------------------------- stateless forms
def banned_ngram_tokens(tokens, size: int) -> set:
    """Tokens that would complete an n-gram of length ``size`` already present in ``tokens``."""
    return ReplyHistory(size, tokens).blocked()


def sample_token(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, generator, *,
                 previous_tokens=(), repetition_penalty: float = 1.0, banned_tokens=()):
    settings = SamplingSettings(temperature=temperature, top_k=top_k, top_p=top_p,
                                repetition_penalty=repetition_penalty)
    return Sampler(settings, generator).pick(logits, previous_tokens, banned_tokens)
