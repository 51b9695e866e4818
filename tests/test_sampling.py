"""Next-token selection (`serve/sampling.py`): arg-max, seeded draws, repetition penalty, n-gram bans, filters.

The behaviour under test is the reference probe's (chat.py:154-193); the vectors are this file's own.
"""
import math

import pytest
import torch

from warpstate_ai_b200.serve.sampling import (ReplyHistory, Sampler, SamplingSettings, banned_ngram_tokens,
                                              sample_token)


def generator(seed):
    return torch.Generator().manual_seed(seed)


def test_arg_max_leaves_the_scores_alone_and_seeded_draws_repeat():
    logits = torch.tensor([-1.0, 0.3, 2.5, -30.0, 2.4])
    kept = logits.clone()
    assert sample_token(logits, 0.0, 0, 1.0, generator(1)) == 2

    def reply(seed):
        g = generator(seed)
        return [sample_token(logits, 0.9, 4, 0.95, g) for _ in range(20)]

    first = reply(7)
    assert first == reply(7)
    assert 3 not in first                      # outside the top four
    assert len(set(first)) > 1                 # and it is a draw, not the arg-max
    assert torch.equal(logits, kept)


def test_draws_come_from_the_callers_generator_only():
    state = torch.get_rng_state()
    g = generator(11)
    for _ in range(8):
        sample_token(torch.randn(16, generator=g), 1.0, 0, 1.0, g, previous_tokens=[1, 2], repetition_penalty=1.3)
    assert torch.equal(torch.get_rng_state(), state)


@pytest.mark.parametrize("bad", [float("nan"), float("inf"), float("-inf")])
def test_scores_that_are_not_finite_are_refused(bad):
    with pytest.raises(ValueError, match="Non-finite"):
        sample_token(torch.tensor([0.0, bad, 1.0]), 0.0, 0, 1.0, generator(0))


def test_repetition_penalty_pushes_both_signs_down_once_per_token():
    logits = torch.tensor([4.0, 3.0, -1.0, -1.5])
    # token 0 was seen three times: 4 / 2 = 2 < 3, so token 1 wins; had the penalty applied per occurrence the
    # score would be 0.5, had it applied to unseen tokens token 1 would have dropped too
    assert sample_token(logits, 0.0, 0, 1.0, generator(0), previous_tokens=[0, 0, 0], repetition_penalty=2.0) == 1
    only_negative = torch.tensor([-1.0, -1.5, -9.0])
    # -1 * 2 = -2 < -1.5: a negative score is multiplied, not divided
    assert sample_token(only_negative, 0.0, 0, 1.0, generator(0), previous_tokens=[0], repetition_penalty=2.0) == 1
    sampler = Sampler(SamplingSettings(repetition_penalty=1.5))
    assert sampler.pick(torch.tensor([3.0, 2.5]), seen=[0, 0]) == 1       # 3 / 1.5 = 2 < 2.5
    assert sampler.pick(torch.tensor([3.0, 1.9]), seen=[0, 0]) == 0       # applied once, not 3 / 2.25


@pytest.mark.parametrize("tokens, size, expected", [
    ([5, 6, 7, 5, 6], 3, {7}),
    ([5, 6, 7, 5, 6, 8, 5, 6], 3, {7, 8}),            # two earlier followers of (5, 6)
    ([4, 4, 4], 2, {4}),                              # overlapping matches
    ([4, 4, 4], 3, {4}),
    ([1, 2, 3], 1, {1, 2, 3}),                        # size one forbids every token of the reply
    ([1, 2], 3, set()),                               # too short to complete anything
    ([1, 2, 3, 4], 0, set()),                         # rule off
    ([9, 1, 2, 9, 3], 2, set()),                      # (3,) was never followed by anything
])
def test_ngram_ban_lists(tokens, size, expected):
    assert banned_ngram_tokens(tokens, size) == expected
    grown = ReplyHistory(size)
    for token in tokens:
        grown.push(token)
    assert grown.blocked() == expected
    assert grown.tokens == tokens and grown.distinct == set(tokens)


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_bans_apply_before_the_choice_and_running_out_is_none(temperature):
    logits = torch.tensor([5.0, 1.0, 0.5])
    settings = SamplingSettings(temperature=temperature, top_k=1)
    sampler = Sampler(settings, generator(3))
    assert sampler.pick(logits, blocked={0}) == 1        # the best token left, although top-k is one
    assert sampler.pick(logits, blocked={0, 1}) == 2
    assert sampler.pick(logits, blocked={0, 1, 2}) is None
    history = ReplyHistory(2, [0, 1, 0])
    assert history.blocked() == {1}
    assert sampler.next(torch.tensor([0.0, 9.0, 1.0]), history) == 2


def test_top_k_keeps_ties_and_the_nucleus_keeps_the_crossing_token():
    tied = torch.tensor([2.0, 2.0, 2.0, -4.0])
    seen = {Sampler(SamplingSettings(temperature=1.0, top_k=1), generator(s)).pick(tied) for s in range(40)}
    assert seen == {0, 1, 2}                              # all three share the cut; the fourth is out
    probs = torch.tensor([0.5, 0.3, 0.15, 0.05])
    logits = probs.log()
    # mass strictly before each token: 0, 0.5, 0.8, 0.95
    def support(top_p):
        return {Sampler(SamplingSettings(temperature=1.0, top_p=top_p), generator(s)).pick(logits) for s in range(200)}
    assert support(0.45) == {0}
    assert support(0.55) == {0, 1}                        # token 1 crosses 0.55 and is kept
    assert support(0.85) == {0, 1, 2}
    assert support(1.0) == {0, 1, 2, 3}


def test_draw_frequencies_follow_the_temperature():
    logits = torch.tensor([0.0, math.log(3.0)])
    g = generator(5)
    sampler = Sampler(SamplingSettings(temperature=1.0), g)
    ones = sum(sampler.pick(logits) for _ in range(4000))
    assert abs(ones / 4000 - 0.75) < 0.03
    cold = Sampler(SamplingSettings(temperature=0.5), g)        # p1 / p0 = 3 ** 2
    ones = sum(cold.pick(logits) for _ in range(4000))
    assert abs(ones / 4000 - 0.9) < 0.03


@pytest.mark.parametrize("bad", [dict(temperature=-0.1), dict(temperature=float("nan")), dict(top_k=-1), dict(top_p=0.0),
                                 dict(top_p=1.5), dict(repetition_penalty=0.9), dict(repetition_penalty=float("inf")),
                                 dict(no_repeat_ngram=-2), dict(no_repeat_ngram=1.5)])
def test_settings_are_checked_once_up_front(bad):
    with pytest.raises(ValueError, match="Invalid sampling settings"):
        SamplingSettings(**bad)
