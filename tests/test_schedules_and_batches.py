"""Learning-rate schedules of the three stages and the token-stream batching contracts.

Contracts restated from the reference: run_40b.py:729-733 (warm-up then cosine), posttrain.py:192-197 and dpo.py:92-98
(ratio warm-up, cosine resp. linear decay), run_40b.py:347-358 (cyclic window, labels masked past ``valid``) and
run_40b.py:423-427 (disjoint per-rank slices of an update, empty ones included).
"""
import math

import numpy as np
import pytest
import torch

from warpstate_ai_b200.data.tokens import HostBatcher, SyntheticTokens, batches, host_batch, update_slices, window
from warpstate_ai_b200.optim.adamw import cosine_lr
from warpstate_ai_b200.train import dpo, sft
from warpstate_ai_b200.train.stage import schedule_position, warmup_steps


# ------------------------------------------------------------------------------------------- schedules
def test_pretraining_rate_warms_up_linearly_then_follows_a_cosine():
    kw = dict(lr=2e-4, min_lr=2e-5, warmup_steps=10, total_steps=110)
    rates = [cosine_lr(step, **kw) for step in range(110)]
    assert rates[0] == pytest.approx(2e-5) and rates[4] == pytest.approx(1e-4) and rates[9] == pytest.approx(2e-4)
    assert rates[10] == pytest.approx(2e-4)                                     # the cosine starts at the peak
    assert rates[60] == pytest.approx(0.5 * (2e-4 + 2e-5))                      # and is half-way down in the middle
    assert all(a > b for a, b in zip(rates[10:], rates[11:]))
    assert cosine_lr(110, **kw) == pytest.approx(2e-5)
    # a run shorter than the warm-up never leaves it, and never divides by zero
    short = [cosine_lr(step, lr=1.0, min_lr=0.1, warmup_steps=1000, total_steps=4) for step in range(4)]
    assert short == pytest.approx([0.25, 0.5, 0.75, 1.0])


@pytest.mark.parametrize("total, ratio, warm", [(100, 0.03, 3), (100, 0.1, 10), (7, 0.5, 4), (1, 0.5, 0), (2, 1.0, 1), (50, 0.0, 0)])
def test_ratio_warm_up_leaves_at_least_one_decay_step(total, ratio, warm):
    assert warmup_steps(total, ratio) == warm
    assert schedule_position(total - 1, total, ratio)[0] == "decay"
    if warm:
        assert schedule_position(warm - 1, total, ratio) == ("warmup", warm)
    phase, x = schedule_position(warm, total, ratio)
    assert phase == "decay" and x == 0.0
    assert schedule_position(total - 1, total, ratio)[1] == (1.0 if total - warm > 1 else 0.0)


@pytest.mark.parametrize("stage, shape", [(sft, "cosine"), (dpo, "linear")])
def test_post_training_rates_reach_the_floor_on_the_last_step(stage, shape):
    s = {"lr": 1e-5, "min_lr": 1e-6, "warmup_ratio": 0.1}
    total = 41
    rates = [stage.learning_rate(step, total, s) for step in range(total)]
    warm = warmup_steps(total, 0.1)
    assert warm == 5
    assert rates[:warm] == pytest.approx([1e-5 * (i + 1) / warm for i in range(warm)])
    assert rates[warm] == pytest.approx(1e-5) and rates[-1] == pytest.approx(1e-6)
    assert all(a > b for a, b in zip(rates[warm:], rates[warm + 1:]))
    middle = rates[warm + (total - warm - 1) // 2]
    halfway = 0.5 * (1e-5 + 1e-6)
    assert middle == pytest.approx(halfway, rel=0.08)
    quarter = rates[warm + (total - warm - 1) // 4]
    if shape == "cosine":
        assert quarter > 1e-6 + 0.75 * 9e-6 + 1e-7          # a cosine stays above the straight line early on
    else:
        assert quarter == pytest.approx(1e-6 + 0.75 * 9e-6, rel=0.05)
    # the rate is a function of the step alone
    assert stage.learning_rate(17, total, s) == rates[17]


# ------------------------------------------------------------------------------------------- token windows
def test_window_wraps_around_the_end_of_the_stream():
    data = np.arange(10, dtype=np.uint16)
    assert window(data, 3, 4).tolist() == [3, 4, 5, 6]
    assert window(data, 8, 5).tolist() == [8, 9, 0, 1, 2]
    assert window(data, 23, 3).tolist() == [3, 4, 5]               # the cursor itself may be many laps in
    assert window(data, 0, 25).tolist() == [i % 10 for i in range(25)]
    assert window(data, 9, 1).dtype == np.int64


def test_labels_are_inputs_shifted_by_one_and_masked_past_valid():
    data = np.arange(100, 120, dtype=np.uint16)
    x, y = host_batch(data, 17, 2, 4, valid=5)
    assert x.tolist() == [[117, 118, 119, 100], [101, 102, 103, 104]]
    assert y.tolist() == [[118, 119, 100, 101], [102, -100, -100, -100]]
    x0, y0 = host_batch(data, 17, 2, 4, valid=0)                   # a rank with nothing to score still gets a batch
    assert torch.equal(x0, x) and bool((y0 == -100).all())
    bx, by = batches(data, 17, 2, 4, 8, torch.device("cpu"))
    assert torch.equal(bx, x) and by.tolist() == [[118, 119, 100, 101], [102, 103, 104, 105]]
    assert bx.dtype == torch.int64 and by.dtype == torch.int64


@pytest.mark.parametrize("world", [1, 2, 3, 5])
@pytest.mark.parametrize("target, micro", [(73, 32), (64, 32), (9, 32), (1, 8), (1000, 24), (96, 32)])
def test_update_slices_tile_the_update_exactly_once(world, target, micro):
    per_rank = [list(update_slices(target, micro, world, rank)) for rank in range(world)]
    iterations = {len(slices) for slices in per_rank}
    assert iterations == {math.ceil(target / (world * micro))}     # every rank runs the same number of micro-steps
    covered = np.zeros(target + world * micro, dtype=np.int64)
    for slices in per_rank:
        for offset, valid in slices:
            assert 0 <= valid <= micro
            covered[offset:offset + valid] += 1
    assert covered[:target].tolist() == [1] * target and not covered[target:].any()
    # offsets advance rank-major inside an iteration, so a rank's slices never depend on the others' validity
    for rank, slices in enumerate(per_rank):
        assert [offset for offset, _ in slices] == [(i * world + rank) * micro for i in range(len(slices))]


def test_the_73_token_fixture_ends_with_an_empty_rank():
    # updates of 32, 32 and 9 tokens on two ranks with 16-token micro-batches: the last update leaves rank 1 idle
    last = [list(update_slices(9, 16, 2, rank)) for rank in range(2)]
    assert last == [[(0, 9)], [(16, 0)]]


def test_synthetic_stream_is_reproducible_and_in_range():
    a, b, c = SyntheticTokens(4096, 32768, seed=3), SyntheticTokens(4096, 32768, seed=3), SyntheticTokens(4096, 32768, seed=4)
    assert len(a) == 4096 and a.array.dtype == np.uint16
    assert np.array_equal(a[:], b[:]) and not np.array_equal(a[:], c[:])
    assert int(a[:].max()) < 32768 and len(np.unique(a[:])) > 3000
    assert SyntheticTokens(16, 100000).array.dtype == np.int32
    assert window(a, 4090, 10).tolist() == [int(t) for t in list(a[4090:]) + list(a[:4])]


def test_host_batcher_on_cpu_is_the_plain_batch():
    data = SyntheticTokens(500, 1000, seed=1)
    batcher = HostBatcher(2, 16, torch.device("cpu"))
    handle = batcher.stage(data, 490, valid=20)
    x, y = batcher.take(handle)
    batcher.release(handle)
    ex, ey = host_batch(data, 490, 2, 16, 20)
    assert torch.equal(x, ex) and torch.equal(y, ey)
    assert batcher.bytes_per_batch == 2 * 2 * 16 * 8
