"""Chunk attention + memory kernels against the plain-PyTorch composite (FP32 oracle)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def make_core(h=4, parallel=True):
    from warpstate_ai_b200 import WarpStateConfig
    from warpstate_ai_b200.models.warpstate import WarpStateCore
    cfg = WarpStateConfig(vocab_size=64, d_model=64 * h, n_heads=h, n_cores=1, logical_depth=1, ffn_hidden=128,
                          chunk_size=128, gradient_checkpointing=False, parallel_memory=parallel)
    core = WarpStateCore(cfg).cuda()
    with torch.no_grad():
        core.fast_decay_logit.add_(torch.randn(h, device="cuda") * 0.3)
        core.slow_decay_logit.add_(torch.randn(h, device="cuda") * 0.3)
        core.memory_mix_logit.add_(torch.randn(h, device="cuda") * 0.5)
    return core


@pytest.mark.parametrize("batch,seq,h", [(1, 128, 1), (2, 512, 4), (3, 2048, 8)])
def test_forward_matches_composite(batch, seq, h):
    from warpstate_ai_b200.ops import attention, reference as R
    from warpstate_ai_b200.ops.gemm import check_device_errors
    torch.manual_seed(0)
    core = make_core(h)
    d = 64 * h
    qkvgu = (torch.randn(batch * seq, 5 * d, device="cuda") * 1.5).bfloat16()
    y, writes, states, (ff, fs) = attention.forward_only(qkvgu, core, batch, seq, want_final=True)
    check_device_errors()
    x32 = qkvgu.float().view(batch, seq, 5 * d)
    ref, (rf, rs) = R.attention_memory(x32, core.fast_decay_logit, core.slow_decay_logit, core.memory_mix_logit,
                                       h, 128, True, core.rope_cos, core.rope_sin, return_state=True)
    # writes
    q, k, v, g, u = x32.chunk(5, dim=-1)
    def chunked(t):
        return t.reshape(batch, seq // 128, 128, h, 64).permute(0, 1, 3, 2, 4)
    kr = R.apply_rope(chunked(k), core.rope_cos.view(1, 1, 1, 128, 64), core.rope_sin.view(1, 1, 1, 128, 64))
    ref_w = R.chunk_writes(kr, chunked(u), 128)
    assert rel_l2(writes, ref_w) < 0.01
    assert rel_l2(ff, rf) < 0.01 and rel_l2(fs, rs) < 0.01
    assert rel_l2(y, ref.reshape(batch * seq, d)) < 0.01


# 17 chunks: two groups of the reverse scan, the second with one chunk; 70 chunks: beyond the 64 of the
# earlier register-array kernel, five groups, the last one partial
@pytest.mark.parametrize("batch,seq,h", [(1, 128, 1), (2, 512, 4), (2, 2048, 8), (2, 128 * 17, 2), (1, 128 * 70, 1)])
def test_backward_matches_autograd_of_composite(batch, seq, h):
    from warpstate_ai_b200.ops import attention, reference as R
    from warpstate_ai_b200.ops.gemm import check_device_errors
    torch.manual_seed(1)
    core = make_core(h)
    d = 64 * h
    qkvgu = (torch.randn(batch * seq, 5 * d, device="cuda") * 1.5).bfloat16()
    dy = torch.randn(batch * seq, d, device="cuda").bfloat16()
    y, saved = attention.forward(qkvgu, core, batch, seq)
    dq, g_fast, g_slow, g_mix = attention.backward(dy, qkvgu, saved, core, batch, seq)
    check_device_errors()
    leaf = qkvgu.float().view(batch, seq, 5 * d).requires_grad_(True)
    ref = R.attention_memory(leaf, core.fast_decay_logit, core.slow_decay_logit, core.memory_mix_logit,
                             h, 128, True, core.rope_cos, core.rope_sin)
    grads = torch.autograd.grad(ref, [leaf, core.fast_decay_logit, core.slow_decay_logit, core.memory_mix_logit],
                                dy.float().view(batch, seq, d))
    want = grads[0].reshape(batch * seq, 5 * d)
    names = ["dQ", "dK", "dV", "dGate", "dU"]
    for i, name in enumerate(names):
        err = rel_l2(dq[:, i * d:(i + 1) * d], want[:, i * d:(i + 1) * d])
        assert err < 0.02, (name, err)
    if seq > 128:  # with a single chunk nothing reads the memory: these gradients are exactly zero
        assert rel_l2(g_fast, grads[1]) < 0.03, ("fast", g_fast, grads[1])
        assert rel_l2(g_slow, grads[2]) < 0.03, ("slow", g_slow, grads[2])
        assert rel_l2(g_mix, grads[3]) < 0.03, ("mix", g_mix, grads[3])
    else:
        assert float(g_fast.abs().max()) == 0.0 and float(g_mix.abs().max()) == 0.0


@pytest.mark.parametrize("batch,seq,h", [(1, 128, 1), (2, 640, 4), (4, 2048, 32)])
def test_streaming_tile_kernels_equal_the_one_tile_per_cta_kernels(batch, seq, h):
    """The persistent, warp-specialised form of the chunk-writes kernel (TMA ring, worker warps, MMA issue, epilogue
    warps with a double-buffered accumulator) against the one-tile-per-CTA form: the same arithmetic in the same
    order, so the results must be equal bit for bit -- fewer tiles than SMs, a ragged last round, and the
    production count (2048 tiles on 148 SMs)."""
    from warpstate_ai_b200.ops import _ext, attention
    from warpstate_ai_b200.ops.gemm import check_device_errors, error_flag
    ops = torch.ops.ws_b200
    lib = _ext.cdll()
    torch.manual_seed(5)
    d = 64 * h
    qkvgu = (torch.randn(batch * seq, 5 * d, device="cuda") * 1.5).bfloat16()
    rope = attention.rope_table(qkvgu.device, pair_major=True)
    try:
        lib.ws_attn_set_stream_mode(0)
        tile_form = ops.chunk_writes(qkvgu, rope, batch, seq, h, error_flag(qkvgu.device))
        lib.ws_attn_set_stream_mode(1)
        stream_form = ops.chunk_writes(qkvgu, rope, batch, seq, h, error_flag(qkvgu.device))
        again = ops.chunk_writes(qkvgu, rope, batch, seq, h, error_flag(qkvgu.device))
    finally:
        lib.ws_attn_set_stream_mode(-1)
    check_device_errors()
    assert torch.equal(stream_form, tile_form) and torch.equal(again, tile_form)
    assert float(tile_form.abs().max()) > 0
    # the state-gradient kernel has the same two forms; it feeds the reverse scan and the backward kernel, so the
    # packed gradient and the decay / mix gradients of the whole backward must be equal bit for bit as well
    core = make_core(h)
    dy = torch.randn(batch * seq, d, device="cuda").bfloat16()
    results = {}
    try:
        for mode in (0, 1):
            lib.ws_attn_set_stream_mode(mode)
            y, saved = attention.forward(qkvgu, core, batch, seq)
            results[mode] = (y, *attention.backward(dy, qkvgu, saved, core, batch, seq))
    finally:
        lib.ws_attn_set_stream_mode(-1)
    check_device_errors()
    for mine, theirs in zip(results[1], results[0]):
        assert torch.equal(mine, theirs)
