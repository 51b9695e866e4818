"""Decode engine: batched chunked prefill + step equals the full forward (reference bar for
decode-vs-forward in FP32: rtol 2e-5 / atol 2e-6, test_chat.py:48-57; cached decoder in BF16:
rtol = atol = 0.025, test_posttrain_chat.py:100), and the sampling rules."""
import pytest
import torch

from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
from warpstate_ai_b200.serve.engine import DecodeEngine
from warpstate_ai_b200.serve.sampling import banned_ngram_tokens, sample_token


def tiny(parallel=True, chunk=8):
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=97, d_model=32, n_heads=4, n_cores=2, logical_depth=4, ffn_hidden=48,
                          chunk_size=chunk, gradient_checkpointing=False, parallel_memory=parallel)
    model = WarpStateLM(cfg).eval()
    with torch.no_grad():
        model.depth_scale.normal_(0, 0.1)
        model.depth_bias.normal_(0, 0.1)
    return model


@pytest.mark.parametrize("parallel", [True, False])
@pytest.mark.parametrize("prompt", [3, 8, 19, 24])
def test_prefill_and_steps_match_full_forward(parallel, prompt):
    model = tiny(parallel)
    total = 40
    ids = torch.randint(0, 97, (3, total))
    with torch.no_grad():
        full = model(ids)  # [B, T, V]
    engine = DecodeEngine(model, dtype=torch.float32, use_cuda_graph=False)
    logits = engine.prefill(ids[:, :prompt])
    assert torch.allclose(logits, full[:, prompt - 1], rtol=2e-5, atol=2e-5)
    for t in range(prompt, total):
        logits = engine.step(ids[:, t])
        assert torch.allclose(logits, full[:, t], rtol=2e-5, atol=2e-5), t


def test_sampling_rules():
    g = torch.Generator().manual_seed(0)
    logits = torch.tensor([1.0, 3.0, 2.0, -1.0])
    assert sample_token(logits, 0.0, 0, 1.0, g) == 1
    assert sample_token(logits, 0.0, 0, 1.0, g, banned_tokens={1}) == 2
    assert sample_token(logits, 0.0, 0, 1.0, g, previous_tokens=[1], repetition_penalty=2.0) == 2
    assert sample_token(logits, 1.0, 1, 1.0, g) == 1            # top-k = 1 is greedy
    assert sample_token(logits, 1.0, 0, 1e-6, g) == 1           # tiny top-p keeps only the best token
    assert sample_token(torch.tensor([0.0, 0.0]), 0.0, 0, 1.0, g, banned_tokens={0, 1}) is None
    with pytest.raises(ValueError):
        sample_token(logits, -1.0, 0, 1.0, g)
    with pytest.raises(ValueError):
        sample_token(torch.tensor([float("nan")]), 0.0, 0, 1.0, g)
    assert banned_ngram_tokens([1, 2, 3, 1, 2], 3) == {3}
    assert banned_ngram_tokens([1, 2], 4) == set()
    assert banned_ngram_tokens([5, 6, 5], 1) == {5, 6}


@pytest.mark.gpu
def test_cuda_engine_matches_forward_in_bf16():
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=512, d_model=256, n_heads=4, n_cores=2, logical_depth=2, ffn_hidden=512,
                          chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    model = WarpStateLM(cfg).cuda().eval()
    ids = torch.randint(0, 512, (4, 384), device="cuda")
    with torch.no_grad():
        full = model(ids).float()  # FP32 oracle
    engine = DecodeEngine(model, dtype=torch.bfloat16)
    logits = engine.prefill(ids[:, :256])      # two complete chunks through the fused kernels
    assert torch.allclose(logits, full[:, 255], rtol=0.05, atol=0.05)
    for t in range(256, 384):                  # CUDA-graph replay per token, crossing a chunk boundary
        logits = engine.step(ids[:, t])
        if t in (300, 383):
            assert torch.allclose(logits, full[:, t], rtol=0.05, atol=0.05), t
    engine2 = DecodeEngine(model, dtype=torch.bfloat16, use_cuda_graph=False)
    engine2.prefill(ids[:, :130])              # one chunk fused + 2 stepped tokens
    for t in range(130, 384):
        last = engine2.step(ids[:, t])
    assert torch.allclose(last, logits, rtol=0.05, atol=0.05)


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [1, 16, 17, 64])
def test_decode_gemm_against_fp32(batch):
    """Weight-streaming GEMM: all four epilogues, with and without K splits, ragged batch."""
    from warpstate_ai_b200.ops import _ext, gemm
    from warpstate_ai_b200.ops.decode import pack_weight
    _ext.require()
    ops = torch.ops.ws_b200
    torch.manual_seed(batch)
    flag = gemm.error_flag(torch.device("cuda"))

    def rel(a, b):
        return float((a.float() - b).norm() / b.norm().clamp_min(1e-12))

    for n, k in [(1280, 256), (256, 1024), (2048, 2048), (2048, 7168), (1000, 512)]:
        w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        x = torch.randn(batch, k, device="cuda").bfloat16()
        ref = x.float() @ w.float().T
        out = torch.full((batch, n), float("nan"), device="cuda", dtype=torch.bfloat16)
        ops.decode_gemm(w, x, n, 0, out, flag)
        assert rel(out, ref) < 0.004, (n, k, "bf16")
        out32 = torch.full((batch, n), float("nan"), device="cuda")
        ops.decode_gemm(w, x, n, 3, out32, flag)
        assert rel(out32, ref) < 1e-4, (n, k, "f32")
        splits = ops.decode_gemm_splits(n, k)
        part = torch.full((splits, batch, n), float("nan"), device="cuda")
        ops.decode_gemm(w, x, n, 1, part, flag)
        assert rel(part.sum(0), ref) < 1e-4, (n, k, "split", splits)
        # the tile-contiguous weight copy gives the same results bit for bit
        wp = pack_weight(w)
        out_p = torch.full_like(out, float("nan"))
        ops.decode_gemm(wp, x, n, 0, out_p, flag, True)
        assert torch.equal(out_p, out), (n, k, "packed bf16")
        part_p = torch.full_like(part, float("nan"))
        ops.decode_gemm(wp, x, n, 1, part_p, flag, True)
        assert torch.equal(part_p, part), (n, k, "packed split")
    assert ops.decode_gemm_splits(2048, 2048) > 1 and ops.decode_gemm_splits(10240, 2048) == 1
    h, k = 512, 256
    w = (torch.randn(2 * h, k, device="cuda") * 0.05).bfloat16()
    x = torch.randn(batch, k, device="cuda").bfloat16()
    both = x.float() @ w.float().T
    ref = both[:, :h] * torch.nn.functional.silu(both[:, h:])
    act = torch.full((batch, h), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.decode_gemm(w, x, h, 2, act, flag)
    assert rel(act, ref) < 0.006
    act_p = torch.full_like(act, float("nan"))
    ops.decode_gemm(pack_weight(w, swiglu=True), x, h, 2, act_p, flag, True)
    assert torch.equal(act_p, act)
    gemm.check_device_errors()


@pytest.mark.gpu
def test_decode_reduce_norm_and_attention_step_kernels():
    from warpstate_ai_b200.ops import _ext, attention
    _ext.require()
    ops = torch.ops.ws_b200
    torch.manual_seed(3)
    b, d, h = 5, 256, 4
    x = torch.randn(b, d, device="cuda")
    part = torch.randn(3, b, d, device="cuda")
    scale, bias, w = (torch.randn(d, device="cuda") * 0.1 for _ in range(3))
    want = (x + part.sum(0)) * (1 + scale) + bias
    out = torch.empty(b, d, device="cuda", dtype=torch.bfloat16)
    xx = x.clone()
    ops.decode_reduce_norm(xx, part, None, None, scale, bias, w, 1e-5, out)
    assert torch.allclose(xx, want, rtol=1e-5, atol=1e-5)
    normed = want * torch.rsqrt(want.pow(2).mean(-1, keepdim=True) + 1e-5) * w
    assert torch.allclose(out.float(), normed, rtol=0.02, atol=0.02)
    table = torch.randn(50, d, device="cuda")
    tok = torch.tensor([0, 49, 7, 7, 3], device="cuda")
    ops.decode_reduce_norm(xx, None, tok, table, None, None, w, 1e-5, out)
    assert torch.equal(xx, table[tok])
    # attention step at several in-chunk positions against the PyTorch formulation
    from warpstate_ai_b200.ops import reference as R
    rope = attention.rope_table(torch.device("cuda"))
    cos, sin = R.rope_tables(128, 64, torch.device("cuda"), torch.float32)
    kc, vc, uc = (torch.randn(b, h, 128, 64, device="cuda").bfloat16() for _ in range(3))
    mixed = (torch.randn(b, h, 64, 64, device="cuda") * 0.2).bfloat16()
    for pos in (0, 1, 63, 127):
        qkvgu = torch.randn(b, 5 * d, device="cuda").bfloat16()
        q, k, v, g, u = (t.view(b, h, 64) for t in qkvgu.chunk(5, dim=-1))
        c, s = cos[pos].view(1, 1, 64), sin[pos].view(1, 1, 64)
        qr = (q.float() * c + R.rotate_pairs(q.float()) * s).bfloat16()
        kr = (k.float() * c + R.rotate_pairs(k.float()) * s).bfloat16()
        k2, v2, u2 = kc.clone(), vc.clone(), uc.clone()
        k2[:, :, pos], v2[:, :, pos], u2[:, :, pos] = kr, v, u
        scores = torch.einsum("bhd,bhcd->bhc", qr.float(), k2.float()) * 0.125
        visible = (torch.arange(128, device="cuda") <= pos).view(1, 1, 128)
        p = torch.softmax(scores.masked_fill(~visible, -torch.inf), dim=-1)
        local = torch.einsum("bhc,bhcd->bhd", p, v2.float())
        memory = torch.einsum("bhi,bhij->bhj", qr.float(), mixed.float()) * 0.125
        gate = torch.sigmoid(g.float())
        ref = (gate * local + (1 - gate) * memory).reshape(b, d)
        y = torch.empty(b, d, device="cuda", dtype=torch.bfloat16)
        ka, va, ua = kc.clone(), vc.clone(), uc.clone()
        ops.decode_attn(qkvgu, ka, va, ua, mixed, rope, torch.tensor(pos, device="cuda"), h, y)
        assert torch.allclose(y.float(), ref, rtol=0.02, atol=0.02), pos
        assert torch.equal(ka, k2) and torch.equal(va, v2) and torch.equal(ua, u2)


@pytest.mark.gpu
def test_kernel_decode_path_matches_pytorch_path():
    torch.manual_seed(1)
    cfg = WarpStateConfig(vocab_size=512, d_model=256, n_heads=4, n_cores=2, logical_depth=3, ffn_hidden=512,
                          chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    model = WarpStateLM(cfg).cuda().eval()
    ids = torch.randint(0, 512, (3, 200), device="cuda")
    fast = DecodeEngine(model, dtype=torch.bfloat16)
    slow = DecodeEngine(model, dtype=torch.bfloat16, use_kernels=False, use_cuda_graph=False)
    assert fast._kernels_usable(3) and not slow._kernels_usable(3)
    for t in range(200):   # crosses a chunk boundary at 128
        a, b = fast.step(ids[:, t]), slow.step(ids[:, t])
        if t % 37 == 0 or t == 199:
            assert torch.allclose(a, b, rtol=0.05, atol=0.05), t
    assert fast._kbufs is not None and slow._kbufs is None
    # capture / replay evidence: one capture, every step a replay; the eager engine replays nothing
    assert fast.graph_counters.as_dict() == {"capture_calls": 1, "replay_calls": 200, "eager_steps": 0, "invalidations": 0,
                                             "kernels_per_replay": 2 * 3 + 3 if fast._layer_tail else 7 * 3 + 2,
                                                 "replay_calls_by_batch": {"3": 200}}
    assert slow.graph_counters.replay_calls == 0 and slow.graph_counters.eager_steps == 200
    from warpstate_ai_b200.serve.graph_stats import collect_graph_diagnostics
    with collect_graph_diagnostics(fast) as diagnostics:
        fast.step(ids[:, 0])
        fast.step(ids[:2, 0])        # another batch size: the captured graph is dropped and a new one recorded
    assert diagnostics.snapshot() == {"capture_calls": 1, "replay_calls": 2, "eager_steps": 0, "invalidations": 1,
                                      "kernels_per_replay": 7 * 3 + 2, "replay_calls_by_batch": {"3": 1, "2": 1}}
    # the engine on tile-contiguous weight copies produces the same logits bit for bit
    packed = DecodeEngine(model, dtype=torch.bfloat16, pack_weights=True)
    plain = DecodeEngine(model, dtype=torch.bfloat16, use_cuda_graph=False)
    for t in range(5):
        assert torch.equal(packed.step(ids[:, t]), plain.step(ids[:, t])), t


def test_graph_counters_on_cpu_count_eager_steps():
    from warpstate_ai_b200.serve.graph_stats import collect_graph_diagnostics
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=64, d_model=32, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=48, chunk_size=8,
                          gradient_checkpointing=False)
    engine = DecodeEngine(WarpStateLM(cfg).eval(), dtype=torch.float32)
    with collect_graph_diagnostics(engine) as diagnostics:
        for token in range(5):
            engine.step(torch.tensor([token, token + 1]))
    assert diagnostics.snapshot() == {"capture_calls": 0, "replay_calls": 0, "eager_steps": 5, "invalidations": 0,
                                      "kernels_per_replay": 0, "replay_calls_by_batch": {}}


def test_pack_weight_round_trip_and_tile_order():
    """CPU: the tile-by-tile copy restores to the original, and a tile is the promised block."""
    from warpstate_ai_b200.ops.decode import pack_weight, unpack_weight
    torch.manual_seed(0)
    w = torch.randn(300, 200).bfloat16()
    packed = pack_weight(w)
    assert packed.shape == (3, 4, 128, 64) and packed.is_contiguous()
    assert torch.equal(unpack_weight(packed, 300, 200), w)
    assert torch.equal(packed[1, 2, :, :], w[128:256, 128:192])
    assert float(packed[2, 0, 300 - 256:, :].abs().sum()) == 0.0  # rows past the weight are zero
    ug = torch.randn(2 * 128, 64).bfloat16()
    p2 = pack_weight(ug, swiglu=True)
    assert p2.shape == (2, 1, 128, 64)
    assert torch.equal(p2[1, 0, :64], ug[64:128]) and torch.equal(p2[1, 0, 64:], ug[128 + 64:256])
    assert torch.equal(unpack_weight(p2, 256, 64, swiglu=True), ug)
    with pytest.raises(ValueError):
        pack_weight(torch.randn(2 * 96, 64), swiglu=True)


@pytest.mark.gpu
def test_greedy_decode_without_the_host_matches_the_host_driven_loop():
    """`decode_greedy` (token pick, hand-back and position counter inside the step graph; steps queued without any
    synchronisation) against arg-max on the host after every `step`, across a chunk boundary and across a read-out of
    the history buffer: the same tokens, and the engines end in the same state."""
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.serve.engine import DecodeEngine
    torch.manual_seed(3)
    cfg = WarpStateConfig(vocab_size=512, d_model=128, n_heads=2, n_cores=2, logical_depth=3, ffn_hidden=256, chunk_size=128,
                          gradient_checkpointing=False, parallel_memory=True)
    with torch.device("cuda"):
        model = WarpStateLM(cfg)
    model.eval().requires_grad_(False)
    prompt = torch.randint(0, 512, (5, 100), device="cuda")
    steps = 70                                  # positions 100 .. 169: crosses the chunk boundary at 128
    host = DecodeEngine(model, dtype=torch.bfloat16)
    token = torch.argmax(host.prefill(prompt), dim=-1)
    first = token.clone()
    want = []
    for _ in range(steps):
        token = torch.argmax(host.step(token), dim=-1)
        want.append(token)
    want = torch.stack(want, dim=1)
    device_side = DecodeEngine(model, dtype=torch.bfloat16)
    device_side.GREEDY_CAPACITY = 32            # three read-outs of the history buffer
    assert torch.equal(torch.argmax(device_side.prefill(prompt), dim=-1), first)
    events = []
    got = device_side.decode_greedy(first, steps, events)
    torch.cuda.synchronize()
    assert got.shape == (5, steps) and torch.equal(got, want)
    assert len(events) == steps + 1 and all(a.elapsed_time(b) > 0 for a, b in zip(events, events[1:]))
    assert device_side.pos == host.pos == (100 + steps) % 128 and int(device_side.pos_dev) == device_side.pos
    for mine, theirs in zip(device_side.states, host.states):
        assert torch.equal(mine.fast, theirs.fast) and torch.equal(mine.k, theirs.k)
    counters = device_side.graph_counters.as_dict()
    assert counters["replay_calls"] >= steps and counters["eager_steps"] == 0
    # a host-driven step after the device-driven run continues from the same position
    assert torch.equal(torch.argmax(device_side.step(got[:, -1]), dim=-1), torch.argmax(host.step(want[:, -1]), dim=-1))


@pytest.mark.gpu
@pytest.mark.parametrize("batch,d,heads,ffn", [(5, 128, 2, 256), (64, 512, 8, 1024), (33, 2048, 32, 7168)])
def test_persistent_layer_tail_is_bit_identical_to_the_launch_per_projection_step(monkeypatch, batch, d, heads, ffn):
    """One cooperative launch per layer for out_proj .. next in_proj (grid barriers in place of kernel boundaries)
    against the seven launches it replaces: the same k-block order and the same reduction order, so the logits of
    every step must be equal bit for bit -- which also checks every barrier, since a phase that ran early would read
    stale activations.  The last shape is the production layer (144 work items on 148 SMs)."""
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.ops.gemm import check_device_errors
    from warpstate_ai_b200.serve.engine import DecodeEngine
    torch.manual_seed(11)
    cfg = WarpStateConfig(vocab_size=1024, d_model=d, n_heads=heads, n_cores=2, logical_depth=3, ffn_hidden=ffn,
                          chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    with torch.device("cuda"):
        model = WarpStateLM(cfg)
    model.eval().requires_grad_(False)
    prompt = torch.randint(0, 1024, (batch, 40), device="cuda")
    monkeypatch.setenv("WS_DECODE_LAYER_TAIL", "0")
    plain = DecodeEngine(model, dtype=torch.bfloat16)
    token = torch.argmax(plain.prefill(prompt), dim=-1)
    assert plain._kbufs is not None and not plain._layer_tail
    monkeypatch.setenv("WS_DECODE_LAYER_TAIL", "1")
    fused = DecodeEngine(model, dtype=torch.bfloat16)
    assert torch.equal(torch.argmax(fused.prefill(prompt), dim=-1), token)
    assert fused._layer_tail
    for step in range(6):
        want = plain.step(token).clone()
        got = fused.step(token).clone()
        check_device_errors()
        assert torch.equal(got, want), (step, float((got - want).abs().max()))
        token = torch.argmax(want, dim=-1)
    # 2 + 2 launches per layer + 3: embedding norm, first in_proj, head
    assert fused.graph_counters.kernels_per_replay == 2 * 3 + 3
    assert plain.graph_counters.kernels_per_replay == 7 * 3 + 2


def test_decode_greedy_on_cpu_is_the_plain_loop():
    """Where there is no kernel path (CPU) `decode_greedy` is arg-max after every `step`, across a chunk boundary."""
    torch.manual_seed(2)
    cfg = WarpStateConfig(vocab_size=97, d_model=32, n_heads=2, n_cores=2, logical_depth=2, ffn_hidden=48, chunk_size=8,
                          gradient_checkpointing=False, parallel_memory=True)
    model = WarpStateLM(cfg).eval().requires_grad_(False)
    prompt = torch.randint(0, 97, (3, 5))
    a, b = DecodeEngine(model, dtype=torch.float32), DecodeEngine(model, dtype=torch.float32)
    token = torch.argmax(a.prefill(prompt), dim=-1)
    assert torch.equal(torch.argmax(b.prefill(prompt), dim=-1), token)
    want, t = [], token
    for _ in range(9):
        t = torch.argmax(a.step(t), dim=-1)
        want.append(t)
    got = b.decode_greedy(token, 9)
    assert got.shape == (3, 9) and torch.equal(got, torch.stack(want, dim=1))
    assert b.pos == a.pos == (5 + 9) % 8
    assert b.decode_greedy(got[:, -1], 0).shape == (3, 0)


def test_an_engine_first_used_in_inference_mode_can_be_used_outside_it():
    """The chat entry points run under ``torch.inference_mode()``; the buffers they leave in the engine cannot be written
    from ordinary code, so a later direct call gets fresh ones rather than an error."""
    engine = DecodeEngine(tiny(), dtype=torch.float32)
    ids = torch.randint(0, 97, (2, 11))
    with torch.inference_mode():
        inside = engine.prefill(ids).clone()
        engine.step(torch.tensor([3, 4]))
    assert engine.states[0].fast.is_inference()
    outside = engine.prefill(ids)                      # same batch size: would clear the old buffers in place
    assert not engine.states[0].fast.is_inference() and torch.equal(outside, inside)
    following = engine.step(torch.tensor([3, 4]))
    with torch.inference_mode():
        again = engine.prefill(ids)
        assert torch.equal(again, inside) and torch.equal(engine.step(torch.tensor([3, 4])), following)
