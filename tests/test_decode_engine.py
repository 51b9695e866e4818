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
