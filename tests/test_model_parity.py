"""The plain-PyTorch model against the reference implementation imported as a library
(baseline/_ref, when installed): same state-dict keys, same losses and gradients in FP32."""
import importlib
import sys
from pathlib import Path

import pytest
import torch

from warpstate_ai_b200 import WarpStateConfig, WarpStateLM, warpstate_2b, warpstate_smoke

REF = Path(__file__).resolve().parents[1] / "baseline" / "_ref"


def load_reference():
    if not (REF / "warpstate" / "model.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    saved = {k: v for k, v in sys.modules.items() if k == "warpstate" or k.startswith("warpstate.")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, str(REF))
    try:
        cfg_mod = importlib.import_module("warpstate.config")
        model_mod = importlib.import_module("warpstate.model")
    finally:
        sys.path.remove(str(REF))
        for k in [k for k in sys.modules if k == "warpstate" or k.startswith("warpstate.")]:
            del sys.modules[k]
        sys.modules.update(saved)
    return cfg_mod, model_mod


def tiny(parallel):
    return dict(vocab_size=97, d_model=32, n_heads=4, n_cores=2, logical_depth=4, ffn_hidden=48,
                chunk_size=8, gradient_checkpointing=False, parallel_memory=parallel, loss_chunk_size=16)


def test_2b_parameter_count_on_meta_device():
    with torch.device("meta"):
        model = WarpStateLM(warpstate_2b())
    assert model.num_parameters() == 2_005_111_424
    assert len(model.state_dict()) == 256


@pytest.mark.parametrize("parallel", [False, True])
def test_matches_reference_forward_backward(parallel):
    cfg_mod, model_mod = load_reference()
    torch.manual_seed(0)
    ours = WarpStateLM(WarpStateConfig(**tiny(parallel)))
    ref = model_mod.WarpStateLM(cfg_mod.WarpStateConfig(**tiny(parallel)))
    assert list(ours.state_dict().keys()) == list(ref.state_dict().keys())
    ref.load_state_dict(ours.state_dict())
    with torch.no_grad():
        for m in (ours, ref):
            m.depth_scale.normal_(0, 0.1)
            m.depth_bias.normal_(0, 0.1)
        ref.load_state_dict(ours.state_dict())
    ids = torch.randint(0, 97, (2, 32))
    tgt = torch.randint(0, 97, (2, 32))
    tgt[0, :5] = -100
    for return_logits in (True, False):
        ours.zero_grad()
        ref.zero_grad()
        if return_logits:
            t = tgt.clamp_min(0)
            lo, loss_o = ours(ids, t)
            lr, loss_r = ref(ids, t)
            assert torch.allclose(lo, lr, rtol=1e-5, atol=1e-6)
        else:
            _, loss_o = ours(ids, tgt, return_logits=False)
            _, loss_r = ref(ids, tgt, return_logits=False)
        assert torch.allclose(loss_o, loss_r, rtol=1e-6, atol=1e-6)
        loss_o.backward()
        loss_r.backward()
        for (name, po), (_, pr) in zip(ours.named_parameters(), ref.named_parameters()):
            assert torch.allclose(po.grad, pr.grad, rtol=1e-4, atol=1e-6), name


@pytest.mark.parametrize("parallel", [False, True])
def test_decode_matches_reference(parallel):
    cfg_mod, model_mod = load_reference()
    torch.manual_seed(1)
    ours = WarpStateLM(WarpStateConfig(**tiny(parallel))).eval()
    ref = model_mod.WarpStateLM(cfg_mod.WarpStateConfig(**tiny(parallel))).eval()
    ref.load_state_dict(ours.state_dict())
    ids = torch.randint(0, 97, (2, 20))
    co = ours.init_generation_cache(2, torch.device("cpu"), torch.float32)
    cr = ref.init_generation_cache(2, torch.device("cpu"), torch.float32)
    for t in range(20):
        a = ours.step(ids[:, t:t + 1], co)
        b = ref.step(ids[:, t:t + 1], cr)
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("parallel", [False, True])
def test_step_equals_forward_across_chunk_boundaries(parallel):
    torch.manual_seed(2)
    model = WarpStateLM(WarpStateConfig(**tiny(parallel))).eval()
    ids = torch.randint(0, 97, (2, 24))
    with torch.no_grad():
        full = model(ids)
        caches = model.init_generation_cache(2, torch.device("cpu"), torch.float32)
        steps = torch.cat([model.step(ids[:, t:t + 1], caches) for t in range(24)], dim=1)
    assert torch.allclose(full, steps, rtol=2e-5, atol=2e-6)


def test_smoke_config_forward_backward_adamw_roundtrip(tmp_path):
    torch.manual_seed(0)
    cfg = warpstate_smoke()
    model = WarpStateLM(cfg)
    ids = torch.randint(0, cfg.vocab_size, (2, 512))
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.1, betas=(0.9, 0.95))
    _, loss = model(ids[:, :-1].contiguous()[:, :384], ids[:, 1:].contiguous()[:, :384], return_logits=False)
    assert abs(float(loss) - 10.4) < 0.3
    loss.backward()
    opt.step()
    path = tmp_path / "m.pt"
    torch.save({"config": vars(cfg), "model": model.state_dict()}, path)
    blob = torch.load(path, weights_only=False)
    again = WarpStateLM(WarpStateConfig(**blob["config"]))
    again.load_state_dict(blob["model"])
    for a, b in zip(model.parameters(), again.parameters()):
        assert torch.equal(a, b)


def test_all_masked_labels_give_zero_loss_and_zero_grads():
    torch.manual_seed(3)
    model = WarpStateLM(WarpStateConfig(**tiny(True)))
    ids = torch.randint(0, 97, (1, 16))
    _, loss = model(ids, torch.full((1, 16), -100), return_logits=False)
    assert float(loss) == 0.0
    loss.backward()
    assert all(p.grad is None or float(p.grad.abs().sum()) == 0.0 for p in model.parameters())


def test_shim_package_exports():
    import warpstate
    from warpstate.model import WarpStateLM as Shim
    assert warpstate.WarpStateLM is Shim is WarpStateLM


def test_exported_helpers_match_the_reference():
    """`warpstate.model` also exports the rotary helpers and the small modules; same numbers, same call forms."""
    _, ref = load_reference()
    import warpstate.model as ours
    torch.manual_seed(3)
    cos_o, sin_o = ours.rope_cos_sin(8, 6, torch.device("cpu"), torch.float32)
    cos_r, sin_r = ref.rope_cos_sin(8, 6, torch.device("cpu"), torch.float32)
    assert torch.equal(cos_o, cos_r) and torch.equal(sin_o, sin_r)
    x = torch.randn(2, 3, 4, 8, 6)
    assert torch.equal(ours.rotate_half(x), ref.rotate_half(x))
    assert torch.allclose(ours.apply_rope(x, cos_o, sin_o), ref.apply_rope(x, cos_r, sin_r), rtol=0, atol=1e-7)
    norm_o, norm_r = ours.RMSNorm(6, eps=1e-5), ref.RMSNorm(6, eps=1e-5)
    with torch.no_grad():
        norm_o.weight.normal_()
        norm_r.weight.copy_(norm_o.weight)
    for value in (x, x.bfloat16()):
        assert torch.equal(norm_o(value), norm_r(value))
    ffn_o, ffn_r = ours.SwiGLU(6, 10), ref.SwiGLU(6, 10)
    ffn_r.load_state_dict(ffn_o.state_dict())
    assert torch.allclose(ffn_o(x), ffn_r(x), rtol=1e-6, atol=1e-7)
    assert [f for f in ours.LayerCache.__dataclass_fields__] == [f for f in ref.LayerCache.__dataclass_fields__]


@pytest.mark.parametrize("parallel", [False, True])
def test_one_core_matches_the_reference_core_with_gradients(parallel):
    cfg_mod, ref = load_reference()
    from warpstate_ai_b200.models.warpstate import WarpStateCore
    torch.manual_seed(4)
    ours = WarpStateCore(WarpStateConfig(**tiny(parallel)))
    theirs = ref.WarpStateCore(cfg_mod.WarpStateConfig(**tiny(parallel)))
    with torch.no_grad():
        for logit in (ours.fast_decay_logit, ours.slow_decay_logit, ours.memory_mix_logit):
            logit.add_(torch.randn_like(logit))
    theirs.load_state_dict(ours.state_dict())
    assert torch.equal(ours.rope_cos, theirs.rope_cos) and torch.equal(ours.rope_sin, theirs.rope_sin)
    xo = torch.randn(2, 24, 32, requires_grad=True)
    xr = xo.detach().clone().requires_grad_(True)
    weight = torch.randn(2, 24, 32)
    (ours(xo) * weight).sum().backward()
    (theirs(xr) * weight).sum().backward()
    assert torch.allclose(xo.grad, xr.grad, rtol=1e-4, atol=1e-6)
    for (name, po), (_, pr) in zip(ours.named_parameters(), theirs.named_parameters()):
        assert torch.allclose(po.grad, pr.grad, rtol=1e-4, atol=2e-6), name
    caches = (ours.init_cache(2, torch.device("cpu"), torch.float32), theirs.init_cache(2, torch.device("cpu"), torch.float32))
    for position in range(11):                                   # crosses the 8-position chunk boundary
        token = torch.randn(2, 1, 32)
        assert torch.allclose(ours.step(token, caches[0]), theirs.step(token, caches[1]), rtol=1e-5, atol=1e-6)
        assert caches[0].chunk_len == caches[1].chunk_len == (position + 1) % 8
        for field in ("fast_state", "slow_state", "k_cache", "v_cache", "write_accum"):
            assert torch.allclose(getattr(caches[0], field), getattr(caches[1], field), rtol=1e-5, atol=1e-6), field
