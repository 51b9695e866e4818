"""tcgen05 GEMM and its fused epilogues against FP32 PyTorch references.

Tolerances follow the reference's own kernel tests: relative RMS < 0.003 for a BF16 GEMM
(test_matmul_kernels.py:163,188), relative L2 < 0.006 for the fused SwiGLU activation
(test_matmul_epilogue.py:70-79).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_rms(a, b):
    a = a.float()
    b = b.float()
    return float((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt().clamp_min(1e-12))


@pytest.fixture(scope="module", params=["pair", "single"])
def g(request):
    """Every case runs on both kernels: the CTA-pair (cta_group::2) one, taken for problems with at
    least 256 rows, and the single-CTA one."""
    from warpstate_ai_b200.ops import _ext, gemm
    lib = _ext.cdll()
    lib.ws_gemm_set_pair_mode(1 if request.param == "pair" else 0)
    yield gemm
    lib.ws_gemm_set_pair_mode(-1)


SHAPES = [(128, 256, 64), (256, 512, 256), (384, 1280, 256), (1000, 1376, 688), (2048, 2048, 2048),
          (4096, 10240, 2048), (72, 264, 136)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_linear_forward(g, m, n, k):
    torch.manual_seed(0)
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    y = g.linear(x, w)
    ref = x.float() @ w.float().T
    assert rel_rms(y, ref) < 0.003
    rs = torch.rand(m, device="cuda") + 0.5
    y2 = g.linear(x, w, row_scale=rs)
    assert rel_rms(y2, ref * rs[:, None]) < 0.003
    y3 = g.linear_f32(x, w)
    assert rel_rms(y3, ref) < 1e-4
    g.check_device_errors()


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_grad_input(g, m, n, k):
    torch.manual_seed(1)
    dy = torch.randn(m, n, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    dx = g.grad_input(dy, w)
    assert rel_rms(dx, dy.float() @ w.float()) < 0.003
    g.check_device_errors()


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_grad_weight(g, m, n, k):
    torch.manual_seed(2)
    dy = torch.randn(m, n, device="cuda").bfloat16()
    x = torch.randn(m, k, device="cuda").bfloat16()
    ref = dy.float().T @ x.float()
    grad = torch.full((n, k), 3.0, device="cuda")
    g.grad_weight_accumulate(dy, x, grad, accumulate=False)
    assert rel_rms(grad, ref) < 1e-4
    g.grad_weight_accumulate(dy, x, grad, accumulate=True, alpha=0.5)
    assert rel_rms(grad, 1.5 * ref) < 1e-4
    assert rel_rms(g.grad_weight_bf16(dy, x), ref) < 0.003
    g.check_device_errors()


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual(g, m, n, k, dtype):
    torch.manual_seed(3)
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    r = torch.randn(m, n, device="cuda").to(dtype)
    y = g.linear_residual(x, w, r)
    ref = r.float() + x.float() @ w.float().T
    assert y.dtype == dtype
    assert rel_rms(y, ref) < (1e-4 if dtype == torch.float32 else 0.004)
    g.check_device_errors()


@pytest.mark.parametrize("m,h,k", [(128, 128, 64), (256, 688, 256), (1000, 1024, 512), (2048, 7168, 2048)])
def test_swiglu_forward_backward(g, m, h, k):
    torch.manual_seed(4)
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(2 * h, k, device="cuda") * 0.05).bfloat16()
    packed, act = g.linear_swiglu(x, w)
    ref_packed = x.float() @ w.float().T
    assert rel_rms(packed, ref_packed) < 0.003
    up, gate = ref_packed.bfloat16().float().chunk(2, dim=-1)
    ref_act = torch.nn.functional.silu(gate) * up
    assert rel_rms(act, ref_act) < 0.006
    # backward: dAct = dy @ w_down ; (dUp|dGate) = swiglu'(packed) * dAct
    d = k
    dy = torch.randn(m, d, device="cuda").bfloat16()
    w_down = (torch.randn(d, h, device="cuda") * 0.05).bfloat16()
    dpacked = g.grad_input_swiglu(dy, w_down, packed)
    dact = (dy.float() @ w_down.float()).bfloat16().float()
    pu, pg = packed.float().chunk(2, dim=-1)
    s = torch.sigmoid(pg)
    ref_d = torch.cat([dact * pg * s, dact * pu * s * (1 + pg * (1 - s))], dim=-1)
    assert rel_rms(dpacked, ref_d) < 0.006
    g.check_device_errors()


def test_grouped_weight_gradients_match_single_launches(g):
    """Four dW problems of different shapes in one grouped launch == four separate launches, bit for bit."""
    torch.manual_seed(7)
    tokens = 1024
    shapes = [(512, 256), (256, 768), (1280, 256), (304, 264)]  # ragged last tile in both directions
    items, refs = [], []
    for n, k in shapes:
        dy = torch.randn(tokens, n, device="cuda").bfloat16()
        x = torch.randn(tokens, k, device="cuda").bfloat16()
        base = torch.randn(n, k, device="cuda")
        single = g.grad_weight_accumulate(dy, x, base.clone(), accumulate=True)
        refs.append(single)
        items.append((dy, x, base.clone(), True))
    g.grad_weight_accumulate_group(items)
    for (dy, x, grad, _), ref in zip(items, refs):
        assert torch.equal(grad, ref)
        assert rel_rms(grad - 0, ref) == 0.0
    fresh = [(dy, x, torch.full_like(grad, float("nan")), False) for dy, x, grad, _ in items]
    g.grad_weight_accumulate_group(fresh)  # beta = 0 must ignore what was there
    for (dy, x, grad, _) in fresh:
        assert rel_rms(grad, dy.float().T @ x.float()) < 1e-3
    g.check_device_errors()


def test_misaligned_row_pitch_is_rejected(g):
    dy = torch.zeros(64, 300, device="cuda").bfloat16()  # 600-byte pitch: not a legal TMA stride
    x = torch.zeros(64, 264, device="cuda").bfloat16()
    with pytest.raises(RuntimeError, match="row pitches"):
        g.grad_weight_accumulate(dy, x, torch.zeros(300, 264, device="cuda"))


@pytest.mark.gpu
def test_gemm_from_a_thread_whose_first_cuda_action_is_the_tensor_map():
    """A tensor-map encode is a driver call that needs a context current on the calling thread.  A fresh
    thread that only receives already allocated tensors (an autograd worker fed from the caching
    allocator) has none until the library binds it: the GEMM must work there as well."""
    import threading
    from warpstate_ai_b200.ops import gemm as G
    torch.manual_seed(0)
    x = torch.randn(512, 256, device="cuda").bfloat16()
    w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16()
    out = torch.empty(512, 384, device="cuda", dtype=torch.bfloat16)
    G.error_flag(x.device)          # created here, so that the thread allocates nothing
    torch.cuda.synchronize()
    result = {}

    def work():
        try:
            G.linear(x, w, out=out)
            torch.cuda.synchronize()
            result["ok"] = True
        except Exception as exc:   # reported to the main thread
            result["error"] = repr(exc)

    t = threading.Thread(target=work)
    t.start()
    t.join(60)
    assert result.get("ok"), result
    ref = x.float() @ w.float().T
    assert float((out.float() - ref).norm() / ref.norm()) < 0.004
