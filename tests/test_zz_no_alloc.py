"""The allocation-free RMSNorm backward (exported C symbol ``ws_rmsnorm_bwd_static``).

Some embedders of the kernel library may not call cudaMalloc at all -- they gave the whole GPU
to their own pool at start-up, or they run inside a latency-critical loop that must not touch
the allocator.  For them the library carries its scratch memory inside its own image.  This test
plays such a caller: it goes through the plain C ABI with ctypes (no torch op in between; torch
only provides the input and output buffers, which are the caller's business), calls twice in a
row because all calls share the one built-in scratch array, and checks both results against the
regular torch-op entry point.  It also checks that a row wider than the limit is refused up front.

Collected last on purpose: a failure here must not hide any other test from a run that stops at
the first failure.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


@pytest.fixture(scope="module")
def lib():
    from warpstate_ai_b200.ops import _ext
    handle = _ext.cdll()
    fn = handle.ws_rmsnorm_bwd_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    handle.ws_static_scratch_strerror.restype = ctypes.c_char_p
    handle.ws_static_scratch_strerror.argtypes = [ctypes.c_int]
    return handle


def call_static(lib, dz, x, rstd, w, dres, scale, want_bf16=True):
    rows, d = x.shape
    dx = torch.empty_like(x)
    dxb = torch.empty(rows, d, dtype=torch.bfloat16, device=x.device) if want_bf16 else None
    dw = torch.empty(d, dtype=torch.float32, device=x.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ws_rmsnorm_bwd_static(ptr(dz), ptr(x), int(x.dtype == torch.bfloat16), ptr(rstd), ptr(w), ptr(dres),
                                   ptr(scale), rows, d, ptr(dx), ptr(dxb), ptr(dw), stream)
    return rc, dx, dxb, dw


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_regular_entry_point(lib, dtype):
    torch.manual_seed(0)
    torch.cuda.set_device(0)
    ops = torch.ops.ws_b200
    cases = []
    for rows, d in [(4096, 2048), (777, 1280)]:  # second call is smaller: stale partial rows stay behind it
        x = torch.randn(rows, d, device="cuda").to(dtype)
        w = torch.rand(d, device="cuda") + 0.5
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
        dz = torch.randn(rows, d, device="cuda").bfloat16()
        dres = torch.randn(rows, d, device="cuda").to(dtype)
        scale = torch.randn(d, device="cuda") * 0.1
        cases.append((dz, x, rstd, w, dres, scale))
    results = [call_static(lib, *case) for case in cases]  # back to back, same stream
    torch.cuda.synchronize()
    for case, (rc, dx, dxb, dw) in zip(cases, results):
        assert rc == 0, lib.ws_static_scratch_strerror(rc)
        ref_dx, ref_dxb, ref_dw = ops.rmsnorm_bwd(*case, True)
        assert torch.equal(dx, ref_dx)          # same kernel, same launch shape: bit-identical
        assert torch.equal(dxb, ref_dxb)
        assert rel_l2(dw, ref_dw) < 1e-6
    # and against plain FP32 math, within the tolerance the other RMSNorm tests use
    dz, x, rstd, w, dres, scale = cases[0]
    xr = x.float().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr).backward(dz.float())
    expect = (dres.float() + xr.grad) * (1 + scale)
    assert rel_l2(results[0][1], expect) < (2e-3 if dtype == torch.float32 else 8e-3)
    assert rel_l2(results[0][3], wr.grad) < 5e-3


def test_rejects_what_does_not_fit(lib):
    x = torch.zeros(8, 4096, device="cuda")
    rc, *_ = call_static(lib, x.bfloat16(), x, torch.ones(8, device="cuda"), torch.ones(4096, device="cuda"),
                         None, None, want_bf16=False)
    assert rc == -1                                     # WS_STATIC_ERR_BAD_SHAPE: the width limit is the one that binds
    assert b"2048" in lib.ws_static_scratch_strerror(rc)
    assert b"scratch" in lib.ws_static_scratch_strerror(-30)   # the array-bound guard exists but is unreachable
