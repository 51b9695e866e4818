"""Python front-end of the tcgen05 GEMM (csrc/gemm_tcgen05.cu).

All operands are 2-D BF16 tensors with a contiguous last dimension.  The three products of a
linear layer ``y = x @ W.T`` (``x [M,K]``, ``W [N,K]``) are expressed without any transpose copy:

* forward  ``y  = x  @ W.T``   A = x  (K-major),  B = W  (K-major)
* dX       ``dx = dy @ W``     A = dy (K-major),  B = W  read MN-major (contraction over W's rows)
* dW       ``dW = dy.T @ x``   A = dy read MN-major, B = x read MN-major (contraction over tokens)
"""
from __future__ import annotations

import torch

from . import _ext

EPI_BF16 = 0
EPI_RESID_F32 = 1
EPI_SWIGLU = 2
EPI_ACC_F32 = 3
EPI_SWIGLU_BWD = 4
EPI_F32 = 5
EPI_RESID_BF16 = 6

_error_flags: dict[int, torch.Tensor] = {}


def error_flag(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait ran out."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    flag = _error_flags.get(index)
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        _error_flags[index] = flag
    return flag


def check_device_errors(device: torch.device | None = None) -> None:
    """Synchronising check of the error word; raises if any kernel gave up on a wait."""
    for index, flag in _error_flags.items():
        if device is not None and device.index not in (None, index):
            continue
        value = int(flag.item())
        if value != 0:
            flag.zero_()
            what = {5: "attention backward: a wait timed out", 6: "CTA-pair GEMM: a wait timed out",
                    7: "attention backward: dynamic shared memory is not 1024-byte aligned"}.get(
                        value, "a wait timed out")
            raise RuntimeError(f"ws_b200 kernel on cuda:{index} reported an error (code {value}: {what})")


_policy: dict[str, dict] = {}


def load_policy(path) -> int:
    """Adopt a ``candidate-policy.json`` written by ``bench.tune_gemm``: per problem
    (``op:tokens x out x in``) which kernel (``pair`` / ``single``) to use.  Returns the number of
    entries.  Problems without an entry keep the library default."""
    import json
    from pathlib import Path
    data = json.loads(Path(path).read_text())
    if data.get("format") != "warpstate-gemm-policy-v1":
        raise ValueError("not a GEMM policy file")
    _policy.clear()
    for entry in data["entries"]:
        _policy[entry["key"]] = {"kernel": entry["kernel"], "sm_limit": int(entry.get("sm_limit", 0))}
    return len(_policy)


def _policy_key(a_mn, b_mn, m, n, k) -> str:
    if a_mn and b_mn:
        return f"dw:{k}x{m}x{n}"
    if b_mn:
        return f"dx:{m}x{k}x{n}"
    return f"fwd:{m}x{n}x{k}"


def _gemm(a, b, a_mn, b_mn, epi, m, n, k, out, out2=None, aux=None, row_scale=None, alpha=1.0, beta=0.0):
    _ext.require()
    if _policy:
        choice = _policy.get(_policy_key(a_mn, b_mn, m, n, k))
        lib = _ext.cdll()
        lib.ws_gemm_set_pair_mode(-1 if choice is None else (1 if choice["kernel"] == "pair" else 0))
    torch.ops.ws_b200.gemm(a, b, a_mn, b_mn, epi, m, n, k, out, out2, aux, row_scale,
                           float(alpha), float(beta), error_flag(a.device))
    return out


def linear(x: torch.Tensor, w: torch.Tensor, row_scale: torch.Tensor | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """``x [M,K] @ w[N,K].T -> [M,N]`` BF16, optional per-row scale fused in the epilogue."""
    m, k = x.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    return _gemm(x, w, False, False, EPI_BF16, m, n, k, out, row_scale=row_scale)


def linear_f32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    return _gemm(x, w, False, False, EPI_F32, m, n, k, out)


def linear_residual(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """``resid + x @ w.T``; the residual stream may be FP32 or BF16 (output has its dtype)."""
    m, k = x.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty_like(resid)
    epi = EPI_RESID_F32 if resid.dtype == torch.float32 else EPI_RESID_BF16
    return _gemm(x, w, False, False, epi, m, n, k, out, aux=resid)


def linear_swiglu(x: torch.Tensor, w_up_gate: torch.Tensor, row_scale: torch.Tensor | None = None,
                  want_packed: bool = True):
    """Up/gate projection with the SwiGLU epilogue.

    ``w_up_gate`` is ``[2h, K]`` with the first ``h`` rows = up, last ``h`` rows = gate (the
    reference layout, warpstate/model.py:58-60).  Returns ``(packed [M,2h], act [M,h])``.
    """
    m, k = x.shape
    h = w_up_gate.shape[0] // 2
    packed = torch.empty((m, 2 * h), dtype=torch.bfloat16, device=x.device)
    act = torch.empty((m, h), dtype=torch.bfloat16, device=x.device)
    _gemm(x, w_up_gate, False, False, EPI_SWIGLU, m, h, k, packed, out2=act, row_scale=row_scale)
    return packed, act


def grad_input(dy: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``dy [M,N] @ w [N,K] -> [M,K]`` BF16."""
    m, n = dy.shape
    k = w.shape[1]
    if out is None:
        out = torch.empty((m, k), dtype=torch.bfloat16, device=dy.device)
    return _gemm(dy, w, False, True, EPI_BF16, m, k, n, out)


def grad_input_swiglu(dy: torch.Tensor, w_down: torch.Tensor, packed: torch.Tensor) -> torch.Tensor:
    """``dAct = dy [M,d] @ w_down [d,h]`` fused with the SwiGLU backward: returns ``(dUp|dGate) [M,2h]``."""
    m, d = dy.shape
    h = w_down.shape[1]
    out = torch.empty((m, 2 * h), dtype=torch.bfloat16, device=dy.device)
    return _gemm(dy, w_down, False, True, EPI_SWIGLU_BWD, m, h, d, out, aux=packed)


def grad_weight_accumulate(dy: torch.Tensor, x: torch.Tensor, grad: torch.Tensor,
                           accumulate: bool = True, alpha: float = 1.0) -> torch.Tensor:
    """``grad [N,K] (+)= alpha * dy[M,N].T @ x[M,K]`` with FP32 accumulation into ``grad``.

    This fuses what the reference does in three steps (BF16 dW GEMM, BF16->FP32 cast, FP32 add
    in autograd's AccumulateGrad; ops/benchmark_gradient_accumulation.py) and keeps the product
    in FP32 instead of rounding it to BF16 first.
    """
    tokens, n = dy.shape
    k = x.shape[1]
    return _gemm(dy, x, True, True, EPI_ACC_F32, n, k, tokens, grad, alpha=alpha,
                 beta=1.0 if accumulate else 0.0)


def grad_weight_accumulate_group(items) -> None:
    """``items`` = [(dy, x, grad, accumulate), ...]: every ``grad (+)= dy.T @ x`` in ONE persistent
    launch (up to four problems per launch), so the last partial wave of tiles is paid once for
    the group instead of once per weight."""
    _ext.require()
    items = list(items)
    for start in range(0, len(items), 4):
        part = items[start:start + 4]
        torch.ops.ws_b200.grad_weight_group([i[0] for i in part], [i[1] for i in part], [i[2] for i in part],
                                            [1.0 if i[3] else 0.0 for i in part], error_flag(part[0][0].device))


def grad_weight_bf16(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    tokens, n = dy.shape
    k = x.shape[1]
    out = torch.empty((n, k), dtype=torch.bfloat16, device=dy.device)
    return _gemm(dy, x, True, True, EPI_BF16, n, k, tokens, out)
