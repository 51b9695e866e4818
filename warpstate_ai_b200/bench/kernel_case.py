"""Run ONE small, self-terminating case of a named kernel (for `ncu -k <kernel>` captures).

Each case holds well under a few GB on the device, uses operands larger than the 126 MB L2 where
DRAM figures matter, launches the kernel a handful of times and exits.

    python -m warpstate_ai_b200.bench.kernel_case gemm_fwd
    ncu --set full --clock-control none -k regex:gemm_kernel -s 2 -c 1 -o prof \
        python -m warpstate_ai_b200.bench.kernel_case gemm_fwd
"""
from __future__ import annotations

import sys

import torch

from ..ops import attention, gemm as G


def gemm_case(kind: str) -> None:
    m, k, n = 8192, 2048, 10240
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
    dy = torch.randn(m, n, device="cuda").bfloat16()
    grad = torch.zeros(n, k, device="cuda")
    w_down = (torch.randn(k, n // 2, device="cuda") * 0.02).bfloat16()
    packed = torch.randn(m, n, device="cuda").bfloat16()
    for _ in range(3):
        if kind == "gemm_fwd":
            G.linear(x, w)
        elif kind == "gemm_dx":
            G.grad_input(dy, w)
        elif kind == "gemm_dw":
            G.grad_weight_accumulate(dy, x, grad)
        elif kind == "gemm_swiglu":
            G.linear_swiglu(x, w)
        elif kind == "gemm_swiglu_bwd":
            # dAct = dy[m, 2048] @ w_down[2048, 5120]; epilogue reads packed (up|gate) [m, 10240]
            G.grad_input_swiglu(dy[:, :k].contiguous() if False else x, w_down, packed)
    torch.cuda.synchronize()


def attention_case(kind: str) -> None:
    from .. import WarpStateConfig
    from ..models.warpstate import WarpStateCore
    cfg = WarpStateConfig(vocab_size=64, d_model=2048, n_heads=32, n_cores=1, logical_depth=1, ffn_hidden=256,
                          chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    core = WarpStateCore(cfg).cuda()
    batch, seq = 4, 2048
    qkvgu = torch.randn(batch * seq, 5 * 2048, device="cuda").bfloat16()
    dy = torch.randn(batch * seq, 2048, device="cuda").bfloat16()
    for _ in range(3):
        y, saved = attention.forward(qkvgu, core, batch, seq)
        if kind == "attn_bwd":
            attention.backward(dy, qkvgu, saved, core, batch, seq)
    torch.cuda.synchronize()


def main() -> None:
    kind = sys.argv[1] if len(sys.argv) > 1 else "gemm_fwd"
    if kind.startswith("gemm"):
        gemm_case(kind)
    elif kind.startswith("attn"):
        attention_case(kind)
    else:
        raise SystemExit(f"unknown case {kind}")
    G.check_device_errors()
    print(f"{kind}: ok")


if __name__ == "__main__":
    main()
