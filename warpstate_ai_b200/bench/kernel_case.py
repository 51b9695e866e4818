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


def norm_case() -> None:
    """RMSNorm forward (with depth modulation) and backward on [16384, 2048] FP32 rows."""
    ops = torch.ops.ws_b200
    rows, d = 16384, 2048
    x = torch.randn(rows, d, device="cuda")
    w, scale, bias = (torch.randn(d, device="cuda") * 0.1 + (1.0 if i == 0 else 0.0) for i in range(3))
    dz = torch.randn(rows, d, device="cuda").bfloat16()
    dres = torch.randn(rows, d, device="cuda")
    for _ in range(3):
        z, rstd, xmod = ops.rmsnorm_fwd(x, scale, bias, w, 1e-5, True)
        ops.rmsnorm_bwd(dz, xmod, rstd, w, dres, scale, True)
    torch.cuda.synchronize()


def lmhead_case() -> None:
    """Fused LM-head cross entropy (forward statistics GEMM, dlogits GEMM) on 8192 x 32768 x 2048."""
    from ..ops import lmhead
    rows, d, vocab = 8192, 2048, 32768
    h = torch.randn(rows, d, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(vocab, d, device="cuda") * 0.02).bfloat16()
    labels = torch.randint(0, vocab, (rows,), device="cuda")
    for _ in range(3):
        lse, logp = torch.ops.ws_b200.lm_head_fwd(h.detach(), w, labels, -100, G.error_flag(h.device))
        torch.ops.ws_b200.lm_head_dlogits(h.detach(), w, labels, lse, torch.full((rows,), 1.0 / rows, device="cuda"),
                                          G.error_flag(h.device))
    torch.cuda.synchronize()


def adamw_case() -> None:
    """AdamW + clip scale + BF16 re-cast over a 256 M-element arena slice (30 bytes per element)."""
    n = 256 << 20
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda") * 1e-3
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    coef = torch.ones(1, device="cuda")
    for step in range(1, 4):
        torch.ops.ws_b200.adamw_step(p, g, m, v, pb, 1e-4, 0.9, 0.95, 1e-8, 0.1, step, coef, 1.0)
    torch.cuda.synchronize()


def scan_case() -> None:
    """Chunk writes + memory scan (forward) for batch 8 x 2048 tokens x 32 heads."""
    ops = torch.ops.ws_b200
    batch, seq, heads = 8, 2048, 32
    qkvgu = torch.randn(batch * seq, 5 * 2048, device="cuda").bfloat16()
    rope = attention.rope_table(qkvgu.device, pair_major=True)
    logits = [torch.zeros(heads, device="cuda") for _ in range(3)]
    for _ in range(3):
        writes = ops.chunk_writes(qkvgu, rope, batch, seq, heads, G.error_flag(qkvgu.device))
        ops.memory_scan(writes, logits[0], logits[1], logits[2], True, False, None, None)
    torch.cuda.synchronize()


def decode_case() -> None:
    """Decode-step GEMMs at batch 64: in_proj (direct), up/gate (SwiGLU), down (split-K partials);
    each with row-major weights, then with the tile-contiguous copy."""
    ops = torch.ops.ws_b200
    flag = G.error_flag(torch.device("cuda"))
    x = torch.randn(64, 2048, device="cuda").bfloat16()
    act = torch.randn(64, 7168, device="cuda").bfloat16()
    w_in = (torch.randn(10240, 2048, device="cuda") * 0.02).bfloat16()
    w_ug = (torch.randn(14336, 2048, device="cuda") * 0.02).bfloat16()
    w_down = (torch.randn(2048, 7168, device="cuda") * 0.02).bfloat16()
    out = torch.empty(64, 10240, device="cuda", dtype=torch.bfloat16)
    a = torch.empty(64, 7168, device="cuda", dtype=torch.bfloat16)
    part = torch.empty(ops.decode_gemm_splits(2048, 7168), 64, 2048, device="cuda")
    from ..ops.decode import pack_weight
    p_in, p_ug, p_down = pack_weight(w_in), pack_weight(w_ug, swiglu=True), pack_weight(w_down)
    for _ in range(3):
        ops.decode_gemm(w_in, x, 10240, 0, out, flag)
        ops.decode_gemm(w_ug, x, 7168, 2, a, flag)
        ops.decode_gemm(w_down, act, 2048, 1, part, flag)
        ops.decode_gemm(p_in, x, 10240, 0, out, flag, True)
        ops.decode_gemm(p_ug, x, 7168, 2, a, flag, True)
        ops.decode_gemm(p_down, act, 2048, 1, part, flag, True)
    torch.cuda.synchronize()


def main() -> None:
    kind = sys.argv[1] if len(sys.argv) > 1 else "gemm_fwd"
    from ..ops import _ext
    _ext.require()
    if kind.startswith("gemm"):
        gemm_case(kind)
    elif kind.startswith("attn"):
        attention_case(kind)
    elif kind in ("norm", "lmhead", "adamw", "scan", "decode"):
        {"norm": norm_case, "lmhead": lmhead_case, "adamw": adamw_case, "scan": scan_case, "decode": decode_case}[kind]()
    else:
        raise SystemExit(f"unknown case {kind}")
    G.check_device_errors()
    print(f"{kind}: ok")


if __name__ == "__main__":
    main()
