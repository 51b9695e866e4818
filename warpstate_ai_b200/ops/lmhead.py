"""Fused LM-head cross-entropy (front-end of the WS_EPI_CE_* GEMM epilogues and lmhead.cu).

Forward: one tcgen05 GEMM over the tied embedding matrix whose epilogue folds each 128-column
slice of the logits into (max, sum exp) and records the label's logit -- the ``[tokens, vocab]``
logits are never written.  Backward: the same GEMM recomputes the logits and its epilogue emits
``(softmax - onehot) * row_weight`` in BF16, which feeds the dX GEMM (gradient of the hidden
states) and the dW GEMM (FP32 accumulation into the tied embedding's gradient).

`loss_sum` is the summed cross-entropy over labels != -100 (reference warpstate/model.py:316-334,
ops/loss_experiment.py:14-19); `token_logps` is the per-row label log-probability used for
per-sequence sums in DPO (reference dpo.py:150-161).
"""
from __future__ import annotations

import torch

from . import _ext
from . import gemm as G

ROWS_PER_BLOCK = 8192  # bounds the BF16 dlogits scratch to 512 MiB at vocab 32768


def kernels_ready(hidden: torch.Tensor, weight: torch.Tensor) -> bool:
    return (hidden.is_cuda and hidden.dim() == 2 and weight.shape[0] % 8 == 0 and hidden.shape[1] % 8 == 0
            and _ext.available())


class _TokenLogps(torch.autograd.Function):
    """per-row log p(label) (0 where the label is -100); differentiable w.r.t. hidden and weight."""

    @staticmethod
    def forward(ctx, hidden, weight, labels):
        from .fused import bf16_weight
        ops = torch.ops.ws_b200
        hidden = hidden.contiguous()
        labels = labels.contiguous()
        wb = bf16_weight(weight)
        flag = G.error_flag(hidden.device)
        lse, logp = ops.lm_head_fwd(hidden, wb, labels, -100, flag)
        ctx.save_for_backward(hidden, labels, lse)
        ctx.weight = weight
        return logp

    @staticmethod
    def backward(ctx, grad_logp):
        from .fused import bf16_weight
        ops = torch.ops.ws_b200
        hidden, labels, lse = ctx.saved_tensors
        weight = ctx.weight
        wb = bf16_weight(weight)
        flag = G.error_flag(hidden.device)
        # d logp / d logits = onehot - softmax  ->  dlogits = (softmax - onehot) * (-grad), masked rows 0
        row_weight = (-grad_logp.float() * labels.ne(-100)).contiguous()
        dh = torch.empty_like(hidden)
        main = getattr(weight, "main_grad", None)
        grad_w = main if main is not None else torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        for start in range(0, hidden.shape[0], ROWS_PER_BLOCK):
            stop = min(start + ROWS_PER_BLOCK, hidden.shape[0])
            h = hidden[start:stop]
            dlogits = ops.lm_head_dlogits(h, wb, labels[start:stop], lse[start:stop], row_weight[start:stop], flag)
            G.grad_input(dlogits, wb, out=dh[start:stop])
            G.grad_weight_accumulate(dlogits, h, grad_w, accumulate=True)
        return dh, (None if main is not None else grad_w.to(weight.dtype)), None


def token_logps(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return _TokenLogps.apply(hidden, weight, labels)


def loss_sum(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return -token_logps(hidden, weight, labels).sum()
