"""Run-twice determinism of the whole training step on the GPU (the substitute for a race
detector that the reference also relies on): two trainers built from the same seed and fed the
same data must produce bit-identical losses, gradient norms and parameters after several updates,
and ragged shapes must not write outside their outputs (canary rows around GEMM outputs)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def run_updates(seed: int):
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.data.tokens import SyntheticTokens
    from warpstate_ai_b200.train.engine import Trainer
    torch.manual_seed(seed)
    cfg = WarpStateConfig(vocab_size=1024, d_model=256, n_heads=4, n_cores=2, logical_depth=4, ffn_hidden=512,
                          chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    device = torch.device("cuda")
    model = WarpStateLM(cfg).to(device)
    trainer = Trainer(model, device=device, lr=1e-3, weight_decay=0.1)
    data = SyntheticTokens(1 << 16, cfg.vocab_size, seed=5)
    losses, norms = [], []
    cursor = 0
    for _ in range(3):
        result = trainer.pretrain_update(data, cursor, 4 * 2 * 512, 2, 512, 1e-3)  # 4 micro-batches
        losses.append(result.loss)
        norms.append(result.grad_norm)
        cursor += 4 * 2 * 512
    return losses, norms, trainer.arena.master.clone(), trainer.optimizer.exp_avg_sq.clone()


def test_training_step_is_bitwise_reproducible():
    a = run_updates(0)
    b = run_updates(0)
    assert a[0] == b[0] and a[1] == b[1]
    assert torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
    c = run_updates(1)
    assert not torch.equal(a[2], c[2])


def test_ragged_gemm_outputs_stay_inside_their_rows():
    from warpstate_ai_b200.ops import gemm
    torch.manual_seed(0)
    m, n, k = 1000, 1368, 264   # ragged in every dimension; staged (TMA-clipped) and direct epilogues
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    canary = torch.full((m + 64, n), 7.0, device="cuda", dtype=torch.bfloat16)
    out = canary[32:32 + m]
    gemm.linear(x, w, out=out)
    assert torch.all(canary[:32] == 7.0) and torch.all(canary[32 + m:] == 7.0)
    resid = torch.randn(m, n, device="cuda")
    big = torch.full((m + 64, n), 7.0, device="cuda")
    gemm.linear_residual(x, w, resid, out=big[32:32 + m])
    assert torch.all(big[:32] == 7.0) and torch.all(big[32 + m:] == 7.0)
    ref = resid + x.float() @ w.float().T
    assert float((big[32:32 + m] - ref).norm() / ref.norm()) < 0.003
    h = 688
    wug = (torch.randn(2 * h, k, device="cuda") * 0.05).bfloat16()
    packed, act = gemm.linear_swiglu(x, wug)
    both = x.float() @ wug.float().T
    want = both[:, :h] * torch.nn.functional.silu(both[:, h:])
    assert float((act.float() - want).norm() / want.norm()) < 0.006
    dy = torch.randn(m, 256, device="cuda").bfloat16()
    w_down = (torch.randn(256, h, device="cuda") * 0.05).bfloat16()
    dpacked = gemm.grad_input_swiglu(dy, w_down, packed)
    assert torch.isfinite(dpacked.float()).all() and dpacked.shape == (m, 2 * h)
    gemm.check_device_errors()
