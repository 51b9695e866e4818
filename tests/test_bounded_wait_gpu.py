"""A device-side wait that nothing satisfies must run out, report what it waited for, and leave
the context usable (how peer failure surfaces in the collective kernels: a flag that a dead rank
never sets).  Nothing here faults or hangs the GPU: the wait has a 0.3 s budget."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_expired_wait_sets_status_and_context_survives():
    from warpstate_ai_b200.ops import _ext, gemm
    _ext.require()
    flag = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    begin = time.perf_counter()
    torch.ops.ws_b200.wait_probe(flag, 5, status, 0.3)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - begin
    code, bucket, src, expected, seen = status[:5].tolist()
    assert code == 9 and bucket == -1 and src == -1 and expected == 5 and seen == 0
    assert 0.25 < elapsed < 5.0
    # a satisfied wait returns at once and records nothing
    flag[0] = 7
    status.zero_()
    torch.ops.ws_b200.wait_probe(flag, 5, status, 0.3)
    torch.cuda.synchronize()
    assert status[:5].tolist() == [0, 0, 0, 0, 0]
    # the context still runs kernels of every kind
    x = torch.randn(256, 256, device="cuda").bfloat16()
    y = gemm.linear(x, x)
    assert torch.isfinite(y.float()).all()
    gemm.check_device_errors()


def test_trainer_surfaces_a_collective_timeout(monkeypatch):
    """The host side of the same path: a non-zero status word raises with a readable message."""
    from warpstate_ai_b200.parallel.grad_sync import FusedGradSync
    sync = FusedGradSync.__new__(FusedGradSync)
    sync.rank = 3
    sync.status = torch.tensor([1, 12, 5, 40, 39, 0, 0, 0], dtype=torch.int32, device="cuda")
    message = sync.describe_error()
    assert "rank 3" in message and "bucket 12" in message and "peer 5" in message and "expected 40" in message
