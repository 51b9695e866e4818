"""Fused all-gather + FP32->BF16 cast + GEMM over a row-sharded weight (`parallel/sharded_linear.py`).

* CPU: shard sizing; two gloo ranks on the collective fallback (ownership, cached re-use, publish, gradient
  scatter to the row owners, SwiGLU form).
* One GPU: the kernel with 1, 3, 4 and 8 emulated shards (all on the device) against a plain
  PyTorch FP32 product of the BF16-rounded operands; the landing buffer must equal the BF16 cast of
  the weight bit for bit, and the cached second call (ordinary GEMM on the landing buffer) must
  equal the fused call bit for bit.  A wait that cannot be satisfied (a flag nobody sets) is not
  constructible here without a missing peer, so the time-out path is covered by the 2-GPU grad-sync test.
* Two GPUs (child processes, file-store rendezvous): real peer shards in symmetric memory.
"""
import json
import sys
from pathlib import Path

import pytest
import torch

from warpstate_ai_b200.parallel.sharded_linear import rows_per_shard

ROOT = Path(__file__).resolve().parents[1]


def test_rows_per_shard_covers_and_aligns():
    for n in (8, 1000, 2048, 10240, 14336, 32768):
        for world in (1, 2, 3, 4, 8):
            per = rows_per_shard(n, world)
            assert per % 8 == 0 and per * world >= n and (per - 8) * world < n + 8 * world


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 3, 4, 8])
def test_fused_gather_cast_gemm_emulated_shards(world):
    from warpstate_ai_b200.ops import _ext, gemm
    from warpstate_ai_b200.parallel.sharded_linear import ShardedWeight
    _ext.require()
    torch.manual_seed(world)
    for m, n, k in [(512, 1024, 512), (300, 1000, 256), (4096, 10240, 2048)]:
        w = torch.randn(n, k, device="cuda") * 0.05
        x = torch.randn(m, k, device="cuda").bfloat16()
        sw = ShardedWeight.emulated(w, world)
        assert torch.equal(sw.full_weight(), w)
        y = sw.forward(x)
        assert torch.equal(sw.gathered, w.bfloat16()), (m, n, k, "landing buffer")
        ref = x.float() @ w.bfloat16().float().T
        rel = float((y.float() - ref).norm() / ref.norm())
        assert rel < 0.004, (m, n, k, rel)
        again = sw.forward_cached(x)
        assert torch.equal(again, y), (m, n, k, "cached GEMM differs from the fused launch")
        # a changed shard is picked up by the next fused launch
        sw._keep[world - 1].mul_(2.0)
        sw.publish()
        y2 = sw.forward(x)
        assert torch.equal(sw.gathered, sw.full_weight().bfloat16())
        assert not torch.equal(y2, y)
    gemm.check_device_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 4, 8])
def test_fused_gather_cast_swiglu_gemm_emulated_shards(world):
    """Up/gate weight [2h, k]: the launch gathers up and gate rows alternately and applies the SwiGLU epilogue."""
    from warpstate_ai_b200.ops import _ext, gemm
    from warpstate_ai_b200.parallel.sharded_linear import ShardedWeight
    _ext.require()
    torch.manual_seed(10 + world)
    for m, h, k in [(512, 256, 512), (300, 384, 256), (2048, 7168, 2048)]:
        w = torch.randn(2 * h, k, device="cuda") * 0.05
        x = torch.randn(m, k, device="cuda").bfloat16()
        sw = ShardedWeight.emulated(w, world, swiglu=True)
        packed, act = sw.forward(x)
        assert torch.equal(sw.gathered, w.bfloat16()), (m, h, k, "landing buffer")
        both = x.float() @ w.bfloat16().float().T
        assert float((packed.float() - both).norm() / both.norm()) < 0.004, (m, h, k)
        ref = both[:, :h] * torch.nn.functional.silu(both[:, h:])
        assert float((act.float() - ref).norm() / ref.norm()) < 0.008, (m, h, k)
        packed2, act2 = sw.forward_cached(x)
        assert torch.equal(packed2, packed) and torch.equal(act2, act), (m, h, k, "cached GEMM differs")
    gemm.check_device_errors()
    with pytest.raises(ValueError):
        ShardedWeight.emulated(torch.randn(2 * 96, 64, device="cuda"), 1, swiglu=True)


@pytest.mark.gpu
def test_sharded_linear_module_gradients_single_rank():
    from warpstate_ai_b200.ops import _ext
    from warpstate_ai_b200.parallel.sharded_linear import ShardedLinear, ShardedWeight
    _ext.require()
    torch.manual_seed(5)
    n, k = 768, 512
    w = torch.randn(n, k, device="cuda") * 0.05
    layer = ShardedLinear(ShardedWeight.emulated(w, 1))
    grads = []
    for step in range(2):                      # the second micro-batch reuses the landing buffer
        x = torch.randn(2, 256, k, device="cuda", requires_grad=True)
        dy = torch.randn(2, 256, n, device="cuda").bfloat16()
        y = layer(x)
        y.backward(dy)
        xr = x.detach().bfloat16().float().requires_grad_(True)
        wr = w.bfloat16().float().requires_grad_(True)
        yr = xr @ wr.T
        yr.backward(dy.float())
        assert float((y.float() - yr).norm() / yr.norm()) < 0.004
        assert float((x.grad - xr.grad).norm() / xr.grad.norm()) < 0.006
        grads.append(wr.grad)
    total = grads[0] + grads[1]
    assert float((layer.weight.shard_grad.view(-1, k)[:n] - total).norm() / total.norm()) < 0.004
    assert layer.weight.gathered_valid
    layer.publish()
    assert not layer.weight.gathered_valid


def worker(rank: int, world: int, out_dir: Path) -> None:
    import torch.distributed as dist
    from warpstate_ai_b200.ops import _ext, gemm
    from warpstate_ai_b200.parallel.sharded_linear import ShardedWeight
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=(out_dir / "rendezvous").as_uri(), rank=rank, world_size=world,
                            device_id=device)
    _ext.require()
    report = {}
    torch.manual_seed(0)                       # the same full weight on every rank
    n, k, m = 2048, 1024, 1024
    w = torch.randn(n, k, device=device) * 0.05
    torch.manual_seed(100 + rank)              # different activations per rank
    x = torch.randn(m, k, device=device).bfloat16()
    sw = ShardedWeight.from_full(w, rank, world)
    y = sw.forward(x)
    report["landing_equal"] = bool(torch.equal(sw.gathered, w.bfloat16()))
    ref = x.float() @ w.bfloat16().float().T
    report["rel"] = float((y.float() - ref).norm() / ref.norm())
    report["cached_equal"] = bool(torch.equal(sw.forward_cached(x), y))
    # every rank scales its own shard; after publish() all ranks see all the new rows
    sw.shard.mul_(1.0 + 0.5 * (rank + 1))
    sw.publish()
    y2 = sw.forward(x)
    per = sw.rows
    expect = w.clone()
    for r in range(world):
        expect[r * per:(r + 1) * per].mul_(1.0 + 0.5 * (r + 1))
    report["landing_equal_after_update"] = bool(torch.equal(sw.gathered, expect.bfloat16()))
    ref2 = x.float() @ expect.bfloat16().float().T
    report["rel_after_update"] = float((y2.float() - ref2).norm() / ref2.norm())
    # module: dW rows of every owner are the sum over ranks
    from warpstate_ai_b200.parallel.sharded_linear import ShardedLinear
    layer = ShardedLinear(sw)
    xg = x.float().requires_grad_(True)
    torch.manual_seed(200 + rank)
    dy = torch.randn(m, n, device=device).bfloat16()
    layer(xg).backward(dy)
    dw_local = dy.float().T @ x.float()        # this rank's contribution, all rows
    dist.all_reduce(dw_local)
    mine = dw_local[rank * per:(rank + 1) * per]
    got = sw.shard_grad.view(per, k)[:mine.shape[0]]
    report["dw_rel"] = float((got - mine).norm() / mine.norm())
    dxr = dy.float() @ expect.bfloat16().float()
    report["dx_rel"] = float((xg.grad - dxr).norm() / dxr.norm())
    gemm.check_device_errors()
    torch.cuda.synchronize()
    dist.barrier()
    (out_dir / f"report-{rank}.json").write_text(json.dumps(report))
    dist.destroy_process_group()


needs_two_gpus = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                    reason="needs two CUDA devices")


@pytest.mark.gpu
@pytest.mark.multigpu
@needs_two_gpus
def test_fused_gather_cast_gemm_two_gpus(tmp_path):
    import os
    import subprocess
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    procs = [subprocess.Popen([sys.executable, __file__, str(rank), "2", str(tmp_path)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(2)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outputs.append(out)
    for rank, p in enumerate(procs):
        assert p.returncode == 0, f"rank {rank} failed:\n{outputs[rank][-3000:]}"
    for rank in range(2):
        r = json.loads((tmp_path / f"report-{rank}.json").read_text())
        assert r["landing_equal"] and r["cached_equal"] and r["landing_equal_after_update"], r
        assert r["rel"] < 0.004 and r["rel_after_update"] < 0.004, r
        assert r["dw_rel"] < 0.004 and r["dx_rel"] < 0.006, r


def cpu_worker(rank: int, world: int, out_dir: Path) -> None:
    """gloo ranks on CPU: the collective fallback keeps ownership, publish, re-use and gradient scatter."""
    import torch.distributed as dist
    from warpstate_ai_b200.parallel.sharded_linear import ShardedLinear, ShardedWeight
    dist.init_process_group("gloo", init_method=(out_dir / "rendezvous").as_uri(), rank=rank, world_size=world)
    torch.manual_seed(0)
    n, k, m = 40, 16, 24
    w = torch.randn(n, k)
    torch.manual_seed(100 + rank)
    x = torch.randn(m, k).bfloat16()
    dy = torch.randn(m, n).bfloat16()
    sw = ShardedWeight.from_full_collective(w, rank, world)
    layer = ShardedLinear(sw)
    report = {"rows": sw.rows}
    xg = x.float().requires_grad_(True)
    y = layer(xg)
    ref = x.float() @ w.bfloat16().float().T
    report["rel"] = float((y.float() - ref).norm() / ref.norm())
    y.backward(dy)
    dw = dy.float().T @ x.float()
    dist.all_reduce(dw)
    padded = torch.zeros(sw.rows * world, k)
    padded[:n] = dw
    mine = padded[rank * sw.rows:(rank + 1) * sw.rows]
    report["dw_err"] = float((sw.shard_grad.view(sw.rows, k) - mine).abs().max())
    report["cached"] = bool(sw.gathered_valid)
    # every owner changes its rows; after publish() the next forward sees all of them
    sw.shard.mul_(2.0 + rank)
    layer.publish()
    report["stale_after_publish"] = not sw.gathered_valid
    y2 = layer(x.float())
    expect = torch.zeros(sw.rows * world, k)
    expect[:n] = w
    for r in range(world):
        expect[r * sw.rows:(r + 1) * sw.rows] *= 2.0 + r
    ref2 = x.float() @ expect[:n].bfloat16().float().T
    report["rel_after_update"] = float((y2.float() - ref2).norm() / ref2.norm())
    # two updates of owner-only AdamW equal dense AdamW on the whole weight with the summed gradient
    from warpstate_ai_b200.parallel.sharded_linear import ShardedRowsAdamW
    torch.manual_seed(0)
    w0 = torch.randn(n, k)
    st = ShardedWeight.from_full_collective(w0, rank, world)
    lin = ShardedLinear(st)
    opt = ShardedRowsAdamW([lin], lr=1e-2, weight_decay=0.1)
    dense = torch.nn.Parameter(w0.clone())
    ref_opt = torch.optim.AdamW([dense], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for it in range(2):
        torch.manual_seed(300 + 10 * it + rank)
        xi = torch.randn(m, k).bfloat16()
        gi = torch.randn(m, n).bfloat16()
        opt.zero_grad()
        lin(xi.float().requires_grad_(True)).backward(gi)
        opt.step()
        grad = gi.float().T @ xi.float()
        dist.all_reduce(grad)
        ref_opt.zero_grad()
        dense.grad = grad
        ref_opt.step()
    full = torch.zeros(st.rows * world, k)
    full[:n] = dense.detach()
    mine_rows = full[rank * st.rows:(rank + 1) * st.rows]
    report["adamw_err"] = float((st.shard.view(st.rows, k) - mine_rows).abs().max())
    report["adamw_moment_bytes"] = opt.memory_bytes()
    # SwiGLU form
    torch.manual_seed(1)
    wug = torch.randn(2 * 128, k)
    sg = ShardedWeight.from_full_collective(wug, rank, world, swiglu=True)
    packed, act = sg.forward(x)
    both = x.float() @ wug.bfloat16().float().T
    report["swiglu_rel"] = float((act.float() - both[:, :128] * torch.nn.functional.silu(both[:, 128:])).norm()
                                 / (both[:, :128] * torch.nn.functional.silu(both[:, 128:])).norm())
    (out_dir / f"report-{rank}.json").write_text(json.dumps(report))
    dist.barrier()
    dist.destroy_process_group()


def test_collective_fallback_two_cpu_ranks(tmp_path):
    import os
    import subprocess
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    procs = [subprocess.Popen([sys.executable, __file__, str(rank), "2", str(tmp_path), "cpu"], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(2)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=180)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outputs.append(out)
    for rank, p in enumerate(procs):
        assert p.returncode == 0, f"rank {rank} failed:\n{outputs[rank][-3000:]}"
    for rank in range(2):
        r = json.loads((tmp_path / f"report-{rank}.json").read_text())
        assert r["rows"] == 24 and r["cached"] and r["stale_after_publish"], r
        assert r["rel"] < 0.01 and r["rel_after_update"] < 0.01 and r["swiglu_rel"] < 0.02, r
        assert r["dw_err"] < 1e-3, r
        assert r["adamw_err"] < 2e-5 and r["adamw_moment_bytes"] == 2 * 4 * 24 * 16, r


if __name__ == "__main__":
    if len(sys.argv) > 4 and sys.argv[4] == "cpu":
        cpu_worker(int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3]))
    else:
        worker(int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3]))


def test_gather_chunk_and_flag_arithmetic_mirrors_the_kernel():
    """CPU mirror of the index arithmetic of the gather warps and of the producer's wait in
    `gemm2_kernel<..., GATHER=true>`: every weight row is copied exactly once, no chunk straddles two
    shards, and the number of chunks counted into a 128-row block equals what the producer waits for."""
    import re
    src = (ROOT / "warpstate_ai_b200" / "ops" / "csrc" / "gemm2_tcgen05.cu").read_text()
    rows_per_chunk = int(re.search(r"constexpr int GATHER_ROWS = (\d+);", src).group(1))
    block = int(re.search(r"constexpr int GATHER_BLOCK = (\d+);", src).group(1))
    assert block % rows_per_chunk == 0 and 8 % rows_per_chunk == 0
    for total_rows, h in [(1000, 0), (10240, 0), (1024, 0), (2 * 384, 384), (2 * 7168, 7168), (2 * 128, 128)]:
        for world in (1, 2, 3, 8):
            per = rows_per_shard(total_rows, world)
            chunks = (total_rows + rows_per_chunk - 1) // rows_per_chunk
            covered = [0] * total_rows
            counted = {}
            for c in range(chunks):
                row0 = (c & 1) * h + (c >> 1) * rows_per_chunk if h else c * rows_per_chunk
                rows = min(rows_per_chunk, total_rows - row0)
                assert rows > 0 and row0 // per == (row0 + rows - 1) // per, (total_rows, h, world, c)
                for r in range(row0, row0 + rows):
                    covered[r] += 1
                counted[row0 // block] = counted.get(row0 // block, 0) + 1
            assert all(v == 1 for v in covered), (total_rows, h, world)
            n_tile = 128 if h else 256
            out_features = h if h else total_rows
            for nb in range((out_features + n_tile - 1) // n_tile):
                for rank in (0, 1):
                    b = (h // block + nb if rank else nb) if h else 2 * nb + rank
                    block_rows = min(block, total_rows - b * block)
                    want = 0 if block_rows <= 0 else (block_rows + rows_per_chunk - 1) // rows_per_chunk
                    assert counted.get(b, 0) == want, (total_rows, h, world, nb, rank)
