"""Data-parallel gradient synchronisation.

The file doubles as the worker (the reference's pattern, test_distributed_execution.py:78-177):
the test spawns ranks as child processes with a file-store rendezvous, each rank writes a JSON
report, the parent asserts on the reports.

* CPU (gloo, 2 ranks): two-rank training with `CollectiveGradSync` equals single-process
  training on the concatenated batch (the global token-mean objective), including an update in
  which one rank has no valid tokens.
* GPU (2 ranks, needs two devices): the in-kernel all-reduce over symmetric memory equals
  NCCL all_reduce / world on random buffers (peer-load path and, when offered, the multimem
  path), and two-rank training with the fused synchroniser equals the NCCL synchroniser.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def spawn(mode: str, world: int, tmp_path: Path, env_extra=None, timeout=240):
    env = dict(os.environ)
    env.update(env_extra or {})
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    procs = []
    for rank in range(world):
        procs.append(subprocess.Popen([sys.executable, __file__, mode, str(rank), str(world), str(tmp_path)],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outputs.append(out)
    for rank, p in enumerate(procs):
        assert p.returncode == 0, f"rank {rank} failed:\n{outputs[rank][-3000:]}"
    return [json.loads((tmp_path / f"report-{rank}.json").read_text()) for rank in range(world)]


def tiny_model(device):
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=128, d_model=256 if device.type == "cuda" else 32, n_heads=4, n_cores=2,
                          logical_depth=2, ffn_hidden=256 if device.type == "cuda" else 48,
                          chunk_size=128 if device.type == "cuda" else 8, gradient_checkpointing=False,
                          parallel_memory=True)
    return WarpStateLM(cfg).to(device), cfg


def run_updates(trainer, cfg, world, rank, seq, micro_batch, targets, after_first=None):
    from warpstate_ai_b200.data.tokens import SyntheticTokens
    data = SyntheticTokens(4096, cfg.vocab_size, seed=3)
    losses = []
    cursor = 0
    for index, target in enumerate(targets):
        result = trainer.pretrain_update(data, cursor, target, micro_batch, seq, 1e-3)
        losses.append(result.loss)
        cursor += target
        if index == 0 and after_first is not None:
            after_first()
    return losses


def assert_same_training(a: torch.Tensor, b: torch.Tensor, lr: float, updates: int, what: str = "") -> None:
    """Two runs whose gradients agree to rounding but whose global norm was summed in a different order:
    AdamW turns a last-bit difference of a near-zero gradient into a difference of up to ``lr`` per update in
    that one element (its update is ~ ``lr * sign(g)``), so the comparison is statistical: almost every
    element within the reference's reconfiguration tolerances (test_training_execution.py:561-567), none
    further apart than the optimizer could move it."""
    diff = (a.double() - b.double()).abs()
    beyond = diff > (2e-5 + 1e-3 * b.double().abs())
    assert float(beyond.double().mean()) < 0.02, (what, float(beyond.double().mean()))
    assert float(diff.max()) <= 2.0 * lr * updates, (what, float(diff.max()))


def worker(mode: str, rank: int, world: int, out_dir: Path) -> None:
    import torch.distributed as dist
    from warpstate_ai_b200.train.engine import Trainer
    cuda = mode.startswith("gpu")
    if cuda:
        torch.cuda.set_device(rank)
        device = torch.device("cuda", rank)
    else:
        device = torch.device("cpu")
    dist.init_process_group("nccl" if cuda else "gloo", init_method=(out_dir / "rendezvous").as_uri(),
                            rank=rank, world_size=world, **({"device_id": device} if cuda else {}))
    report = {}
    seq = 256 if cuda else 16
    mb = 2
    if mode in ("cpu_train", "gpu_train"):
        from warpstate_ai_b200.parallel.grad_sync import CollectiveGradSync, FusedGradSync
        kinds = (["collective", "fused", "collective-sharded", "fused-sharded"] if cuda
                 else ["collective", "collective-sharded"])
        # 2 full updates, then one where the second rank's slice is empty
        targets = [world * mb * seq * 2, world * mb * seq * 2, mb * seq]
        for kind in kinds:
            model, cfg = tiny_model(device)
            sync = (FusedGradSync(device, world, rank, budget_seconds=20.0) if kind.startswith("fused")
                    else CollectiveGradSync(device, world, rank))
            trainer = Trainer(model, device=device, rank=rank, world_size=world, lr=1e-3, weight_decay=0.1,
                              grad_sync=sync, shard_optimizer=kind.endswith("sharded"))
            def first_update_snapshot(kind=kind, trainer=trainer):
                trainer.gather_for_checkpoint()
                torch.save(trainer.arena.master.detach().float().cpu(), out_dir / f"params1-{kind}-{rank}.pt")

            losses = run_updates(trainer, cfg, world, rank, seq, mb, targets, after_first=first_update_snapshot)
            trainer.gather_for_checkpoint()
            flat = trainer.arena.master.detach().float().cpu()
            state = trainer.optimizer.state_dict()
            if rank == 0:
                torch.save({k: {n: t.cpu() for n, t in v.items()} for k, v in state["state"].items()},
                           out_dir / f"adam-{kind}.pt")
            if kind.endswith("sharded"):
                report[kind + "-moment-bytes"] = trainer.optimizer.memory_bytes()
            report[kind] = {"losses": losses, "checksum": float(flat.double().sum()), "norm": float(flat.norm()),
                            "sync": sync.kind}
            torch.save(flat, out_dir / f"params-{kind}-{rank}.pt")
            dist.barrier()
    elif mode == "gpu_absent_peer":
        # A peer that never launches its side of a bucket reduction: the surviving rank's kernel
        # must give up after its time budget, say what it waited for, and leave the GPU usable.
        # Plain peer loads only (no multimem): NVLS is off for tests in which a rank goes quiet.
        from warpstate_ai_b200.ops import _ext, gemm
        from warpstate_ai_b200.parallel import symm
        _ext.require()
        n = 1 << 20
        buf = symm.allocate(n, torch.float32, device)
        flags = symm.allocate(64, torch.int32, device)
        status = torch.zeros(8, dtype=torch.int32, device=device)
        buf.tensor.fill_(float(rank + 1))
        torch.cuda.synchronize()
        dist.barrier()
        # step 1: both ranks take part
        torch.ops.ws_b200.grad_allreduce(buf.peer_ptrs, flags.peer_ptrs, 0, rank, world, 0, n, 0, 1, 1.0 / world, True, 8,
                                         None, status, 5.0)
        torch.cuda.synchronize()
        assert int(status[0]) == 0 and float(buf.tensor[0]) == 1.5
        dist.barrier()
        # step 2: rank 1 stays away (it is idle on the host, nothing of it is in flight)
        import time
        if rank == 0:
            begin = time.perf_counter()
            torch.ops.ws_b200.grad_allreduce(buf.peer_ptrs, flags.peer_ptrs, 0, rank, world, 0, n, 0, 2, 1.0 / world, True,
                                             8, None, status, 1.0)
            torch.cuda.synchronize()
            report["seconds"] = time.perf_counter() - begin
            report["status"] = status[:5].tolist()
            x = torch.randn(256, 256, device=device).bfloat16()
            report["context_alive"] = bool(torch.isfinite(gemm.linear(x, x).float()).all())
        dist.barrier()
    elif mode == "gpu_kernel":
        from warpstate_ai_b200.ops import _ext
        from warpstate_ai_b200.parallel import symm
        _ext.require()
        n = 3 * 1024 * 1024 + 256
        torch.manual_seed(100 + rank)
        for use_nvls in (False, True):
            buf = symm.allocate(n, torch.float32, device)
            flags = symm.allocate(64, torch.int32, device)
            mc = buf.multicast_ptr if use_nvls else 0
            if use_nvls and not mc:
                report["nvls"] = "unavailable"
                continue
            status = torch.zeros(8, dtype=torch.int32, device=device)
            worst = 0.0
            for seq_no in (1, 2):
                src = torch.randn(n, device=device)
                buf.tensor.copy_(src)
                want = src.clone()
                dist.all_reduce(want)
                want /= world
                torch.cuda.synchronize()
                dist.barrier()
                torch.ops.ws_b200.grad_allreduce(buf.peer_ptrs, flags.peer_ptrs, mc, rank, world, 256, n - 256, 0,
                                                 seq_no, 1.0 / world, True, 16, None, status, 20.0)
                torch.cuda.synchronize()
                dist.barrier()
                assert int(status[0]) == 0, status.tolist()
                assert torch.equal(buf.tensor[:256], src[:256])  # outside the bucket: untouched
                err = float((buf.tensor[256:] - want[256:]).abs().max())
                worst = max(worst, err)
                gathered = [torch.empty_like(buf.tensor) for _ in range(world)]
                dist.all_gather(gathered, buf.tensor)
                assert all(torch.equal(gathered[0][256:], g[256:]) for g in gathered)  # bit-identical on every rank
            report["nvls" if use_nvls else "p2p"] = worst
    (out_dir / f"report-{rank}.json").write_text(json.dumps(report))
    dist.barrier()
    dist.destroy_process_group()


# ----------------------------------------------------------------------------------- tests
def test_two_cpu_ranks_match_single_process(tmp_path):
    reports = spawn("cpu_train", 2, tmp_path, env_extra={"CUDA_VISIBLE_DEVICES": ""})
    a = torch.load(tmp_path / "params-collective-0.pt")
    b = torch.load(tmp_path / "params-collective-1.pt")
    assert torch.equal(a, b)
    assert reports[0]["collective"]["losses"] == pytest.approx(reports[1]["collective"]["losses"], rel=1e-6)
    # single process over the same global batches
    from warpstate_ai_b200.train.engine import Trainer
    device = torch.device("cpu")
    model, cfg = tiny_model(device)
    trainer = Trainer(model, device=device, lr=1e-3, weight_decay=0.1)
    losses = run_updates(trainer, cfg, 1, 0, 16, 2, [2 * 2 * 16 * 2, 2 * 2 * 16 * 2, 2 * 16])
    assert losses == pytest.approx(reports[0]["collective"]["losses"], rel=2e-5, abs=2e-6)
    assert torch.allclose(trainer.arena.master.detach().cpu(), a, rtol=1e-4, atol=2e-6)
    # the sharded optimizer (each rank updates half of every bucket) gives the same bits
    for rank in (0, 1):
        assert torch.equal(torch.load(tmp_path / f"params-collective-sharded-{rank}.pt"), a)
    assert reports[0]["collective-sharded"]["losses"] == reports[0]["collective"]["losses"]
    whole, sharded = torch.load(tmp_path / "adam-collective.pt"), torch.load(tmp_path / "adam-collective-sharded.pt")
    assert whole.keys() == sharded.keys()
    for index in whole:
        for name in ("step", "exp_avg", "exp_avg_sq"):
            assert torch.equal(whole[index][name], sharded[index][name]), (index, name)
    full_bytes = 2 * 4 * trainer.arena.numel
    assert reports[0]["collective-sharded-moment-bytes"] <= full_bytes // 2 + 64 * len(trainer.arena.buckets)


needs_two_gpus = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                    reason="needs two CUDA devices")


@pytest.mark.gpu
@pytest.mark.multigpu
@needs_two_gpus
def test_fused_allreduce_kernel_matches_nccl(tmp_path):
    reports = spawn("gpu_kernel", 2, tmp_path)
    for r in reports:
        assert r["p2p"] < 1e-6
        assert r["nvls"] == "unavailable" or r["nvls"] < 1e-5


@pytest.mark.gpu
@pytest.mark.multigpu
@needs_two_gpus
def test_absent_peer_times_out_with_a_status_and_a_usable_gpu(tmp_path):
    reports = spawn("gpu_absent_peer", 2, tmp_path, env_extra={"NCCL_NVLS_ENABLE": "0", "WARPSTATE_NVLS": "0"})
    r = reports[0]
    code, bucket, peer, expected, seen = r["status"]
    assert code == 1 and bucket == 0 and peer == 1 and expected == 2 and seen == 1  # waited for rank 1's "ready" of step 2
    assert 0.9 < r["seconds"] < 10.0 and r["context_alive"] is True


@pytest.mark.gpu
@pytest.mark.multigpu
@needs_two_gpus
def test_fused_sync_training_matches_nccl_sync(tmp_path):
    reports = spawn("gpu_train", 2, tmp_path)
    for kind in ("collective", "fused"):
        assert torch.equal(torch.load(tmp_path / f"params-{kind}-0.pt"), torch.load(tmp_path / f"params-{kind}-1.pt"))
    a = torch.load(tmp_path / "params-collective-0.pt")
    b = torch.load(tmp_path / "params-fused-0.pt")
    # after ONE update the two agree to rounding: the averaged gradients are bit-identical at two ranks and only
    # the global norm differs in its last bits (NCCL path: one kernel over the arena; fused path: per-CTA
    # partials of the reduce kernel, exchanged and added in rank order)
    assert torch.allclose(torch.load(tmp_path / "params1-collective-0.pt"), torch.load(tmp_path / "params1-fused-0.pt"),
                          rtol=1e-5, atol=1e-7)
    assert_same_training(b, a, 1e-3, 3, "fused vs collective")
    assert reports[0]["fused"]["losses"] == pytest.approx(reports[0]["collective"]["losses"], rel=1e-3)
    # sharded optimizer: reduce-scatter + update-and-broadcast kernel == all-reduce + replicated AdamW
    for kind in ("collective-sharded", "fused-sharded"):
        assert torch.equal(torch.load(tmp_path / f"params-{kind}-0.pt"), torch.load(tmp_path / f"params-{kind}-1.pt"))
    assert torch.allclose(torch.load(tmp_path / "params1-fused-sharded-0.pt"), torch.load(tmp_path / "params1-fused-0.pt"),
                          rtol=1e-5, atol=1e-7)
    assert_same_training(torch.load(tmp_path / "params-fused-sharded-0.pt"), b, 1e-3, 3, "fused-sharded vs fused")
    assert torch.allclose(torch.load(tmp_path / "params-collective-sharded-0.pt"), a, rtol=1e-5, atol=1e-7)
    assert reports[0]["fused-sharded"]["losses"] == pytest.approx(reports[0]["fused"]["losses"], rel=1e-3)


if __name__ == "__main__":
    worker(sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), Path(sys.argv[4]))


def test_allreduce_loop_partition_mirrors_the_kernel():
    """CPU mirror of the element loop of `grad_reduce_kernel` (four pieces per thread and pass, then a
    one-piece tail): every 16-byte piece of a rank's slice is handled exactly once, in increasing order per
    thread, for ragged slice lengths and CTA counts."""
    import re
    src = (ROOT / "warpstate_ai_b200" / "ops" / "csrc" / "comm.cu").read_text()
    unroll = int(re.search(r"constexpr int U = (\d+);", src).group(1))
    threads = int(re.search(r"constexpr int COMM_THREADS = (\d+);", src).group(1))
    for count4, world, ctas in [(1, 2, 1), (1000, 2, 3), (4096 + 7, 8, 4), (100000, 3, 16)]:
        per = (count4 + world - 1) // world
        seen = [0] * count4
        for rank in range(world):
            lo, hi = per * rank, min(count4, per * rank + per)
            stride = ctas * threads
            for cta in range(ctas):
                for tid in range(threads):
                    order = []
                    i = lo + cta * threads + tid
                    while i + (unroll - 1) * stride < hi:
                        order += [i + u * stride for u in range(unroll)]
                        i += unroll * stride
                    while i < hi:
                        order.append(i)
                        i += stride
                    assert order == sorted(order)
                    for index in order:
                        seen[index] += 1
        assert all(v == 1 for v in seen), (count4, world, ctas)
