"""Fully sharded parameters, gradients and optimizer state (`parallel/fsdp.py`) through the `Trainer`.

The file doubles as the worker: the tests spawn ranks as child processes with a file-store rendezvous,
each rank writes its results, the parent asserts on them.

* CPU (gloo, 2 ranks): sharded training equals replicated two-rank training bit for bit (same
  all-reduced gradients, same AdamW arithmetic, only the ownership differs), each rank holds half of the
  projection rows and moments, the unsharded checkpoint it writes (model and torch-format optimizer state)
  resumes in ONE replicated process to the weights of the uninterrupted run, and a skipped update
  (non-finite norm) leaves parameters and moments untouched.
* GPU (2 ranks, needs two devices): the same comparison through the fused kernels -- gather + cast + GEMM
  launches, side-stream gathers, segmented reduce-scatter, in-kernel norm exchange -- in both landing modes,
  with and without activation checkpointing.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def spawn(mode: str, world: int, tmp_path: Path, env_extra=None, timeout=420):
    env = dict(os.environ)
    env.update(env_extra or {})
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    procs = [subprocess.Popen([sys.executable, __file__, mode, str(rank), str(world), str(tmp_path)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(world)]
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


def tiny_model(device, checkpointing=False):
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    torch.manual_seed(0)
    cuda = device.type == "cuda"
    cfg = WarpStateConfig(vocab_size=128, d_model=256 if cuda else 32, n_heads=4, n_cores=3, logical_depth=3,
                          ffn_hidden=256 if cuda else 48, chunk_size=128 if cuda else 8,
                          gradient_checkpointing=checkpointing, parallel_memory=True)
    return WarpStateLM(cfg).to(device), cfg


def flat_state(state: dict) -> torch.Tensor:
    return torch.cat([state[k].detach().float().cpu().reshape(-1) for k in sorted(state)])


def run_updates(trainer, cfg, seq, micro_batch, targets, first=0, after_first=None):
    from warpstate_ai_b200.data.tokens import SyntheticTokens
    data = SyntheticTokens(8192, cfg.vocab_size, seed=3)
    losses = []
    cursor = sum(targets[:first])
    for index, target in enumerate(targets[first:]):
        result = trainer.pretrain_update(data, cursor, target, micro_batch, seq, 1e-3)
        losses.append(result.loss)
        cursor += target
        if index == 0 and after_first is not None:
            after_first()
    return losses


def assert_same_training(a: torch.Tensor, b: torch.Tensor, lr: float, updates: int, what: str = "") -> None:
    """Statistical comparison of two runs whose gradients agree to rounding (see tests/test_grad_sync.py):
    almost every element within the reference's reconfiguration tolerances, none further apart than AdamW
    could have moved it."""
    diff = (a.double() - b.double()).abs()
    beyond = diff > (2e-5 + 1e-3 * b.double().abs())
    assert float(beyond.double().mean()) < 0.02, (what, float(beyond.double().mean()))
    assert float(diff.max()) <= 2.0 * lr * updates, (what, float(diff.max()))


def worker(mode: str, rank: int, world: int, out_dir: Path) -> None:
    import torch.distributed as dist
    from warpstate_ai_b200.parallel.grad_sync import CollectiveGradSync, FusedGradSync
    from warpstate_ai_b200.train.engine import Trainer
    cuda = mode.startswith("gpu")
    if cuda:
        torch.cuda.set_device(rank)
        device = torch.device("cuda", rank)
    else:
        device = torch.device("cpu")
    dist.init_process_group("nccl" if cuda else "gloo", init_method=(out_dir / "rendezvous").as_uri(),
                            rank=rank, world_size=world, **({"device_id": device} if cuda else {}))
    seq, mb = (256, 2) if cuda else (16, 2)
    targets = [world * mb * seq * 2, world * mb * seq * 2, world * mb * seq]
    report = {}
    if cuda:
        kinds = [("replicated", None, False), ("stream", "stream", False), ("resident", "resident", False),
                 ("stream-ckpt", "stream", True)]
    else:
        kinds = [("replicated", None, False), ("stream", "stream", False)]
    for kind, shard, ckpt in kinds:
        model, cfg = tiny_model(device, checkpointing=ckpt)
        sync = FusedGradSync(device, world, rank, budget_seconds=20.0) if cuda else CollectiveGradSync(device, world, rank)
        trainer = Trainer(model, device=device, rank=rank, world_size=world, lr=1e-3, weight_decay=0.1,
                          grad_sync=sync, shard_params=shard)
        def first_update_snapshot(kind=kind, trainer=trainer):
            torch.save(flat_state(trainer.model_state_dict()), out_dir / f"params1-{kind}-{rank}.pt")

        losses = run_updates(trainer, cfg, seq, mb, targets[:2], after_first=first_update_snapshot)
        if shard and kind == "stream":
            # unsharded checkpoint after two updates (collective), then a skipped update that must change nothing
            checkpoint = {"model": trainer.model_state_dict(), "optimizer": trainer.optimizer.state_dict()}
            if rank == 0:
                torch.save(checkpoint, out_dir / "checkpoint.pt")
            report["held"] = trainer.sharded.memory_report()
            report["full_matrix_elements"] = sum(m.n * m.k for m in trainer.arena.matrices)
            report["owned_matrix_elements"] = int(trainer.sharded.master.numel())
        losses += run_updates(trainer, cfg, seq, mb, targets, first=2)
        state = trainer.model_state_dict()
        torch.save(flat_state(state), out_dir / f"params-{kind}-{rank}.pt")
        report[kind] = {"losses": losses, "sync": sync.kind}
        if shard and kind == "stream" and not cuda:
            before = flat_state(trainer.model_state_dict())
            moments = trainer.optimizer.m_sh.clone()
            steps = trainer.optimizer.step_count
            trainer.begin_update()
            trainer.arena.grad.fill_(float("nan"))
            stats = trainer.finish_update(1e-3)
            try:
                trainer.read_update_scalars(stats)
                report["skip_raised"] = False
            except RuntimeError:
                report["skip_raised"] = True
            report["skip_unchanged"] = bool(torch.equal(before, flat_state(trainer.model_state_dict()))
                                            and torch.equal(moments, trainer.optimizer.m_sh)
                                            and trainer.optimizer.step_count == steps)
        dist.barrier()
        del trainer, model
    if cuda:
        from warpstate_ai_b200.ops.gemm import check_device_errors
        check_device_errors()
    (out_dir / f"report-{rank}.json").write_text(json.dumps(report))
    dist.barrier()
    dist.destroy_process_group()


def test_two_cpu_ranks_sharded_equals_replicated_and_resumes_unsharded(tmp_path):
    reports = spawn("cpu", 2, tmp_path, env_extra={"CUDA_VISIBLE_DEVICES": ""})
    rep = torch.load(tmp_path / "params-replicated-0.pt")
    for rank in (0, 1):
        assert torch.equal(torch.load(tmp_path / f"params-stream-{rank}.pt"), rep)
    assert reports[0]["stream"]["losses"] == reports[0]["replicated"]["losses"]
    assert reports[0]["owned_matrix_elements"] * 2 == reports[0]["full_matrix_elements"]
    assert reports[0]["skip_raised"] is True and reports[0]["skip_unchanged"] is True
    # the unsharded checkpoint of the two sharded ranks resumes in one replicated process
    from warpstate_ai_b200.train.engine import Trainer
    device = torch.device("cpu")
    checkpoint = torch.load(tmp_path / "checkpoint.pt")
    model, cfg = tiny_model(device)
    trainer = Trainer(model, device=device, lr=1e-3, weight_decay=0.1)
    trainer.load_model_state_dict(checkpoint["model"])
    trainer.optimizer.load_state_dict(checkpoint["optimizer"])
    seq, mb, world = 16, 2, 2
    targets = [world * mb * seq * 2, world * mb * seq * 2, world * mb * seq]
    run_updates(trainer, cfg, seq, mb, targets, first=2)
    resumed = flat_state(trainer.model_state_dict())
    assert torch.allclose(resumed, rep, rtol=1e-4, atol=2e-6)
    # ... and in a sharded single process (another world size) as well
    model, cfg = tiny_model(device)
    trainer = Trainer(model, device=device, lr=1e-3, weight_decay=0.1, shard_params="stream")
    trainer.load_model_state_dict(checkpoint["model"])
    trainer.optimizer.load_state_dict(checkpoint["optimizer"])
    run_updates(trainer, cfg, seq, mb, targets, first=2)
    assert torch.equal(flat_state(trainer.model_state_dict()), resumed)


def test_skipped_update_leaves_replicated_state_untouched():
    """A non-finite gradient norm: the optimizer changes nothing and the trainer raises afterwards."""
    from warpstate_ai_b200.train.engine import Trainer
    device = torch.device("cpu")
    model, cfg = tiny_model(device)
    trainer = Trainer(model, device=device, lr=1e-3, weight_decay=0.1)
    run_updates(trainer, cfg, 16, 2, [64])
    before = trainer.arena.master.clone()
    m, v, steps = trainer.optimizer.exp_avg.clone(), trainer.optimizer.exp_avg_sq.clone(), trainer.optimizer.step_count
    trainer.begin_update()
    trainer.arena.grad[3] = float("inf")
    stats = trainer.finish_update(1e-3)
    with pytest.raises(RuntimeError, match="non-finite"):
        trainer.read_update_scalars(stats)
    assert torch.equal(trainer.arena.master, before)
    assert torch.equal(trainer.optimizer.exp_avg, m) and torch.equal(trainer.optimizer.exp_avg_sq, v)
    assert trainer.optimizer.step_count == steps


needs_two_gpus = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                    reason="needs two CUDA devices")


@pytest.mark.gpu
@pytest.mark.multigpu
@needs_two_gpus
def test_two_gpus_sharded_parameters_match_replicated(tmp_path):
    reports = spawn("gpu", 2, tmp_path)
    rep = torch.load(tmp_path / "params-replicated-0.pt")
    for kind in ("stream", "resident", "stream-ckpt"):
        a, b = torch.load(tmp_path / f"params-{kind}-0.pt"), torch.load(tmp_path / f"params-{kind}-1.pt")
        assert torch.equal(a, b), kind
        # one update: same gradients up to the rounding of the BF16 GEMMs (the gather casts the same FP32 rows)
        first = torch.load(tmp_path / f"params1-{kind}-0.pt")
        assert torch.allclose(first, torch.load(tmp_path / "params1-replicated-0.pt"), rtol=1e-4, atol=1e-6), kind
        assert_same_training(a, rep, 1e-3, 3, kind)
        assert reports[0][kind]["losses"] == pytest.approx(reports[0]["replicated"]["losses"], rel=1e-3), kind
    assert reports[0]["owned_matrix_elements"] * 2 == reports[0]["full_matrix_elements"]


@pytest.mark.gpu
def test_one_gpu_sharded_layout_matches_replicated():
    """World size 1 on a GPU: the gather + cast + GEMM launches, the landing slots and the segmented optimizer
    against the replicated trainer on the same data."""
    from warpstate_ai_b200.ops.gemm import check_device_errors
    from warpstate_ai_b200.train.engine import Trainer
    device = torch.device("cuda", 0)
    results = {}
    for kind, shard, ckpt in (("replicated", None, False), ("stream", "stream", False), ("resident", "resident", False),
                              ("stream-ckpt", "stream", True), ("replicated-ckpt", None, True)):
        model, cfg = tiny_model(device, checkpointing=ckpt)
        trainer = Trainer(model, device=device, lr=1e-3, weight_decay=0.1, shard_params=shard)
        losses = run_updates(trainer, cfg, 256, 2, [2 * 256 * 2, 2 * 256 * 2, 2 * 256])
        results[kind] = (losses, flat_state(trainer.model_state_dict()))
        check_device_errors()
    rep_losses, rep = results["replicated"]
    for kind in ("stream", "resident", "stream-ckpt", "replicated-ckpt"):
        losses, flat = results[kind]
        assert losses == pytest.approx(rep_losses, rel=1e-4), kind
        assert torch.allclose(flat, rep, rtol=1e-4, atol=1e-6), kind


@pytest.mark.gpu
@pytest.mark.parametrize("shard", [None, "stream"])
def test_gpu_update_is_skipped_on_nonfinite_norm_or_failed_exchange(shard):
    """The device gates the update: a non-finite norm, or a non-zero status word of the gradient exchange
    (set here on the host), leaves master weights, moments and the BF16 mirror as they were; the trainer raises
    when it reads the update's scalars."""
    from warpstate_ai_b200.train.engine import Trainer
    device = torch.device("cuda", 0)
    model, cfg = tiny_model(device)
    trainer = Trainer(model, device=device, lr=1e-3, weight_decay=0.1, shard_params=shard)
    run_updates(trainer, cfg, 256, 2, [2 * 256])
    opt = trainer.optimizer

    def snapshot():
        tensors = [trainer.arena.master, trainer.arena.bf16.float()]
        tensors += [opt.m_sh, opt.v_sh, opt.m_rep, opt.v_rep, trainer.sharded.master] if shard else [opt.exp_avg, opt.exp_avg_sq]
        return [t.detach().clone() for t in tensors], opt.step_count

    before, steps = snapshot()
    trainer.begin_update()
    trainer.arena.grad.normal_()
    trainer.arena.grad[5] = float("nan")
    stats = trainer.finish_update(1e-3)
    with pytest.raises(RuntimeError, match="non-finite"):
        trainer.read_update_scalars(stats)
    after, steps_after = snapshot()
    assert steps_after == steps and all(torch.equal(a, b) for a, b in zip(before, after))
    # a failed exchange: status word != 0 on the device
    status = torch.tensor([2, 0, 1, 5, 4, 0, 0, 0], dtype=torch.int32, device=device)
    trainer.arena.grad.normal_()
    stats = torch.ops.ws_b200.grad_norm_clip(trainer.arena.grad, 1.0, None, status)
    assert float(stats[3]) == 1.0 and float(stats[1]) == 0.0 and float(stats[0]) > 0
    opt.step(lr=1e-3, stats=stats)
    opt.rollback_step()
    after, steps_after = snapshot()
    assert steps_after == steps and all(torch.equal(a, b) for a, b in zip(before, after))
    # and a clean update still goes through
    trainer.arena.grad.normal_()
    opt.step(lr=1e-3, stats=torch.ops.ws_b200.grad_norm_clip(trainer.arena.grad, 1.0, None, None))
    assert not torch.equal(snapshot()[0][0], before[0])


if __name__ == "__main__":
    worker(sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), Path(sys.argv[4]))
