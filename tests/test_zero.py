"""Sharded optimizer state (`parallel/zero.py`, ZeRO stage 1) on the CPU: ownership, equality with the replicated
optimizer, and the unsharded checkpoint form.

The file doubles as the worker of its two-rank case (gloo, file-store rendezvous; the pattern of the reference's
test_distributed_execution.py:78-177).  Both ranks hold the same averaged gradient, as after the all-reduce; each
updates only the slices it owns and the ranks exchange them.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def tiny_model():
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=96, d_model=32, n_heads=4, n_cores=2, logical_depth=2, ffn_hidden=48, chunk_size=8,
                          gradient_checkpointing=False, parallel_memory=True)
    return WarpStateLM(cfg)


def gradient(arena, step):
    """The same flat gradient on every rank; the alignment padding between parameters stays zero, as in a real run."""
    g = torch.Generator().manual_seed(100 + step)
    noise = torch.randn(arena.numel, generator=g) * (10.0 if step == 1 else 0.01)       # the second step gets clipped
    flat = torch.zeros(arena.numel)
    for slot in arena.slots:
        flat[slot.offset:slot.offset + slot.numel] = noise[slot.offset:slot.offset + slot.numel]
    return flat


def replicated_run(steps):
    from warpstate_ai_b200.optim import ArenaAdamW, ParamArena
    arena = ParamArena(tiny_model(), bf16_mirror=True)
    opt = ArenaAdamW(arena, lr=1e-2, weight_decay=0.1)
    norms = []
    for step in range(steps):
        arena.grad.copy_(gradient(arena, step))
        norms.append(float(opt.step()[0]))
    return arena, opt, norms


# ------------------------------------------------------------------------------------------- ownership
@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("start, stop", [(0, 256), (256, 256 + 4 * 7), (1024, 1024 + 4 * 1000), (0, 4), (512, 512)])
def test_every_bucket_is_split_into_disjoint_float4_aligned_slices(world, start, stop):
    from warpstate_ai_b200.parallel.zero import bucket_slice
    slices = [bucket_slice(start, stop, rank, world) for rank in range(world)]
    position = start
    for lo, hi in slices:
        assert lo == position and lo <= hi and (lo - start) % 4 == 0 and (hi - start) % 4 == 0
        position = hi
    assert position == stop
    sizes = [hi - lo for lo, hi in slices]
    assert max(sizes) - min(s for s in sizes if s or True) <= max(sizes)               # later ranks may own nothing
    assert sizes == sorted(sizes, reverse=True) and max(sizes) == 4 * -(-((stop - start) // 4) // world)


def test_one_rank_owns_everything_and_matches_the_replicated_optimizer_bit_for_bit():
    from warpstate_ai_b200.optim import ParamArena
    from warpstate_ai_b200.parallel.zero import ShardedAdamW
    reference_arena, reference_opt, norms = replicated_run(3)
    arena = ParamArena(tiny_model(), bf16_mirror=True)
    opt = ShardedAdamW(arena, rank=0, world=1, lr=1e-2, weight_decay=0.1)
    assert opt.ranges == [(b.start, b.stop) for b in arena.buckets] and not opt.fused
    for step in range(3):
        arena.grad.copy_(gradient(arena, step))
        stats = opt.step()
        assert float(stats[0]) == pytest.approx(norms[step], rel=1e-6)
    assert torch.equal(arena.master, reference_arena.master) and torch.equal(arena.bf16, reference_arena.bf16)
    mine, theirs = opt.state_dict(), reference_opt.state_dict()
    assert mine["param_groups"] == theirs["param_groups"] and set(mine["state"]) == set(theirs["state"])
    for index, entry in theirs["state"].items():
        assert all(torch.equal(mine["state"][index][k], entry[k]) for k in ("step", "exp_avg", "exp_avg_sq"))


def test_the_update_matches_torch_adamw_with_global_norm_clipping():
    arena, opt, norms = replicated_run(3)
    model = tiny_model()
    torch_opt = torch.optim.AdamW(model.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    from warpstate_ai_b200.optim import ParamArena
    layout = ParamArena(tiny_model(), bf16_mirror=False)
    for step in range(3):
        flat = gradient(layout, step)
        for name, p in model.named_parameters():
            slot = layout.by_name[name]
            p.grad = flat[slot.offset:slot.offset + slot.numel].view(slot.shape).clone()
        norm = torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        assert float(norm) == pytest.approx(norms[step], rel=1e-5)
        torch_opt.step()
    for name, p in model.named_parameters():
        slot = arena.by_name[name]
        torch.testing.assert_close(arena.master[slot.offset:slot.offset + slot.numel].view(slot.shape), p.detach(),
                                   rtol=1e-5, atol=1e-7)


def test_a_skipped_update_changes_nothing_and_gives_its_step_back():
    from warpstate_ai_b200.optim import ParamArena
    from warpstate_ai_b200.parallel.zero import ShardedAdamW
    arena = ParamArena(tiny_model(), bf16_mirror=True)
    opt = ShardedAdamW(arena, rank=0, world=1, lr=1e-2)
    arena.grad.copy_(gradient(arena, 0))
    opt.step()
    before = (arena.master.clone(), opt.exp_avg.clone(), opt.exp_avg_sq.clone(), opt.step_count)
    arena.grad.copy_(gradient(arena, 1))
    arena.grad[5] = float("nan")
    stats = opt.step()
    assert float(stats[3]) == 1.0 and float(stats[1]) == 0.0                             # skip flag set, coefficient zero
    opt.rollback_step()
    assert torch.equal(arena.master, before[0]) and torch.equal(opt.exp_avg, before[1]) and torch.equal(opt.exp_avg_sq, before[2])
    assert opt.step_count == before[3]
    status = torch.tensor([3], dtype=torch.int32)                                       # the gradient exchange gave up
    arena.grad.copy_(gradient(arena, 1))
    assert float(opt.clip_stats(status=status)[3]) == 1.0


# ------------------------------------------------------------------------------------------- two ranks (gloo)
def test_two_ranks_own_half_the_moments_and_end_where_one_rank_does(tmp_path):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    procs = [subprocess.Popen([sys.executable, __file__, str(rank), "2", str(tmp_path)], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for rank in range(2)]
    outputs = []
    for p in procs:
        try:
            outputs.append(p.communicate(timeout=240)[0])
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
    for rank, p in enumerate(procs):
        assert p.returncode == 0, f"rank {rank} failed:\n{outputs[rank][-3000:]}"
    reports = [json.loads((tmp_path / f"report-{rank}.json").read_text()) for rank in range(2)]
    for report in reports:
        assert report["master_equal"] and report["mirror_equal"] and report["state_equal"] and report["reloaded_equal"]
        assert report["norms"] == pytest.approx(reports[0]["norms"], rel=1e-6)
        assert report["resumed_equal"]
    owned = [r["owned_elements"] for r in reports]
    assert sum(owned) == reports[0]["arena_elements"] and abs(owned[0] - owned[1]) <= 4 * reports[0]["buckets"]
    assert reports[0]["memory_bytes"] == 8 * owned[0]


def worker(rank: int, world: int, directory: Path) -> None:
    import torch.distributed as dist
    from warpstate_ai_b200.optim import ParamArena
    from warpstate_ai_b200.parallel.zero import ShardedAdamW
    dist.init_process_group("gloo", init_method=(directory / "rendezvous").as_uri(), rank=rank, world_size=world)
    reference_arena, reference_opt, norms = replicated_run(3)
    arena = ParamArena(tiny_model(), bf16_mirror=True)
    opt = ShardedAdamW(arena, rank=rank, world=world, lr=1e-2, weight_decay=0.1)
    mine = []
    for step in range(3):
        arena.grad.copy_(gradient(arena, step))
        mine.append(float(opt.step()[0]))
    state = opt.state_dict()                                                             # collective: gathers the moments
    wanted = reference_opt.state_dict()
    # equal to the one-rank optimizer up to the last bit of the clip coefficient (the norm's FP64 partial sums are
    # added in another order), which is far inside these bounds
    def close(a, b):
        return bool(torch.allclose(a, b, rtol=1e-6, atol=1e-9))

    state_equal = state["param_groups"] == wanted["param_groups"] and all(
        close(state["state"][i][k], wanted["state"][i][k]) for i in wanted["state"] for k in ("step", "exp_avg", "exp_avg_sq"))
    # a fresh sharded optimizer loads the unsharded state and holds the same slices again
    again = ShardedAdamW(ParamArena(tiny_model(), bf16_mirror=True), rank=rank, world=world)
    again.load_state_dict(wanted)
    reloaded_equal = (torch.equal(again.exp_avg, opt.exp_avg) and torch.equal(again.exp_avg_sq, opt.exp_avg_sq)
                      and again.step_count == 3 and again.lr == 1e-2 and again.weight_decay == 0.1)
    # and continues exactly like the run that never stopped
    again.arena.master.copy_(arena.master)
    again.arena.refresh_bf16()
    for o in (opt, again):
        o.arena.grad.copy_(gradient(o.arena, 3))
        o.step()
    resumed_equal = torch.equal(again.arena.master, arena.master) and torch.equal(again.exp_avg, opt.exp_avg)
    reference_arena_3 = reference_arena.master.clone()
    report = dict(master_equal=True, mirror_equal=True, state_equal=state_equal, reloaded_equal=reloaded_equal,
                  resumed_equal=resumed_equal, norms=mine, owned_elements=sum(hi - lo for lo, hi in opt.ranges),
                  arena_elements=arena.numel, buckets=len(arena.buckets), memory_bytes=opt.memory_bytes())
    # compare against the replicated run advanced by the same fourth step
    reference_arena.grad.copy_(gradient(reference_arena, 3))
    reference_opt.step()
    report["master_equal"] = close(arena.master, reference_arena.master) and not torch.equal(arena.master, reference_arena_3)
    report["mirror_equal"] = float((arena.bf16.float() - reference_arena.bf16.float()).abs().max()) <= 2 ** -7 * float(
        reference_arena.bf16.float().abs().max())
    report["bitwise"] = bool(torch.equal(arena.master, reference_arena.master))
    assert mine == pytest.approx(norms, rel=1e-6)
    (directory / f"report-{rank}.json").write_text(json.dumps(report))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    worker(int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3]))
