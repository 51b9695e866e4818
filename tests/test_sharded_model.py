"""WarpState with row-sharded projection weights (`parallel/sharded_model.py`).

Two gloo ranks on CPU, each with half of the batch and half of every projection's rows, must train to the
same weights as one process that holds everything (same layer code with world 1): ownership, gather on
first use, gradient scatter to the owners, owner-only AdamW, all-reduce of the replicated gradients and the
unsharded state dict are what differ between the two runs.  A checkpoint written by the two ranks after one
update (unsharded weights and Adam moments) resumes on ONE rank to the weights of the uninterrupted run.
The file doubles as the worker.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]


def build(seed: int = 0):
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    torch.manual_seed(seed)
    cfg = WarpStateConfig(vocab_size=64, d_model=32, n_heads=2, n_cores=2, logical_depth=3, ffn_hidden=48,
                          chunk_size=8, gradient_checkpointing=False, parallel_memory=True)
    return WarpStateLM(cfg), cfg


def train(rank: int, world: int, group=None, updates: int = 2, first: int = 0, resume: dict | None = None,
          want_optimizer: bool = False):
    from warpstate_ai_b200.parallel.sharded_linear import ShardedRowsAdamW
    from warpstate_ai_b200.parallel.sharded_model import (allreduce_replicated_grads, gather_state_dict,
                                                          replicated_parameters, shard_core_linears, sharded_bytes)
    model, cfg = build()
    dense_keys = set(model.state_dict().keys())
    if resume is not None:
        model.load_state_dict(resume["model"])      # the unsharded checkpoint, then shard for this world size
    layers = shard_core_linears(model, rank, world, group, symmetric=False)
    assert len(layers) == 4 * cfg.n_cores and model.sharded_linears
    rows_opt = ShardedRowsAdamW(layers, lr=1e-2, weight_decay=0.1)
    rest_opt = torch.optim.AdamW(replicated_parameters(model), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    if resume is not None:
        rows_opt.load_state(resume["rows_optimizer"])
        rest_opt.load_state_dict(resume["rest_optimizer"])
    torch.manual_seed(7)
    tokens = torch.randint(0, cfg.vocab_size, (2, 4, 17))
    per = 4 // world
    losses = []
    for step in range(first, first + updates):
        batch = tokens[step, rank * per:(rank + 1) * per]
        x, y = batch[:, :-1], batch[:, 1:]
        rows_opt.zero_grad()
        rest_opt.zero_grad()
        _, loss = model(x, y, return_logits=False)
        (loss / world).backward()           # equal token counts per rank: the sum over ranks is the global mean
        allreduce_replicated_grads(model, group)
        rows_opt.step()
        rest_opt.step()
        losses.append(float(loss.detach()))
    state = gather_state_dict(model, group)
    assert set(state.keys()) == dense_keys, sorted(set(state.keys()) ^ dense_keys)
    if want_optimizer:
        return {"model": state, "rows_optimizer": rows_opt.gather_state(group), "rest_optimizer": rest_opt.state_dict()}
    return state, losses, sharded_bytes(layers)


def worker(rank: int, world: int, out_dir: Path) -> None:
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=(out_dir / "rendezvous").as_uri(), rank=rank, world_size=world)
    state, losses, held = train(rank, world)
    if rank == 0:
        torch.save(state, out_dir / "state.pt")
    (out_dir / f"report-{rank}.json").write_text(json.dumps({"losses": losses, "held": held}))
    checkpoint = train(rank, world, updates=1, want_optimizer=True)   # one update, then an unsharded checkpoint
    if rank == 0:
        torch.save(checkpoint, out_dir / "checkpoint.pt")
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_with_sharded_projections_match_one_process(tmp_path):
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    env["CUDA_VISIBLE_DEVICES"] = ""
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
    whole, losses, held_whole = train(0, 1)
    split = torch.load(tmp_path / "state.pt")
    for key, value in whole.items():
        assert torch.allclose(split[key], value, rtol=1e-4, atol=1e-4), key
    reports = [json.loads((tmp_path / f"report-{r}.json").read_text()) for r in range(2)]
    # the two ranks' local losses average to the one-process loss
    for step, ref in enumerate(losses):
        assert abs(0.5 * (reports[0]["losses"][step] + reports[1]["losses"][step]) - ref) < 1e-4
    # each rank holds half of the FP32 master rows (row counts are rounded up to multiples of 8)
    assert reports[0]["held"]["master_rows"] <= held_whole["master_rows"] // 2 + 4 * 8 * 48 * 8
    assert reports[0]["held"]["master_rows"] < 0.6 * held_whole["master_rows"]
    # world-size change on resume: the two-rank checkpoint after one update continues on one rank to the
    # weights of the uninterrupted run
    checkpoint = torch.load(tmp_path / "checkpoint.pt")
    assert checkpoint["rows_optimizer"]["steps"] == 1
    resumed, _, _ = train(0, 1, updates=1, first=1, resume=checkpoint)
    for key, value in whole.items():
        assert torch.allclose(resumed[key], value, rtol=1e-4, atol=1e-4), key


if __name__ == "__main__":
    worker(int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3]))
