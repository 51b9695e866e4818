"""DPO post-training throughput of the 2.005 B model (trainable policy + frozen BF16 reference).

Synthetic workload: every example is a chosen / rejected pair sharing a random prompt of 256-1024
tokens; each response has 128-1024 uniform-random tokens; sequences are padded to ``--seq-len``
and only response tokens carry a label (prompt and padding are masked with -100).  Each rank
processes ``--pairs-per-gpu`` pairs per update in micro-batches of ``--micro-pairs`` pairs
(2 rows per pair).  The frozen reference is a BF16 copy resident on the same GPU and is scored
inside the update (the trainer's "resident" reference mode); beta 0.1.

The timed region is the trainer's own `training_update` (forward of the reference, forward /
backward of the policy through the fused kernels and the fused LM-head log-probabilities,
gradient synchronisation, clip, AdamW), device-synchronised on both sides, max over ranks.

    torchrun --nproc-per-node 8 -m warpstate_ai_b200.bench.dpo_bench --pairs-per-gpu 16

``--reference cached`` times this framework's update with precomputed reference scores (what the reference
framework always does: its frozen model is scored once into a cache, reference dpo.py:224-329, and the update
runs the policy only).  ``--impl reference`` runs the comparison arm on the same synthetic pairs: the unmodified
reference from ``baseline/_ref`` -- its ``dpo.load_model`` (compiled cores, per-sequence log-probability head,
BF16 residual views), its DDP wrap (reference dpo.py:490-493), fused AdamW and its own ``training_update``
(reference dpo.py:331-361) with cached reference scores.
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import time

import torch


def synthetic_pairs(pairs: int, seq_len: int, vocab: int, generator: torch.Generator):
    """(x, y) [2*pairs, seq_len] int64 with -100 outside the responses, rows 2i / 2i+1 = chosen / rejected."""
    x = torch.zeros(2 * pairs, seq_len, dtype=torch.long)
    y = torch.full((2 * pairs, seq_len), -100, dtype=torch.long)
    for i in range(pairs):
        prompt_len = int(torch.randint(256, 1025, (1,), generator=generator))
        prompt = torch.randint(0, vocab, (prompt_len,), generator=generator)
        for branch in range(2):
            response_len = int(torch.randint(128, 1025, (1,), generator=generator))
            response_len = min(response_len, seq_len + 1 - prompt_len)
            tokens = torch.cat([prompt, torch.randint(0, vocab, (response_len,), generator=generator)])
            n = tokens.numel() - 1
            row = 2 * i + branch
            x[row, :n] = tokens[:-1]
            y[row, prompt_len - 1:n] = tokens[prompt_len:]
    return x, y


def run_reference_arm(a, micro, global_pairs, world, rank, local, device):
    """Seconds per update of the reference's own DPO update, or a one-line reason why it cannot run."""
    import sys
    from pathlib import Path
    import torch.distributed as dist
    root = Path(__file__).resolve().parents[2]
    ref_root = root / "baseline" / "_ref"
    if not (ref_root / "dpo.py").exists():
        return None, "baseline/_ref is not installed"
    for name in [m for m in sys.modules if m in ("dpo", "posttrain", "run_40b", "ops") or m.startswith(("warpstate.", "ops."))
                 or m == "warpstate"]:
        del sys.modules[name]
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != root]
    sys.path.insert(0, str(ref_root))
    try:
        import dpo as ref_dpo
        from warpstate import WarpStateConfig, WarpStateLM
    except Exception as error:  # depends on the installed torch
        return None, f"import failed: {error!r}"[:300]
    assert "baseline/_ref" in str(Path(ref_dpo.__file__))
    if a.model == "2b":
        cfg = WarpStateConfig(vocab_size=32768, d_model=2048, n_heads=32, n_cores=28, logical_depth=28, ffn_hidden=7168,
                              chunk_size=128, dropout=0.0, rms_eps=1e-5, gradient_checkpointing=False,
                              parallel_memory=True, loss_chunk_size=128)
    else:
        cfg = WarpStateConfig(vocab_size=32768, d_model=256, n_heads=4, n_cores=2, logical_depth=4, ffn_hidden=688,
                              chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    torch.manual_seed(1337)
    with torch.device(device):
        seed_model = WarpStateLM(cfg)
    checkpoint = {"config": dict(vars(cfg)), "model": seed_model.state_dict()}
    settings = dict(ref_dpo.DEFAULTS, beta=a.beta, sequence_length=a.seq_len, micro_batch=a.micro_pairs, lr=5e-7)

    class Vocabulary:
        def vocab_size(self):
            return cfg.vocab_size

    raw, _ = ref_dpo.load_model(checkpoint, settings, device, Vocabulary())
    del seed_model, checkpoint
    raw.requires_grad_(True).train()
    optimizer = torch.optim.AdamW(raw.parameters(), lr=settings["lr"], betas=(0.9, 0.95), eps=1e-8,
                                  weight_decay=settings["weight_decay"], fused=True)
    model = raw
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(raw, device_ids=[local], broadcast_buffers=False,
                                                          gradient_as_bucket_view=True, bucket_cap_mb=128)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(a.warmup):
        values, norm = ref_dpo.training_update(model, optimizer, micro, global_pairs, world, device, settings)
    barrier()
    begin = time.perf_counter()
    for _ in range(a.steps):
        values, norm = ref_dpo.training_update(model, optimizer, micro, global_pairs, world, device, settings)
    barrier()
    elapsed = torch.tensor([time.perf_counter() - begin], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    return (float(elapsed) / a.steps, values, norm), None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--reference", choices=["resident", "cached"], default="resident",
                    help="ours: score the frozen BF16 reference inside the update, or use precomputed scores")
    ap.add_argument("--model", choices=["2b", "smoke"], default="2b")
    ap.add_argument("--pairs-per-gpu", type=int, default=16)
    ap.add_argument("--micro-pairs", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--beta", type=float, default=0.1)
    ap.add_argument("--device", choices=["cuda", "cpu"], default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--profile", action="store_true",
                    help="ours: after the timed updates, run one more under torch.profiler and print the kernels that "
                         "carry its device time (rank 0)")
    a = ap.parse_args(argv)
    if a.profile:
        os.environ.setdefault("WS_TRAIN_PDL", "0")   # dependents would book their in-kernel wait as their own time
    import torch.distributed as dist
    from .. import WarpStateLM, warpstate_2b, warpstate_smoke
    from ..train import dpo as DPO
    from ..train.engine import Trainer

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    if a.device == "cuda":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if a.device == "cuda" else "gloo", **({"device_id": device} if a.device == "cuda" else {}))
    cfg = warpstate_2b() if a.model == "2b" else warpstate_smoke()
    cfg.gradient_checkpointing = False
    gen = torch.Generator().manual_seed(7 + rank)
    micro = []
    for start in range(0, a.pairs_per_gpu, a.micro_pairs):
        pairs = min(a.micro_pairs, a.pairs_per_gpu - start)
        x, y = synthetic_pairs(pairs, a.seq_len, cfg.vocab_size, gen)
        micro.append((x.pin_memory() if a.device == "cuda" else x, y.pin_memory() if a.device == "cuda" else y,
                      torch.ones(pairs, dtype=torch.bool), torch.zeros(pairs, 2)))
    global_pairs = a.pairs_per_gpu * world
    tokens = sum(int(y.ne(-100).sum()) for _, y, _, _ in micro)
    if a.impl == "reference":
        outcome, why = run_reference_arm(a, micro, global_pairs, world, rank, local, device)
        if rank == 0:
            if outcome is None:
                print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
            else:
                seconds, values, norm = outcome
                print(json.dumps({"metric": "DPO pairs/sec (policy update, cached reference scores)", "impl": "reference",
                                  "value": global_pairs / seconds, "unit": "pairs/s", "n_gpus": world,
                                  "seconds_per_update": seconds, "pairs_per_gpu": a.pairs_per_gpu,
                                  "micro_pairs": a.micro_pairs, "seq_len": a.seq_len, "beta": a.beta,
                                  "response_tokens_per_gpu": tokens, "loss": values["loss"], "grad_norm": norm,
                                  "model": a.model, "peak_mem_gib": torch.cuda.max_memory_allocated(device) / 2 ** 30}),
                      flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0
    torch.manual_seed(1337)
    with torch.device(device):
        policy = WarpStateLM(cfg)
    reference = None
    if a.reference == "resident":
        reference = copy.deepcopy(policy).to(torch.bfloat16 if a.device == "cuda" else torch.float32)
        reference.requires_grad_(False).eval()
    policy.train()
    sync = None
    if world > 1:
        from ..parallel.grad_sync import make_grad_sync
        sync = make_grad_sync(device, world, rank, None)
    trainer = Trainer(policy, device=device, rank=rank, world_size=world, lr=5e-7, weight_decay=0.0, grad_sync=sync)
    settings = dict(DPO.DEFAULTS, beta=a.beta, sequence_length=a.seq_len, head_chunk_size=256)

    def sync_all():
        if world > 1:
            dist.barrier()
        if a.device == "cuda":
            torch.cuda.synchronize(device)

    values = None
    for _ in range(a.warmup):
        values, norm = DPO.training_update(trainer, micro, global_pairs, settings, 5e-7, resident=reference)
    sync_all()
    begin = time.perf_counter()
    for _ in range(a.steps):
        values, norm = DPO.training_update(trainer, micro, global_pairs, settings, 5e-7, resident=reference)
    sync_all()
    elapsed = torch.tensor([time.perf_counter() - begin], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    seconds = float(elapsed) / a.steps
    if a.profile and a.device == "cuda":
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as trace:
            DPO.training_update(trainer, micro, global_pairs, settings, 5e-7, resident=reference)
            torch.cuda.synchronize(device)
        if rank == 0:
            rows = sorted(trace.key_averages(), key=lambda e: -e.device_time_total)
            busy = sum(e.device_time_total for e in rows)
            print(json.dumps({"profiled_update_device_ms": busy / 1e3,
                              "kernels": [{"name": e.key[:90], "calls": e.count, "ms": round(e.device_time_total / 1e3, 2)}
                                          for e in rows[:25]]}), flush=True)
    if rank == 0:
        what = "policy + resident BF16 reference" if a.reference == "resident" else "policy update, cached reference scores"
        print(json.dumps({"metric": f"DPO pairs/sec ({what})", "impl": "ours", "value": global_pairs / seconds,
                          "unit": "pairs/s", "n_gpus": world, "seconds_per_update": seconds, "pairs_per_gpu": a.pairs_per_gpu,
                          "micro_pairs": a.micro_pairs, "seq_len": a.seq_len, "beta": a.beta,
                          "response_tokens_per_gpu": tokens, "padded_tokens_per_second": 2 * global_pairs * a.seq_len / seconds,
                          "loss": values["loss"], "grad_norm": norm, "model": a.model,
                          "peak_mem_gib": torch.cuda.max_memory_allocated(device) / 2 ** 30 if a.device == "cuda" else None}),
              flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
