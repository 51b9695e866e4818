"""Batched prefill + greedy decode benchmark (2.005 B model by default).

Protocol: a batch of prompts of uniform-random tokens is prefilled with the chunked memory scan,
then ``--new-tokens`` tokens are decoded greedily carrying only the fast/slow memory states and
the current chunk's K/V/U.  Reports decode tokens/s over the whole batch, p50 per-token latency
and prefill tokens/s as one JSON line.  The reference publishes no such number (its CLIs decode
at batch 1 with token-by-token prefill, chat.py:212-214).

    python -m warpstate_ai_b200.bench.decode_bench --batch 64 --prompt 2048 --new-tokens 512

Under ``torchrun`` every rank serves its own batch on its own GPU (decode carries no cross-sequence state, so
replicas are independent): the line printed by rank 0 then reports the sum of the ranks' tokens/s and the
slowest rank's latencies.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def combine_ranks(per_rank: list[dict]) -> dict:
    """Whole-job figures from per-rank results: throughputs add, latencies and times take the slowest rank."""
    return {"tokens_per_second": sum(r["tokens_per_second"] for r in per_rank),
            "prefill_tokens_per_second": sum(r["prefill_tokens_per_second"] for r in per_rank),
            "p50_latency_seconds": max(r["p50_latency_seconds"] for r in per_rank),
            "prefill_seconds": max(r["prefill_seconds"] for r in per_rank),
            "peak_mem_gib": max(r["peak_mem_gib"] for r in per_rank)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="2b", choices=["2b", "smoke"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="PyTorch/cuBLAS formulation of the step (the comparison arm)")
    args = ap.parse_args()
    from .. import WarpStateLM, warpstate_2b, warpstate_smoke
    from ..ops import _ext
    from ..serve.engine import DecodeEngine
    from ..serve.posttrain_chat import generate_batch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    cfg = warpstate_2b() if args.model == "2b" else warpstate_smoke()
    torch.manual_seed(0)          # the same weights on every rank
    with torch.device(device):
        model = WarpStateLM(cfg)
    model.eval().requires_grad_(False)
    engine = DecodeEngine(model, dtype=torch.bfloat16, use_cuda_graph=not args.no_graph, use_kernels=not args.no_kernels)
    torch.manual_seed(1 + rank)   # its own prompts
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt), device=device)
    generate_batch(engine, prompts[:, :256], 4)  # warm-up (graph capture, lazy initialisation)
    before = _ext.launch_count()
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()            # the replicas run at the same time, as they would in service
    result = generate_batch(engine, prompts, args.new_tokens)
    mine = {"tokens_per_second": result["tokens_per_second"], "p50_latency_seconds": result["p50_latency_seconds"],
            "prefill_tokens_per_second": args.batch * args.prompt / result["prefill_seconds"],
            "prefill_seconds": result["prefill_seconds"],
            "peak_mem_gib": torch.cuda.max_memory_allocated(device) / 2 ** 30}
    launches = _ext.launch_count() - before
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        total = combine_ranks(gathered)
    else:
        total = mine
    if rank != 0:
        dist.barrier()
        dist.destroy_process_group()
        return
    line = {"metric": "decode tokens/sec (greedy, batch lock-step)", "value": total["tokens_per_second"],
            "unit": "tokens/s", "n_gpus": world, "batch_per_gpu": args.batch, "batch": args.batch * world,
            "prompt_tokens": args.prompt, "new_tokens": args.new_tokens,
            "p50_token_latency_ms": total["p50_latency_seconds"] * 1e3,
            "prefill_tokens_per_second": total["prefill_tokens_per_second"],
            "prefill_seconds": total["prefill_seconds"], "cuda_graph": not args.no_graph,
            "own_kernel_launches": launches, "model": args.model, "dtype": "bf16",
            "peak_mem_gib": total["peak_mem_gib"]}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
