"""Batched prefill + greedy decode benchmark (2.005 B model by default).

Protocol: a batch of prompts of uniform-random tokens is prefilled with the chunked memory scan,
then ``--new-tokens`` tokens are decoded greedily carrying only the fast/slow memory states and
the current chunk's K/V/U.  Reports decode tokens/s over the whole batch, p50 per-token latency
and prefill tokens/s as one JSON line.  The reference publishes no such number (its CLIs decode
at batch 1 with token-by-token prefill, chat.py:212-214).

    python -m warpstate_ai_b200.bench.decode_bench --batch 64 --prompt 2048 --new-tokens 512

``--impl reference`` runs the comparison arm: the unmodified reference model from ``baseline/_ref`` decoding the
same batch with its own ``WarpStateLM.step`` (reference warpstate/model.py:349-358) under BF16 autocast, prompt fed
token by token as its chat tools do (reference chat.py:212-214, ops/posttrain_chat.py:199-201).

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
            "peak_mem_gib": max(r["peak_mem_gib"] for r in per_rank),
            "host_driven_p50_seconds": max(r["host_driven_p50_seconds"] for r in per_rank)}


def reference_generate_batch(model, prompts: torch.Tensor, new_tokens: int) -> dict:
    """The reference's decode: ``model.step`` one token at a time for prompt and continuation alike."""
    import time
    device = prompts.device
    batch = prompts.shape[0]
    caches = model.init_generation_cache(batch, device, torch.bfloat16)
    latencies, columns = [], []
    with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
        torch.cuda.synchronize(device)
        mark = time.perf_counter()
        for t in range(prompts.shape[1]):
            logits = model.step(prompts[:, t:t + 1], caches)
        torch.cuda.synchronize(device)
        prefill_seconds = time.perf_counter() - mark
        token = logits[:, -1].argmax(dim=-1)
        for _ in range(new_tokens):
            columns.append(token)
            mark = time.perf_counter()
            token = model.step(token.view(batch, 1), caches)[:, -1].argmax(dim=-1)
            torch.cuda.synchronize(device)
            latencies.append(time.perf_counter() - mark)
    total = sum(latencies)
    return {"tokens": torch.stack(columns, dim=1), "prefill_seconds": prefill_seconds, "decode_seconds": total,
            "tokens_per_second": batch * new_tokens / total, "latencies": latencies,
            "p50_latency_seconds": sorted(latencies)[len(latencies) // 2]}


def load_reference_model(model_name: str, device):
    """The reference's own `WarpStateLM` (imported from ``baseline/_ref``), random-initialised."""
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[2]
    ref_root = root / "baseline" / "_ref"
    if not (ref_root / "warpstate" / "model.py").exists():
        return None
    for name in [m for m in sys.modules if m == "warpstate" or m.startswith("warpstate.")]:
        del sys.modules[name]
    sys.path.insert(0, str(ref_root))
    from warpstate import WarpStateConfig, WarpStateLM  # the reference package
    assert "baseline/_ref" in str(Path(sys.modules["warpstate"].__file__))
    if model_name == "2b":
        cfg = WarpStateConfig(vocab_size=32768, d_model=2048, n_heads=32, n_cores=28, logical_depth=28, ffn_hidden=7168,
                              chunk_size=128, dropout=0.0, rms_eps=1e-5, gradient_checkpointing=False,
                              parallel_memory=True, loss_chunk_size=128)
    else:
        cfg = WarpStateConfig(vocab_size=32768, d_model=256, n_heads=4, n_cores=2, logical_depth=4, ffn_hidden=688,
                              chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    torch.manual_seed(0)
    with torch.device(device):
        model = WarpStateLM(cfg)
    return model.to(device).eval().requires_grad_(False), cfg


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
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
    if args.impl == "reference":
        loaded = load_reference_model(args.model, device)
        if loaded is None:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}), flush=True)
            return
        ref_model, cfg = loaded
        torch.manual_seed(1 + rank)
        prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt), device=device)
        reference_generate_batch(ref_model, prompts[:, :8], 4)   # warm-up
        before = _ext.launch_count()
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
        result = reference_generate_batch(ref_model, prompts, args.new_tokens)
    else:
        cfg = warpstate_2b() if args.model == "2b" else warpstate_smoke()
        torch.manual_seed(0)          # the same weights on every rank
        with torch.device(device):
            model = WarpStateLM(cfg)
        model.eval().requires_grad_(False)
        engine = DecodeEngine(model, dtype=torch.bfloat16, use_cuda_graph=not args.no_graph,
                              use_kernels=not args.no_kernels)
        torch.manual_seed(1 + rank)   # its own prompts
        prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt), device=device)
        generate_batch(engine, prompts[:, :256], 4)  # warm-up (graph capture, lazy initialisation)
        before = _ext.launch_count()
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()            # the replicas run at the same time, as they would in service
        from ..serve.graph_stats import collect_graph_diagnostics
        with collect_graph_diagnostics(engine) as diagnostics:
            result = generate_batch(engine, prompts, args.new_tokens)
        graph_report = diagnostics.snapshot()
        # the same engine driven token by token from the host (arg-max on the host stream, one synchronisation per
        # token, wall clock): what a caller that inspects every token before asking for the next one sees
        host_driven = generate_batch(engine, prompts[:, :256], 64, synchronous=True)["p50_latency_seconds"]
    mine = {"tokens_per_second": result["tokens_per_second"], "p50_latency_seconds": result["p50_latency_seconds"],
            "prefill_tokens_per_second": args.batch * args.prompt / result["prefill_seconds"],
            "prefill_seconds": result["prefill_seconds"],
            "peak_mem_gib": torch.cuda.max_memory_allocated(device) / 2 ** 30,
            "host_driven_p50_seconds": host_driven if args.impl == "ours" else result["p50_latency_seconds"]}
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
            "latency_timing": result.get("timing", "host clock, one synchronisation per token"),
            "p50_token_latency_ms_host_driven": total["host_driven_p50_seconds"] * 1e3,
            "prefill_tokens_per_second": total["prefill_tokens_per_second"],
            "prefill_seconds": total["prefill_seconds"], "cuda_graph": not args.no_graph,
            "own_kernel_launches": launches, "cuda_graph_diagnostics": graph_report if args.impl == "ours" else None,
            "model": args.model, "dtype": "bf16", "impl": args.impl,
            "peak_mem_gib": total["peak_mem_gib"]}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
