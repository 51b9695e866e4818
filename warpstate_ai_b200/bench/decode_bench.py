"""Batched prefill + greedy decode benchmark (2.005 B model by default).

Protocol: a batch of prompts of uniform-random tokens is prefilled with the chunked memory scan,
then ``--new-tokens`` tokens are decoded greedily carrying only the fast/slow memory states and
the current chunk's K/V/U.  Reports decode tokens/s over the whole batch, p50 per-token latency
and prefill tokens/s as one JSON line.  The reference publishes no such number (its CLIs decode
at batch 1 with token-by-token prefill, chat.py:212-214).

    python -m warpstate_ai_b200.bench.decode_bench --batch 64 --prompt 2048 --new-tokens 512
"""
from __future__ import annotations

import argparse
import json

import torch


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

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    cfg = warpstate_2b() if args.model == "2b" else warpstate_smoke()
    torch.manual_seed(0)
    with torch.device(device):
        model = WarpStateLM(cfg)
    model.eval().requires_grad_(False)
    engine = DecodeEngine(model, dtype=torch.bfloat16, use_cuda_graph=not args.no_graph, use_kernels=not args.no_kernels)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt), device=device)
    generate_batch(engine, prompts[:, :256], 4)  # warm-up (graph capture, lazy initialisation)
    before = _ext.launch_count()
    result = generate_batch(engine, prompts, args.new_tokens)
    line = {"metric": "decode tokens/sec (greedy, batch lock-step)", "value": result["tokens_per_second"],
            "unit": "tokens/s", "batch": args.batch, "prompt_tokens": args.prompt, "new_tokens": args.new_tokens,
            "p50_token_latency_ms": result["p50_latency_seconds"] * 1e3,
            "prefill_tokens_per_second": args.batch * args.prompt / result["prefill_seconds"],
            "prefill_seconds": result["prefill_seconds"], "cuda_graph": not args.no_graph,
            "own_kernel_launches": _ext.launch_count() - before, "model": args.model, "dtype": "bf16",
            "peak_mem_gib": torch.cuda.max_memory_allocated(device) / 2 ** 30}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
