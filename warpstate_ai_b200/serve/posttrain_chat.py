"""Chat with SFT / DPO snapshots (GPU BF16 compute over FP32 masters, or CPU FP32).

Prompt rendering mirrors the SFT renderer and ends right after an assistant header
(reference ops/posttrain_chat.py:35-65); `generate` returns the reference's result record
(response, token ids, prompt / generated token counts, elapsed, time to first token, tokens/s,
stop reason); `--prompts-json` runs a batch prompt suite into an atomic JSON report
(``warpstate-posttrain-generation-v1``, :365-389).

Unlike the reference (token-by-token prefill, batch hard-wired to 1), the prompt is prefilled in
whole chunks through the training kernels and a suite can be decoded as one lock-step batch with
``--batch`` when its prompts have equal token counts; the default stays one prompt at a time.
"""
from __future__ import annotations

import argparse
import json
import math
import time
from pathlib import Path

import torch

from ..data.sft import RENDER_FORMAT, ROLES, renderer_sha256
from ..utils.io import atomic_json, digest
from .chat import load_model
from .engine import DecodeEngine
from .sampling import sample_token


def encode_prompt(messages, tokenizer) -> list[int]:
    if not isinstance(messages, list) or not messages:
        raise ValueError("Prompt requires nonempty messages")
    if not isinstance(messages[-1], dict) or messages[-1].get("role") not in ("user", "tool"):
        raise ValueError("The conditioning conversation must end in a user/tool message")
    vocab, eos, bos = tokenizer.vocab_size(), tokenizer.eos_id(), tokenizer.bos_id()
    if not 0 <= eos < vocab:
        raise ValueError("Tokenizer requires a real EOS token")
    ids = [bos] if 0 <= bos < vocab else []

    def piece(text):
        encoded = tokenizer.encode(text, out_type=int)
        if any(type(t) is not int or not 0 <= t < vocab for t in encoded):
            raise ValueError("Tokenizer returned invalid token IDs")
        ids.extend(encoded)

    for message in messages:
        if not isinstance(message, dict) or message.get("role") not in ROLES:
            raise ValueError("Unsupported prompt role")
        if not isinstance(message.get("content"), str) or not message["content"].strip():
            raise ValueError("Messages require nonempty text content")
        if message.get("tool_calls"):
            raise ValueError("Tool calls must be serialized into message content")
        piece(f"<|{message['role']}|>\n")
        piece(message["content"])
        if message["role"] == "assistant":
            ids.append(eos)
        piece("\n")
    piece("<|assistant|>\n")
    return ids


@torch.inference_mode()
def generate(engine: DecodeEngine, tokenizer, messages, *, max_new_tokens=256, max_context=2048, temperature=0.0,
             seed=42, on_token=None) -> dict:
    if type(max_new_tokens) is not int or max_new_tokens < 1:
        raise ValueError("max_new_tokens must be positive")
    if type(max_context) is not int or max_context < 2:
        raise ValueError("max_context must exceed one token")
    if not math.isfinite(temperature) or temperature < 0 or type(seed) is not int or seed < 0:
        raise ValueError("Temperature and seed must be nonnegative")
    ids = encode_prompt(messages, tokenizer)
    if len(ids) >= max_context:
        raise ValueError(f"Prompt has {len(ids)} tokens; context limit is {max_context}")
    limit = min(max_new_tokens, max_context - len(ids))
    device = engine.device
    generator = torch.Generator(device="cpu").manual_seed(seed)
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    begin = time.perf_counter()
    logits = engine.prefill(torch.tensor([ids], dtype=torch.long, device=device))[0]
    generated, first = [], None
    stop_reason = "context_limit" if limit < max_new_tokens else "length"
    sampled = 0
    for index in range(limit):
        value = sample_token(logits.cpu(), temperature, 0, 1.0, generator)
        sampled += 1
        if first is None:
            first = time.perf_counter() - begin
        if value == tokenizer.eos_id():
            stop_reason = "eos"
            break
        if value is None:
            raise RuntimeError("No legal continuation token")
        generated.append(value)
        if on_token is not None:
            on_token(tuple(generated))
        if index + 1 < limit:
            logits = engine.step(torch.tensor([value], device=device))[0]
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    elapsed = time.perf_counter() - begin
    return dict(response=tokenizer.decode(generated), token_ids=generated, prompt_tokens=len(ids),
                generated_tokens=len(generated), sampled_tokens=sampled, elapsed_seconds=elapsed,
                first_token_seconds=first, tokens_per_second=len(generated) / elapsed, stop_reason=stop_reason,
                temperature=temperature, seed=seed)


@torch.inference_mode()
def generate_batch(engine: DecodeEngine, prompts: torch.Tensor, max_new_tokens: int, eos_id: int | None = None) -> dict:
    """Greedy lock-step decode of a batch of equal-length prompts ``[B, T]``.  Returns token ids
    ``[B, n]``, tokens/s over the decode phase and per-token latencies (seconds)."""
    device = engine.device
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    logits = engine.prefill(prompts)
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    prefill_seconds = time.perf_counter() - t0
    out, latencies = [], []
    token = logits.argmax(dim=-1)
    for _ in range(max_new_tokens):
        out.append(token)
        t1 = time.perf_counter()
        logits = engine.step(token)
        token = logits.argmax(dim=-1)
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        latencies.append(time.perf_counter() - t1)
    tokens = torch.stack(out, dim=1)
    decode_seconds = sum(latencies)
    return dict(tokens=tokens, prefill_seconds=prefill_seconds, decode_seconds=decode_seconds,
                tokens_per_second=tokens.numel() / decode_seconds, latencies=latencies,
                p50_latency_seconds=sorted(latencies)[len(latencies) // 2])


def read_prompts(path):
    value = json.loads(Path(path).read_text())
    rows = value.get("prompts") if isinstance(value, dict) else value
    if not isinstance(rows, list) or not rows:
        raise ValueError("Prompt suite must be a nonempty list or an object with prompts")
    seen = set()
    for index, row in enumerate(rows):
        if not isinstance(row, dict) or not isinstance(row.get("prompt"), str) or not row["prompt"].strip():
            raise ValueError(f"Invalid prompt suite row {index}")
        identity = row.get("id", str(index))
        if not isinstance(identity, (str, int)) or identity in seen:
            raise ValueError("Prompt suite IDs must be distinct strings or integers")
        seen.add(identity)
    return rows


def conversation(prompt: str, system: str):
    prefix = [{"role": "system", "content": system}] if system.strip() else []
    return prefix + [{"role": "user", "content": prompt}]


def interactive_chat(reply, messages, *, seed) -> int:
    history = []
    print("Enter a message; Ctrl-C cancels input/reply, /reset clears history, /quit exits.", flush=True)
    while True:
        try:
            prompt = input("You: ").strip()
            if prompt in ("/quit", "/exit"):
                break
            if prompt == "/reset":
                history = []
                continue
            if not prompt:
                continue
            turn = history + [{"role": "user", "content": prompt}] if history else messages(prompt)
            try:
                result = reply(turn, seed=seed)
            except ValueError as error:
                print(f"{error}; use /reset to start a new conversation.", flush=True)
                continue
            if result["response"].strip():
                history = turn + [{"role": "assistant", "content": result["response"]}]
        except KeyboardInterrupt:
            print("\nCancelled.", flush=True)
        except EOFError:
            print()
            break
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="Chat with a WarpState SFT/DPO snapshot")
    p.add_argument("--snapshot", type=Path, required=True)
    p.add_argument("--tokenizer", type=Path, help="defaults to tokenizer.model beside the snapshot")
    p.add_argument("--device", default="cuda:0")
    mode = p.add_mutually_exclusive_group()
    mode.add_argument("--prompt")
    mode.add_argument("--prompts-json", type=Path)
    p.add_argument("--output-json", type=Path)
    p.add_argument("--system", default="You are a helpful assistant.")
    p.add_argument("--max-new-tokens", type=int, default=256)
    p.add_argument("--max-context", type=int, default=2048)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--threads", type=int, default=8)
    args = p.parse_args(argv)
    try:
        snapshot = args.snapshot.expanduser().resolve()
        tokenizer = (args.tokenizer or snapshot.with_name("tokenizer.model")).expanduser().resolve()
        rows = read_prompts(args.prompts_json) if args.prompts_json else None
        if args.prompt is not None:
            if not args.prompt.strip():
                raise ValueError("Prompt cannot be empty")
            rows = [dict(id="prompt", prompt=args.prompt)]
        output = args.output_json.expanduser().resolve() if args.output_json else None
        if output is not None and (rows is None or output.exists() or output.is_relative_to(snapshot.parent)):
            raise ValueError("Select a new report file outside the snapshot directory")
        device = torch.device(args.device)
        if args.threads < 1 or not 0 < args.max_new_tokens < args.max_context:
            raise ValueError("Require threads >= 1 and 0 < max_new_tokens < max_context")
        if not math.isfinite(args.temperature) or args.temperature < 0 or args.seed < 0:
            raise ValueError("Temperature and seed must be nonnegative")
        torch.set_num_threads(args.threads)
        print(f"Loading sealed snapshot {snapshot}", flush=True)
        model, sp, metadata = load_model(snapshot, tokenizer, str(device))
        engine = DecodeEngine(model, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
    except (OSError, ValueError, RuntimeError) as error:
        p.error(str(error))
    print(f"{metadata.get('stage', 'posttrain')} step {metadata['step']:,} | {model.num_parameters() / 1e9:.3f}B | "
          f"{device}", flush=True)

    def reply(turn, *, seed):
        result = generate(engine, sp, turn, max_new_tokens=args.max_new_tokens, max_context=args.max_context,
                          temperature=args.temperature, seed=seed)
        print(result["response"], flush=True)
        print(f"[{result['generated_tokens']} tokens; {result['elapsed_seconds']:.2f}s; "
              f"stop={result['stop_reason']}]", flush=True)
        return result

    if rows is not None:
        report = dict(format="warpstate-posttrain-generation-v1", snapshot=str(snapshot),
                      snapshot_sha256=json.loads(snapshot.with_name("snapshot.json").read_text())["snapshot_sha256"],
                      metadata=metadata, tokenizer_sha256=digest(tokenizer), renderer_format=RENDER_FORMAT,
                      renderer_sha256=renderer_sha256(), inference_sha256=digest(__file__), device=str(device),
                      compute_dtype=str(engine.dtype), parameter_dtype="float32", max_context=args.max_context,
                      max_new_tokens=args.max_new_tokens, complete=False, results=[])
        if output:
            output.parent.mkdir(parents=True, exist_ok=True)
        for index, row in enumerate(rows):
            identity = row.get("id", str(index))
            system = row.get("system", args.system)
            print(f"\n[{identity}] {row['prompt']}", flush=True)
            result = reply(conversation(row["prompt"], system), seed=args.seed + index)
            report["results"].append(dict(id=identity, prompt=row["prompt"], system=system, **result))
            if output:
                atomic_json(output, report)
        report["complete"] = True
        if output:
            atomic_json(output, json.loads(json.dumps(report, default=str)))
            print(f"Results saved: {output}", flush=True)
        return 0
    return interactive_chat(reply, lambda prompt: conversation(prompt, args.system), seed=args.seed)


if __name__ == "__main__":
    raise SystemExit(main())
