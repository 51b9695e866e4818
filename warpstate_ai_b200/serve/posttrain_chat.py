"""Chat with SFT / DPO snapshots (GPU: BF16 compute over FP32 masters; CPU: FP32).

Covers the reference's post-training chat tool (reference ops/posttrain_chat.py: prompt encoding
:35-65, generation :68-238, prompt suites and the ``warpstate-posttrain-generation-v1`` report
:365-389) with this framework's serving stack: the prompt is prefilled in whole chunks through the
training kernels and decoded by `DecodeEngine`; a batch of equal-length prompts can be decoded in
lock step (`generate_batch`), which the reference (batch fixed at one, prompt fed token by token)
cannot do.

Pieces: `PromptEncoder` (the SFT renderer plus the open assistant header), `Generation` (one reply
and its timings), `PromptSuite` (validated list of prompts -> report file), `Conversation`
(interactive history).
"""
from __future__ import annotations

import argparse
import json
import math
import time
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..data.sft import RENDER_FORMAT, _Builder, check_message, renderer_sha256
from ..utils.io import atomic_json, digest
from .chat import load_model
from .engine import DecodeEngine
from .sampling import Sampler, SamplingSettings

REPORT_FORMAT = "warpstate-posttrain-generation-v1"
ASSISTANT_HEADER = "<|assistant|>\n"


# ----------------------------------------------------------------------------------- prompt
class PromptEncoder:
    """Renders a conversation exactly as SFT data was rendered (segment by segment: SentencePiece
    normalisation is not compositional) and leaves the assistant header open for the model to continue."""

    def __init__(self, tokenizer):
        self.tokenizer = tokenizer
        vocab = tokenizer.vocab_size()
        self.eos = tokenizer.eos_id()
        if not 0 <= self.eos < vocab:
            raise ValueError("the tokenizer has no end-of-sequence token")
        bos = tokenizer.bos_id()
        self.bos = bos if 0 <= bos < vocab else None

    def __call__(self, messages) -> list[int]:
        if not isinstance(messages, list) or not messages:
            raise ValueError("a prompt needs at least one message")
        last = messages[-1]
        if not isinstance(last, dict) or last.get("role") not in ("user", "tool"):
            raise ValueError("the conversation to continue must end with a user or tool message")
        out = _Builder(self.tokenizer)
        if self.bos is not None:
            out.token(self.bos, False)
        for message in messages:
            check_message(message)
            out.piece(f"<|{message['role']}|>\n")
            out.piece(message["content"])
            if message["role"] == "assistant":
                out.token(self.eos, False)
            out.piece("\n")
        out.piece(ASSISTANT_HEADER)
        return out.ids


def encode_prompt(messages, tokenizer) -> list[int]:
    return PromptEncoder(tokenizer)(messages)


# ----------------------------------------------------------------------------------- one reply
@dataclass
class Generation:
    response: str
    token_ids: list
    prompt_tokens: int
    generated_tokens: int
    sampled_tokens: int
    elapsed_seconds: float
    first_token_seconds: float | None
    tokens_per_second: float
    stop_reason: str               # eos | length | context_limit
    temperature: float
    seed: int

    def as_dict(self) -> dict:
        return dict(self.__dict__)


def _sync(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize(device)


@torch.inference_mode()
def generate(engine: DecodeEngine, tokenizer, messages, *, max_new_tokens=256, max_context=2048, temperature=0.0,
             seed=42, on_token=None) -> dict:
    """One reply to ``messages``; returns the record of `Generation` as a dict."""
    for name, value, least in (("max_new_tokens", max_new_tokens, 1), ("max_context", max_context, 2), ("seed", seed, 0)):
        if type(value) is not int or value < least:
            raise ValueError(f"{name} must be an integer >= {least}")
    settings = SamplingSettings(temperature=temperature)
    ids = PromptEncoder(tokenizer)(messages)
    room = max_context - len(ids)
    if room <= 0:
        raise ValueError(f"the prompt alone is {len(ids)} tokens; the context limit is {max_context}")
    budget = min(max_new_tokens, room)
    sampler = Sampler(settings, torch.Generator(device="cpu").manual_seed(seed))
    device = engine.device
    _sync(device)
    started = time.perf_counter()
    logits = engine.prefill(torch.tensor([ids], dtype=torch.long, device=device))[0]
    reply: list[int] = []
    first = None
    draws = 0
    reason = "length" if budget == max_new_tokens else "context_limit"
    while len(reply) < budget:
        token = sampler.pick(logits.cpu())
        draws += 1
        if first is None:
            first = time.perf_counter() - started
        if token is None:
            raise RuntimeError("no candidate token left")
        if token == tokenizer.eos_id():
            reason = "eos"
            break
        reply.append(token)
        if on_token is not None:
            on_token(tuple(reply))
        if len(reply) < budget:
            logits = engine.step(torch.tensor([token], device=device))[0]
    _sync(device)
    took = time.perf_counter() - started
    return Generation(tokenizer.decode(reply), reply, len(ids), len(reply), draws, took, first, len(reply) / took,
                      reason, temperature, seed).as_dict()


@torch.inference_mode()
def generate_batch(engine: DecodeEngine, prompts: torch.Tensor, max_new_tokens: int, eos_id: int | None = None,
                   synchronous: bool = False) -> dict:
    """Greedy lock-step decode of equal-length prompts ``[B, T]``: token ids ``[B, n]``, tokens/s over the
    decode phase, per-token latencies in seconds and their median.

    On a CUDA device the steps are queued back to back (`DecodeEngine.decode_greedy`: the token pick is part of the
    step graph) and the latencies are the device times between consecutive steps, from CUDA events.
    ``synchronous=True`` is the host-driven loop -- arg-max on the host stream, one synchronisation per token, wall
    clock -- which is also what runs on the CPU."""
    device = engine.device
    _sync(device)
    mark = time.perf_counter()
    logits = engine.prefill(prompts)
    _sync(device)
    prefill_seconds = time.perf_counter() - mark
    token = torch.argmax(logits, dim=-1)
    if device.type == "cuda" and not synchronous and max_new_tokens > 1:
        events: list = []
        chosen = engine.decode_greedy(token, max_new_tokens - 1, events)
        _sync(device)
        tokens = torch.cat([token.unsqueeze(1), chosen], dim=1)
        latencies = [a.elapsed_time(b) / 1e3 for a, b in zip(events, events[1:])]
        timing = "device events between queued steps"
    else:
        columns, latencies = [], []
        for _ in range(max_new_tokens):
            columns.append(token)
            mark = time.perf_counter()
            token = torch.argmax(engine.step(token), dim=-1)
            _sync(device)
            latencies.append(time.perf_counter() - mark)
        tokens = torch.stack(columns, dim=1)
        timing = "host clock, one synchronisation per token"
    total = math.fsum(latencies)
    return {"tokens": tokens, "prefill_seconds": prefill_seconds, "decode_seconds": total,
            "tokens_per_second": tokens.shape[0] * len(latencies) / total, "latencies": latencies,
            "p50_latency_seconds": sorted(latencies)[len(latencies) // 2], "timing": timing}


# ----------------------------------------------------------------------------------- prompt suites
def conversation(prompt: str, system: str) -> list[dict]:
    opening = [{"role": "system", "content": system}] if system.strip() else []
    return [*opening, {"role": "user", "content": prompt}]


@dataclass
class PromptSuite:
    rows: list = field(default_factory=list)

    @classmethod
    def read(cls, path) -> "PromptSuite":
        document = json.loads(Path(path).read_text())
        rows = document.get("prompts") if isinstance(document, dict) else document
        if not isinstance(rows, list) or not rows:
            raise ValueError("a prompt suite is a non-empty list, or an object with a 'prompts' list")
        taken = set()
        for position, row in enumerate(rows):
            text = row.get("prompt") if isinstance(row, dict) else None
            if not isinstance(text, str) or not text.strip():
                raise ValueError(f"prompt suite row {position} has no prompt text")
            key = row.get("id", str(position))
            if not isinstance(key, (str, int)) or key in taken:
                raise ValueError("prompt suite ids must be distinct strings or integers")
            taken.add(key)
        return cls(rows)

    @classmethod
    def single(cls, prompt: str) -> "PromptSuite":
        if not prompt.strip():
            raise ValueError("the prompt is empty")
        return cls([{"id": "prompt", "prompt": prompt}])

    def run(self, answer, header: dict, default_system: str, base_seed: int, output: Path | None) -> dict:
        """``answer(messages, seed) -> record``; the report file is rewritten after every prompt so that an
        interrupted run leaves a valid, incomplete report."""
        report = dict(header, complete=False, results=[])
        if output is not None:
            output.parent.mkdir(parents=True, exist_ok=True)
        for position, row in enumerate(self.rows):
            key, system = row.get("id", str(position)), row.get("system", default_system)
            print(f"\n[{key}] {row['prompt']}", flush=True)
            record = answer(conversation(row["prompt"], system), base_seed + position)
            report["results"].append({"id": key, "prompt": row["prompt"], "system": system, **record})
            if output is not None:
                atomic_json(output, report)
        report["complete"] = True
        if output is not None:
            atomic_json(output, json.loads(json.dumps(report, default=str)))
            print(f"Results saved: {output}", flush=True)
        return report


# ----------------------------------------------------------------------------------- interactive
class Conversation:
    def __init__(self, answer, system: str, seed: int):
        self.answer, self.system, self.seed = answer, system, seed
        self.turns: list[dict] = []

    def say(self, text: str) -> None:
        turn = [*self.turns, {"role": "user", "content": text}] if self.turns else conversation(text, self.system)
        try:
            record = self.answer(turn, self.seed)
        except ValueError as problem:
            print(f"{problem}; /reset starts a new conversation.", flush=True)
            return
        if record["response"].strip():
            self.turns = [*turn, {"role": "assistant", "content": record["response"]}]

    def loop(self) -> int:
        print("Type a message. /reset forgets the conversation, /quit leaves, Ctrl-C cancels the current action.",
              flush=True)
        while True:
            try:
                text = input("You: ").strip()
            except EOFError:
                print()
                return 0
            except KeyboardInterrupt:
                print("\nCancelled.", flush=True)
                continue
            if text in ("/quit", "/exit"):
                return 0
            if text == "/reset":
                self.turns = []
            elif text:
                try:
                    self.say(text)
                except KeyboardInterrupt:
                    print("\nCancelled.", flush=True)


# ----------------------------------------------------------------------------------- command line
def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Chat with a WarpState SFT/DPO snapshot")
    p.add_argument("--snapshot", type=Path, required=True)
    p.add_argument("--tokenizer", type=Path, help="default: tokenizer.model next to the snapshot")
    p.add_argument("--device", default="cuda:0")
    what = p.add_mutually_exclusive_group()
    what.add_argument("--prompt")
    what.add_argument("--prompts-json", type=Path)
    p.add_argument("--output-json", type=Path)
    p.add_argument("--system", default="You are a helpful assistant.")
    p.add_argument("--max-new-tokens", type=int, default=256)
    p.add_argument("--max-context", type=int, default=2048)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--threads", type=int, default=8)
    return p


def main(argv=None) -> int:
    parser = build_parser()
    args = parser.parse_args(argv)
    try:
        snapshot = args.snapshot.expanduser().resolve()
        tokenizer = (args.tokenizer or snapshot.with_name("tokenizer.model")).expanduser().resolve()
        suite = None
        if args.prompts_json:
            suite = PromptSuite.read(args.prompts_json)
        elif args.prompt is not None:
            suite = PromptSuite.single(args.prompt)
        output = args.output_json.expanduser().resolve() if args.output_json else None
        if output is not None:
            if suite is None or output.exists() or output.is_relative_to(snapshot.parent):
                raise ValueError("--output-json needs a prompt or a suite and a new file outside the snapshot directory")
        if args.threads < 1 or args.seed < 0 or not 0 < args.max_new_tokens < args.max_context:
            raise ValueError("need threads >= 1, seed >= 0 and 0 < max-new-tokens < max-context")
        SamplingSettings(temperature=args.temperature)
        device = torch.device(args.device)
        torch.set_num_threads(args.threads)
        print(f"Loading sealed snapshot {snapshot}", flush=True)
        model, sp, metadata = load_model(snapshot, tokenizer, str(device))
        engine = DecodeEngine(model, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
    except (OSError, ValueError, RuntimeError) as problem:
        parser.error(str(problem))
    print(f"{metadata.get('stage', 'posttrain')} step {metadata['step']:,} | {model.num_parameters() / 1e9:.3f}B | "
          f"{device}", flush=True)

    def answer(messages, seed):
        record = generate(engine, sp, messages, max_new_tokens=args.max_new_tokens, max_context=args.max_context,
                          temperature=args.temperature, seed=seed)
        print(record["response"], flush=True)
        print(f"[{record['generated_tokens']} tokens; {record['elapsed_seconds']:.2f}s; stop={record['stop_reason']}]",
              flush=True)
        return record

    if suite is None:
        return Conversation(answer, args.system, args.seed).loop()
    seal = json.loads(snapshot.with_name("snapshot.json").read_text())
    header = {"format": REPORT_FORMAT, "snapshot": str(snapshot), "snapshot_sha256": seal["snapshot_sha256"],
              "metadata": metadata, "tokenizer_sha256": digest(tokenizer), "renderer_format": RENDER_FORMAT,
              "renderer_sha256": renderer_sha256(), "inference_sha256": digest(__file__), "device": str(device),
              "compute_dtype": str(engine.dtype), "parameter_dtype": "float32", "max_context": args.max_context,
              "max_new_tokens": args.max_new_tokens}
    suite.run(answer, header, args.system, args.seed, output)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
