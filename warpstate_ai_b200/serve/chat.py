"""Text generation from a sealed inference snapshot: one-shot prompt or interactive session.

The entry point of the reference's base-model probe (reference chat.py: snapshot capture and
verification :37-151, sampling :154-193, generation :196-255, REPL :258-352), rebuilt on this
framework's serving pieces:

* snapshots are exported, verified and loaded by `serve.snapshots.SnapshotStore`;
* the prompt is prefilled in whole 128-token chunks through the training kernels and decoded by
  the batched `DecodeEngine` (CUDA-graph replay per token on a GPU; ``--device cpu`` runs the
  FP32 PyTorch definition, like the reference's probe), where the reference feeds the prompt
  token by token through ``model.step``;
* token choice is `serve.sampling.Sampler` with a `ReplyHistory` per reply;
* the interactive loop is a `ChatSession` with a table of slash commands.

`capture_latest`, `resolve_snapshot`, `load_model` and `generate` keep the reference's call
signatures for code that imports them.
"""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path

import torch

from ..ckpt.formats import CHAT_FORMAT
from .engine import DecodeEngine
from .sampling import ReplyHistory, Sampler, SamplingSettings
from .snapshots import SnapshotStore

ROOT = Path(__file__).resolve().parents[2]
FORMAT = CHAT_FORMAT


# ----------------------------------------------------------------------------------- snapshot helpers
def capture_latest(source, tokenizer, snapshot_root) -> Path:
    return SnapshotStore(snapshot_root, tokenizer).export(source)


def resolve_snapshot(source, tokenizer, snapshot_root) -> Path:
    return SnapshotStore(snapshot_root, tokenizer).resolve(source)


def load_model(snapshot, tokenizer, device: str = "cpu"):
    return SnapshotStore(Path(snapshot).parent.parent, tokenizer).load(snapshot, device)


# ----------------------------------------------------------------------------------- generation
def _context_window(ids: list, max_new_tokens: int, max_context: int) -> list:
    if not 0 < max_new_tokens < max_context:
        raise ValueError("need 0 < max-new-tokens < max-context")
    if not ids:
        raise ValueError("the prompt encodes to no tokens")
    return ids[-(max_context - max_new_tokens):]


@torch.inference_mode()
def generate(model, sp, prompt: str, *, max_new_tokens=256, temperature=0.8, top_k=40, top_p=0.9, seed=1337,
             max_context=2048, repetition_penalty=1.2, no_repeat_ngram_size=4, engine: DecodeEngine | None = None):
    """Yields the reply's token ids one by one (stops at end-of-sequence, at the length limit or when
    the sampling rules leave no candidate)."""
    settings = SamplingSettings(temperature=temperature, top_k=top_k, top_p=top_p,
                                repetition_penalty=repetition_penalty, no_repeat_ngram=no_repeat_ngram_size)
    ids = _context_window(sp.encode(prompt, out_type=int), max_new_tokens, max_context)
    device = model.embed.weight.device
    if engine is None:
        engine = DecodeEngine(model, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
    sampler = Sampler(settings, torch.Generator(device="cpu").manual_seed(seed))
    history = ReplyHistory(settings.no_repeat_ngram)
    logits = engine.prefill(torch.tensor([ids], dtype=torch.long, device=device))[0]
    stop = sp.eos_id()
    while len(history.tokens) < max_new_tokens:
        token = sampler.next(logits.cpu(), history)
        if token is None or token == stop:
            return
        history.push(token)
        yield token
        if len(history.tokens) < max_new_tokens:
            logits = engine.step(torch.tensor([token], device=device))[0]


class ReplyPrinter:
    """Streams a reply to the terminal as it decodes.  SentencePiece may emit a multi-byte character over
    several byte-fallback tokens; text after the first replacement character is held back until complete."""

    def __init__(self, sp):
        self.sp, self.ids, self.shown = sp, [], ""
        self.started = time.perf_counter()
        self.first_token_at = None

    def _emit(self, text: str) -> None:
        if text.startswith(self.shown):
            print(text[len(self.shown):], end="", flush=True)
            self.shown = text

    def feed(self, token: int) -> None:
        if self.first_token_at is None:
            self.first_token_at = time.perf_counter()
        self.ids.append(token)
        self._emit(self.sp.decode(self.ids).partition("�")[0])

    def finish(self) -> str:
        text = self.sp.decode(self.ids)
        self._emit(text)
        took = time.perf_counter() - self.started
        first = "-" if self.first_token_at is None else f"{self.first_token_at - self.started:.2f}s"
        rate = len(self.ids) / max(took, 1e-9)
        print(f"\n[{len(self.ids)} tokens; {took:.1f}s total; TTFT {first}; {rate:.1f} tok/s]", flush=True)
        return text


def reply(model, sp, prompt, args, engine=None) -> str:
    printer = ReplyPrinter(sp)
    for token in generate(model, sp, prompt, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                          top_k=args.top_k, top_p=args.top_p, seed=args.seed, max_context=args.max_context,
                          repetition_penalty=args.repetition_penalty, no_repeat_ngram_size=args.no_repeat_ngram_size,
                          engine=engine):
        printer.feed(token)
    return printer.finish()


# ----------------------------------------------------------------------------------- interactive session
class ChatSession:
    """Conversation state plus the slash commands.  In Q/A mode a turn is framed as
    ``Question: ...\\nAnswer:`` (the reference's probe format); raw mode continues plain text."""

    def __init__(self, model, sp, metadata: dict, args):
        self.model, self.sp, self.metadata, self.args = model, sp, metadata, args
        self.raw = bool(args.raw)
        self.transcript = ""
        self.commands = {"/new": self._new, "/raw": self._raw, "/chat": self._qa, "/info": self._info,
                         "/help": self._help}

    def _mode(self) -> str:
        return "raw completion" if self.raw else "Q/A probe"

    def _new(self) -> None:
        self.transcript = ""
        print(f"Context cleared. Mode: {self._mode()}")

    def _raw(self) -> None:
        self.raw = True
        self._new()

    def _qa(self) -> None:
        self.raw = False
        self._new()

    def _info(self) -> None:
        print(json.dumps(self.metadata, indent=2, default=str))

    def _help(self) -> None:
        print("/new forget the conversation; /raw plain completion; /chat question/answer framing; "
              "/info snapshot metadata; /exit leave")

    def ask(self, text: str) -> str:
        prompt = self.transcript + (text if self.raw else f"Question: {text}\nAnswer:")
        print("Model: ", end="", flush=True)
        answer = reply(self.model, self.sp, prompt, self.args)
        self.transcript = prompt + ("" if self.raw else " ") + answer + "\n\n"
        return answer

    def banner(self) -> None:
        meta = self.metadata
        print(f"WarpState {self.model.num_parameters() / 1e9:.3f}B | {self.args.device} | step {meta['step']:,} | "
              f"{meta['tokens_seen']:,} training tokens", flush=True)
        print("This is a pretrained base model without instruction tuning; the Q/A framing is a probe only.\n"
              "Commands: " + ", ".join(self.commands) + ", /exit. Ctrl-C cancels the current reply.", flush=True)

    def loop(self) -> None:
        while True:
            try:
                line = input("\nYou: ").strip()
            except EOFError:
                return
            if line in ("/exit", "/quit"):
                return
            if not line:
                continue
            command = self.commands.get(line)
            try:
                command() if command else self.ask(line)
            except KeyboardInterrupt:
                print("\nReply cancelled (a running training job is not touched by this).", flush=True)


# ----------------------------------------------------------------------------------- command line
def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="WarpState base-model probe")
    where = p.add_argument_group("snapshot")
    where.add_argument("--checkpoint", type=Path, default=ROOT / "work/run/latest.pt")
    where.add_argument("--snapshot", type=Path, help="a sealed export to reuse, or a training checkpoint to export first")
    where.add_argument("--snapshot-root", type=Path, default=ROOT / "work/chat")
    where.add_argument("--tokenizer", type=Path, default=ROOT / "tokenizer.model")
    where.add_argument("--capture-only", action="store_true", help="export and stop")
    run = p.add_argument_group("generation")
    run.add_argument("--prompt", help="answer this one prompt and exit")
    run.add_argument("--raw", action="store_true", help="continue plain text instead of the Q/A framing")
    run.add_argument("--device", choices=["cpu", "cuda"], default="cpu")
    run.add_argument("--threads", type=int, default=16)
    run.add_argument("--seed", type=int, default=1337)
    for flag, kind, default, note in (("--max-new-tokens", int, 256, None), ("--max-context", int, 2048, None),
                                      ("--temperature", float, 0.8, "0 selects the most likely token"),
                                      ("--top-k", int, 40, None), ("--top-p", float, 0.9, None),
                                      ("--repetition-penalty", float, 1.2, None),
                                      ("--no-repeat-ngram-size", int, 4, None)):
        run.add_argument(flag, type=kind, default=default, help=note)
    return p


def _check_args(parser, args) -> None:
    if args.threads < 1:
        parser.error("--threads must be at least 1")
    if not 0 < args.max_new_tokens < args.max_context:
        parser.error("need 0 < --max-new-tokens < --max-context")
    try:
        SamplingSettings(args.temperature, args.top_k, args.top_p, args.repetition_penalty, args.no_repeat_ngram_size)
    except ValueError as problem:
        parser.error(str(problem))
    if args.prompt is not None and not args.prompt.strip():
        parser.error("--prompt is empty")


def main(argv=None) -> None:
    parser = build_parser()
    args = parser.parse_args(argv)
    _check_args(parser, args)
    torch.set_num_threads(args.threads)
    store = SnapshotStore(args.snapshot_root, args.tokenizer)
    try:
        snapshot = store.resolve(args.snapshot) if args.snapshot is not None else store.export(args.checkpoint)
        print(f"Snapshot: {snapshot}", flush=True)
        if args.capture_only:
            return
        model, sp, metadata = store.load(snapshot, args.device)
    except (OSError, ValueError) as problem:
        parser.error(str(problem))
    session = ChatSession(model, sp, metadata, args)
    session.banner()
    if args.prompt is not None:
        try:
            session.ask(args.prompt)
        except KeyboardInterrupt:
            print("\nReply cancelled.", flush=True)
        return
    session.loop()


if __name__ == "__main__":
    main()
