"""Interactive / one-shot text generation from a sealed inference snapshot.

Snapshot handling follows the reference probe (chat.py:37-151): a training checkpoint
(``warpstate-server-v1``) is never loaded directly; `capture_latest` pins the published file by
file descriptor (the trainer replaces ``latest.pt`` by rename, so an open descriptor keeps one
complete version), exports the model-only ``warpstate-chat-v1`` snapshot read-only with a
``snapshot.json`` carrying its SHA-256, and `load_model` verifies snapshot hash, tokenizer hash
and a strict meta-device load before any generation.

Generation differs: the prompt is prefilled in whole chunks through the training forward path
and decoded with the batched `DecodeEngine` (CUDA graph replay per token on a GPU); ``--device
cpu`` keeps the reference's FP32 probe behaviour.
"""
from __future__ import annotations

import argparse
import gc
import json
import math
import os
import stat
import tempfile
import time
from pathlib import Path

import torch

from ..ckpt.formats import CHAT_FORMAT, SERVER_FORMAT
from ..config import WarpStateConfig
from ..models.warpstate import WarpStateLM
from ..utils.io import digest, fsync_dir, utc_timestamp
from .engine import DecodeEngine
from .sampling import banned_ngram_tokens, sample_token

ROOT = Path(__file__).resolve().parents[2]
FORMAT = CHAT_FORMAT


def capture_latest(source, tokenizer, snapshot_root) -> Path:
    source, tokenizer, snapshot_root = Path(source), Path(tokenizer), Path(snapshot_root)
    if source.suffix != ".pt" or source.is_symlink():
        raise ValueError("Select a completed regular .pt checkpoint, not a temporary file")
    tokenizer_sha = digest(tokenizer)
    fd = os.open(source, os.O_RDONLY | os.O_NOFOLLOW)
    try:
        before = os.fstat(fd)
        if not stat.S_ISREG(before.st_mode):
            raise ValueError("Checkpoint must be a regular file")
        checkpoint = torch.load(f"/proc/self/fd/{fd}", map_location="cpu", weights_only=False, mmap=True)
        if checkpoint.get("format") == FORMAT:
            raise ValueError(f"Chat snapshot requires its original snapshot.json beside {source}. "
                             "Restore that metadata or export a fresh snapshot from a training checkpoint.")
        if checkpoint.get("format") != SERVER_FORMAT:
            raise ValueError("Expected a full warpstate-server-v1 training checkpoint")
        if checkpoint["signature"]["data"]["signature"]["tokenizer_sha256"] != tokenizer_sha:
            raise ValueError("Tokenizer SHA256 differs from training checkpoint")
        snapshot_root.mkdir(parents=True, exist_ok=True)
        folder = Path(tempfile.mkdtemp(prefix=f"step-{checkpoint['step']}-", dir=snapshot_root))
        destination, temporary = folder / "model.pt", folder / "model.pt.tmp"
        identity = (before.st_dev, before.st_ino, before.st_size, before.st_mtime_ns)
        metadata = dict(format=FORMAT, inference_only=True, config=checkpoint["config"], step=checkpoint["step"],
                        tokens_seen=checkpoint["tokens_seen"], val_loss=checkpoint.get("val_loss"),
                        tokenizer_sha256=tokenizer_sha, captured_at_utc=utc_timestamp(),
                        source=dict(path=str(source.resolve()), device=before.st_dev, inode=before.st_ino,
                                    size=before.st_size, mtime_ns=before.st_mtime_ns))
        print(f"Capturing completed step {metadata['step']:,} / {metadata['tokens_seen']:,} tokens; "
              "model weights only...", flush=True)
        with temporary.open("xb") as stream:
            torch.save(dict(metadata, model=checkpoint["model"]), stream)
            stream.flush()
            os.fsync(stream.fileno())
        after = os.fstat(fd)
        if identity != (after.st_dev, after.st_ino, after.st_size, after.st_mtime_ns):
            raise RuntimeError("Pinned checkpoint contents changed; snapshot not published")
        os.chmod(temporary, 0o444)
        os.replace(temporary, destination)
        metadata["snapshot_sha256"] = digest(destination)
        metadata["snapshot_bytes"] = destination.stat().st_size
        with (folder / "snapshot.json").open("x") as stream:
            json.dump(metadata, stream, indent=2)
            stream.write("\n")
            stream.flush()
            os.fsync(stream.fileno())
        fsync_dir(folder)
        return destination
    finally:
        os.close(fd)


def resolve_snapshot(source, tokenizer, snapshot_root) -> Path:
    source = Path(source)
    if not source.is_file():
        raise ValueError(f"Checkpoint file does not exist or is not a regular file: {source}")
    if source.with_name("snapshot.json").exists():
        return source
    return capture_latest(source, tokenizer, snapshot_root)


def load_model(snapshot, tokenizer, device: str = "cpu"):
    import sentencepiece as spm
    snapshot, tokenizer = Path(snapshot), Path(tokenizer)
    proof_path = snapshot.with_name("snapshot.json")
    try:
        proof = json.loads(proof_path.read_text())
    except FileNotFoundError as exc:
        raise ValueError(f"Missing snapshot metadata: {proof_path}. Use --checkpoint to export training weights, "
                         "or restore the original metadata.") from exc
    if not isinstance(proof, dict) or not isinstance(proof.get("snapshot_sha256"), str):
        raise ValueError(f"Invalid snapshot metadata: {proof_path}")
    if proof["snapshot_sha256"] != digest(snapshot):
        raise ValueError("Inference snapshot SHA256 mismatch")
    checkpoint = torch.load(snapshot, map_location="cpu", weights_only=False, mmap=True)
    if checkpoint.get("format") != FORMAT or not checkpoint.get("inference_only"):
        raise ValueError("Use the independent inference snapshot, not live latest.pt")
    if checkpoint["tokenizer_sha256"] != digest(tokenizer):
        raise ValueError("Tokenizer SHA256 mismatch")
    config = WarpStateConfig(**checkpoint["config"])
    sp = spm.SentencePieceProcessor(model_file=str(tokenizer))
    if sp.vocab_size() != config.vocab_size:
        raise ValueError("Tokenizer vocabulary differs from model")
    with torch.device("meta"):
        model = WarpStateLM(config)
    model.load_state_dict(checkpoint["model"], strict=True, assign=True)
    model.eval().requires_grad_(False)
    if any(p.dtype != torch.float32 for p in model.parameters()):
        raise ValueError("Snapshots hold the original FP32 model parameters")
    model = model.to(device)
    metadata = {k: v for k, v in checkpoint.items() if k != "model"}
    del checkpoint
    gc.collect()
    return model, sp, metadata


@torch.inference_mode()
def generate(model, sp, prompt: str, *, max_new_tokens=256, temperature=0.8, top_k=40, top_p=0.9, seed=1337,
             max_context=2048, repetition_penalty=1.2, no_repeat_ngram_size=4, engine: DecodeEngine | None = None):
    """Yields token ids of the reply."""
    if max_new_tokens < 1 or max_context <= max_new_tokens:
        raise ValueError("Require 0 < max-new-tokens < max-context")
    if not math.isfinite(repetition_penalty) or repetition_penalty < 1:
        raise ValueError("Require a finite repetition-penalty >= 1")
    if not isinstance(no_repeat_ngram_size, int) or no_repeat_ngram_size < 0:
        raise ValueError("Require an integer no-repeat-ngram-size >= 0")
    ids = sp.encode(prompt, out_type=int)
    if not ids:
        raise ValueError("Prompt contains no tokens")
    ids = ids[-(max_context - max_new_tokens):]
    device = model.embed.weight.device
    engine = engine or DecodeEngine(model, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
    logits = engine.prefill(torch.tensor([ids], dtype=torch.long, device=device))[0]
    generator = torch.Generator(device="cpu").manual_seed(seed)
    generated = []
    for index in range(max_new_tokens):
        value = sample_token(logits.cpu(), temperature, top_k, top_p, generator, previous_tokens=generated,
                             repetition_penalty=repetition_penalty,
                             banned_tokens=banned_ngram_tokens(generated, no_repeat_ngram_size))
        if value is None or value == sp.eos_id():
            break
        generated.append(value)
        yield value
        if index + 1 < max_new_tokens:
            logits = engine.step(torch.tensor([value], device=device))[0]


def reply(model, sp, prompt, args, engine=None) -> str:
    ids, emitted = [], ""
    begin, first = time.perf_counter(), None
    for value in generate(model, sp, prompt, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                          top_k=args.top_k, top_p=args.top_p, seed=args.seed, max_context=args.max_context,
                          repetition_penalty=args.repetition_penalty,
                          no_repeat_ngram_size=args.no_repeat_ngram_size, engine=engine):
        if first is None:
            first = time.perf_counter()
        ids.append(value)
        safe = sp.decode(ids).split("�", 1)[0]  # hold back incomplete byte-fallback characters
        if safe.startswith(emitted):
            print(safe[len(emitted):], end="", flush=True)
            emitted = safe
    text = sp.decode(ids)
    if text.startswith(emitted):
        print(text[len(emitted):], end="", flush=True)
    elapsed = time.perf_counter() - begin
    ttft = "-" if first is None else f"{first - begin:.2f}s"
    print(f"\n[{len(ids)} tokens; {elapsed:.1f}s total; TTFT {ttft}; {len(ids) / max(elapsed, 1e-9):.1f} tok/s]", flush=True)
    return text


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="WarpState base-model probe")
    p.add_argument("--checkpoint", type=Path, default=ROOT / "work/run/latest.pt")
    p.add_argument("--snapshot", type=Path, help="reuse a sealed model-only snapshot, or export a training checkpoint")
    p.add_argument("--snapshot-root", type=Path, default=ROOT / "work/chat")
    p.add_argument("--tokenizer", type=Path, default=ROOT / "tokenizer.model")
    p.add_argument("--capture-only", action="store_true")
    p.add_argument("--prompt", help="one-shot probe instead of interactive input")
    p.add_argument("--raw", action="store_true", help="plain text completion instead of Q/A labels")
    p.add_argument("--threads", type=int, default=16)
    p.add_argument("--max-new-tokens", type=int, default=256)
    p.add_argument("--max-context", type=int, default=2048)
    p.add_argument("--temperature", type=float, default=0.8, help="0 = greedy")
    p.add_argument("--top-k", type=int, default=40)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--repetition-penalty", type=float, default=1.2)
    p.add_argument("--no-repeat-ngram-size", type=int, default=4)
    p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--device", choices=["cpu", "cuda"], default="cpu")
    return p


def main(argv=None) -> None:
    parser = build_parser()
    args = parser.parse_args(argv)
    if args.threads < 1 or not 0 < args.max_new_tokens < args.max_context:
        parser.error("Require threads >= 1 and 0 < max-new-tokens < max-context")
    if not math.isfinite(args.temperature) or args.temperature < 0 or args.top_k < 0 or not 0 < args.top_p <= 1:
        parser.error("Invalid temperature / top-k / top-p")
    if not math.isfinite(args.repetition_penalty) or args.repetition_penalty < 1 or args.no_repeat_ngram_size < 0:
        parser.error("Require finite repetition-penalty >= 1 and no-repeat-ngram-size >= 0")
    if args.prompt is not None and not args.prompt.strip():
        parser.error("A one-shot prompt must not be empty")
    torch.set_num_threads(args.threads)
    try:
        if args.snapshot is not None:
            snapshot = resolve_snapshot(args.snapshot, args.tokenizer, args.snapshot_root)
        else:
            snapshot = capture_latest(args.checkpoint, args.tokenizer, args.snapshot_root)
        print(f"Snapshot: {snapshot}", flush=True)
        if args.capture_only:
            return
        model, sp, metadata = load_model(snapshot, args.tokenizer, args.device)
    except (OSError, ValueError) as exc:
        parser.error(str(exc))
    print(f"WarpState {model.num_parameters() / 1e9:.3f}B | {args.device} | step {metadata['step']:,} | "
          f"{metadata['tokens_seen']:,} training tokens", flush=True)
    print("Base pretrained model, not instruction-tuned. Q/A labels are only a probe.\n"
          "Commands: /new, /raw, /chat, /info, /help, /exit. Ctrl-C cancels a reply.", flush=True)
    history = ""
    while True:
        try:
            user = args.prompt if args.prompt is not None else input("\nYou: ").strip()
            if user is None or (args.prompt is None and user in ("/exit", "/quit")):
                break
            if not user:
                continue
            if args.prompt is None and user in ("/new", "/raw", "/chat"):
                history = ""
                if user != "/new":
                    args.raw = user == "/raw"
                print("Context cleared. Mode: " + ("raw completion" if args.raw else "Q/A probe"))
                continue
            if args.prompt is None and user == "/info":
                print(json.dumps(metadata, indent=2, default=str))
                continue
            if args.prompt is None and user == "/help":
                print("/new clears context; /raw plain completion; /chat Q/A; /info snapshot; /exit quit")
                continue
            prompt = history + (user if args.raw else f"Question: {user}\nAnswer:")
            print("Model: ", end="", flush=True)
            answer = reply(model, sp, prompt, args)
            history = prompt + ("" if args.raw else " ") + answer + "\n\n"
            if args.prompt is not None:
                break
        except EOFError:
            break
        except KeyboardInterrupt:
            print("\nReply cancelled; training was not affected.", flush=True)
            if args.prompt is not None:
                break


if __name__ == "__main__":
    main()
