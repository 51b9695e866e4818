"""Conversation rendering, collation and deterministic batching for SFT.

Renderer ``warpstate-segmented-roles-v1`` (reference ops/posttrain_data.py:24-71): optional BOS,
then for each message the role header ``"<|role|>\\n"``, the content, EOS after assistant
content, and ``"\\n"`` -- every segment encoded on its own (SentencePiece normalisation is not
compositional, so inference must use the same segmentation).  Only assistant content and its
EOS are supervised; everything else is labelled -100.  Conversations are never truncated.

`collate` right-pads, shifts by one and masks (reference posttrain.py:159-172);
`update_indices` yields one deterministic global batch per update that never crosses an epoch
boundary (posttrain.py:175-189).  The identity of prepared data includes the SHA-256 of this
file (`renderer_sha256`), so a change to the renderer invalidates prepared data by design.
"""
from __future__ import annotations

import hashlib
import random
from functools import lru_cache
from pathlib import Path

import torch


RENDER_FORMAT = "warpstate-segmented-roles-v1"
from .prepared import DATA_FORMAT  # noqa: E402  (the directory format lives with its reader)
IGNORE_INDEX = -100
ROLES = frozenset({"system", "user", "assistant", "tool"})


def renderer_sha256() -> str:
    return hashlib.sha256(Path(__file__).read_bytes()).hexdigest()


class _Builder:
    def __init__(self, tokenizer):
        self.tok = tokenizer
        self.vocab = tokenizer.vocab_size()
        self.ids: list[int] = []
        self.labels: list[int] = []

    def piece(self, text: str, supervised: bool = False) -> None:
        tokens = self.tok.encode(text, out_type=int)
        if any(type(t) is not int or not 0 <= t < self.vocab for t in tokens):
            raise ValueError("Tokenizer returned invalid token IDs")
        self.ids.extend(tokens)
        self.labels.extend(tokens if supervised else [IGNORE_INDEX] * len(tokens))

    def token(self, token: int, supervised: bool) -> None:
        self.ids.append(token)
        self.labels.append(token if supervised else IGNORE_INDEX)


def check_message(message) -> None:
    if not isinstance(message, dict) or message.get("role") not in ROLES:
        raise ValueError("Unsupported conversation role")
    content = message.get("content")
    if not isinstance(content, str) or not content.strip():
        raise ValueError("Each message requires nonempty text content")
    if message.get("tool_calls"):
        raise ValueError("Structured tool calls must be serialized into content by preparation")


def encode_messages(messages, tokenizer, max_length: int | None = None) -> dict:
    """Unshifted ``input_ids`` / ``labels``; training uses ``x = ids[:-1], y = labels[1:]``."""
    if not isinstance(messages, list) or not messages:
        raise ValueError("messages must be a nonempty list")
    if max_length is not None and (type(max_length) is not int or max_length < 2):
        raise ValueError("max_length must be an integer >= 2")
    eos, bos = tokenizer.eos_id(), tokenizer.bos_id()
    b = _Builder(tokenizer)
    if not 0 <= eos < b.vocab:
        raise ValueError("Tokenizer must define a real EOS token")
    if 0 <= bos < b.vocab:
        b.token(bos, False)
    for message in messages:
        check_message(message)
        assistant = message["role"] == "assistant"
        b.piece(f"<|{message['role']}|>\n")
        b.piece(message["content"], assistant)
        if assistant:
            b.token(eos, True)
        b.piece("\n")
    if max_length is not None and len(b.ids) > max_length:
        raise ValueError(f"Conversation has {len(b.ids)} tokens, exceeds max_length={max_length}")
    if len(b.ids) < 2 or not any(label != IGNORE_INDEX for label in b.labels[1:]):
        raise ValueError("Conversation has no supervised next-token targets")
    return {"input_ids": b.ids, "labels": b.labels}


def supervised_count(record: dict) -> int:
    return sum(label != IGNORE_INDEX for label in record["labels"][1:])


def collate(records, sequence_length: int, pad_id: int):
    """``records`` may contain ``None`` (a fully masked padding row for a rank short of data)."""
    x = torch.full((len(records), sequence_length), pad_id, dtype=torch.long)
    y = torch.full_like(x, IGNORE_INDEX)
    for row, record in enumerate(records):
        if record is None:
            continue
        ids, labels = record["input_ids"], record["labels"]
        if len(ids) != len(labels) or not 2 <= len(ids) <= sequence_length:
            raise ValueError("Invalid encoded record length")
        n = len(ids) - 1
        x[row, :n] = torch.tensor(ids[:-1])
        y[row, :n] = torch.tensor(labels[1:])
    return x, y


@lru_cache(maxsize=4)
def epoch_order(size: int, seed: int, epoch: int) -> tuple:
    order = list(range(size))
    random.Random(seed + epoch).shuffle(order)
    return tuple(order)


def update_indices(size: int, seed: int, cursor: int, epochs: int, global_batch: int):
    """Sample ids of one update and the next cursor; empty when all epochs are consumed."""
    epoch, offset = divmod(cursor, size)
    if epoch >= epochs:
        return [], cursor
    count = min(global_batch, size - offset)
    return list(epoch_order(size, seed, epoch)[offset:offset + count]), cursor + count


def rank_microbatches(indices, records, micro_batch: int, grad_accum: int, world: int, rank: int):
    """Rows of this rank per accumulation step: ``indices[(micro*world+rank)*mb : +mb]`` padded
    with ``None`` (posttrain.py:468-474)."""
    out = []
    for micro in range(grad_accum):
        offset = (micro * world + rank) * micro_batch
        chosen = [records[i] for i in indices[offset:offset + micro_batch]]
        out.append(chosen + [None] * (micro_batch - len(chosen)))
    return out


def load_data(data_dir, tokenizer, tokenizer_hash: str, sequence_length: int):
    """Load and re-encode prepared SFT data, refusing anything partial or inconsistent:
    -> (train records, validation records, manifest, SHA-256 of the manifest file)."""
    from .prepared import PreparedDirectory
    prepared = PreparedDirectory(data_dir, tokenizer_hash, renderer_sha256(), sequence_length)

    def encode(row, number):
        if row.get("tools"):
            raise ValueError(f"row {number}: tool definitions must already be part of the messages")
        return encode_messages(row["messages"], tokenizer, max_length=sequence_length)

    def measure(row, record):
        counts = len(record["input_ids"]), supervised_count(record)
        return counts if (row.get("tokens"), row.get("supervised_tokens")) == counts else None

    train, val = (prepared.split(name, encode, measure) for name in ("sft_train.jsonl", "sft_val.jsonl"))
    return train, val, prepared.manifest, prepared.manifest_digest()
