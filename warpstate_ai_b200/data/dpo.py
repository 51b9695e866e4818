"""Preference pairs for DPO.

A pair is a shared prompt (ending in a user or tool message) with two candidate final assistant
messages, ``chosen`` and ``rejected``.  Both branches are rendered with the SFT renderer's
segmentation and only the final response -- its content and the end-of-sequence token -- is
scored: mask format ``warpstate-final-assistant-response-v1`` (the reference derives the same mask
by rendering the response a second time and blanking the prefix, reference ops/dpo_data.py:13-35;
here the branch is rendered once with supervision switched on for the last message only, which is
the same token and label sequence by construction).

`collate_pairs` interleaves the branches (rows 2i, 2i+1 = chosen, rejected of pair i) and returns
the mask of real pairs; `load_data` reads a prepared directory through `PreparedDirectory`.
"""
from __future__ import annotations

import torch

from .prepared import PreparedDirectory
from .sft import IGNORE_INDEX, _Builder, check_message, collate, renderer_sha256, supervised_count

MASK_FORMAT = "warpstate-final-assistant-response-v1"
BRANCHES = ("chosen", "rejected")


def _render_branch(prompt: list, response: dict, tokenizer, max_length: int | None) -> dict:
    """Prompt messages unsupervised, then the response message with content and EOS supervised."""
    out = _Builder(tokenizer)
    eos, bos = tokenizer.eos_id(), tokenizer.bos_id()
    if not 0 <= eos < out.vocab:
        raise ValueError("Tokenizer must define a real EOS token")
    if 0 <= bos < out.vocab:
        out.token(bos, False)
    for message in (*prompt, response):
        check_message(message)
        scored = message is response
        out.piece(f"<|{message['role']}|>\n")
        out.piece(message["content"], scored)
        if message["role"] == "assistant":
            out.token(eos, scored)
        out.piece("\n")
    if max_length is not None and len(out.ids) > max_length:
        raise ValueError(f"Conversation has {len(out.ids)} tokens, exceeds max_length={max_length}")
    record = {"input_ids": out.ids, "labels": out.labels}
    if supervised_count(record) == 0:
        raise ValueError("a preference branch needs at least one response token to score")
    return record


def encode_pair(row: dict, tokenizer, max_length: int | None) -> dict:
    prompt = row.get("prompt")
    if not isinstance(prompt, list) or not prompt or prompt[-1].get("role") not in ("user", "tool"):
        raise ValueError("a preference pair needs a shared prompt that ends with a user or tool message")
    pair = {}
    for branch in BRANCHES:
        candidates = row.get(branch)
        if not (isinstance(candidates, list) and len(candidates) == 1 and candidates[0].get("role") == "assistant"):
            raise ValueError(f"'{branch}' must be exactly one assistant message")
        pair[branch] = _render_branch(prompt, candidates[0], tokenizer, max_length)
    if pair["chosen"]["input_ids"] == pair["rejected"]["input_ids"]:
        raise ValueError("chosen and rejected render to the same tokens")
    return pair


def collate_pairs(records, sequence_length: int, pad_id: int):
    """Rows 2i / 2i+1 are the chosen / rejected branch of pair i; ``None`` pairs are inactive."""
    rows, real = [], []
    for record in records:
        real.append(record is not None)
        rows.extend((None, None) if record is None else (record["chosen"], record["rejected"]))
    x, y = collate(rows, sequence_length, pad_id)
    return x, y, torch.tensor(real, dtype=torch.bool)


def pair_tokens(record: dict) -> int:
    return sum(len(record[b]["input_ids"]) - 1 for b in BRANCHES)


def pair_targets(record: dict) -> int:
    return sum(supervised_count(record[b]) for b in BRANCHES)


def _measure(row: dict, record: dict):
    tokens = {b: len(record[b]["input_ids"]) for b in BRANCHES}
    scored = {b: supervised_count(record[b]) for b in BRANCHES}
    if any(row.get("tokens", {}).get(b) != tokens[b] or row.get("supervised_tokens", {}).get(b) != scored[b]
           for b in BRANCHES):
        return None
    return sum(tokens.values()), sum(scored.values())


def load_data(data_dir, tokenizer, tokenizer_hash: str, sequence_length: int):
    """-> (train pairs, validation pairs, manifest, SHA-256 of the manifest file)."""
    prepared = PreparedDirectory(data_dir, tokenizer_hash, renderer_sha256(), sequence_length)
    splits = [prepared.split(name, lambda row, _n: encode_pair(row, tokenizer, sequence_length), _measure,
                             progress_every=10000) for name in ("dpo_train.jsonl", "dpo_val.jsonl")]
    return splits[0], splits[1], prepared.manifest, prepared.manifest_digest()
