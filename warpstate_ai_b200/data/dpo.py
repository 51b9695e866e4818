"""Preference pairs for DPO: a shared prompt with a chosen and a rejected final assistant
response, rendered with the SFT renderer and masked so that only the response (content + EOS)
is scored -- mask format ``warpstate-final-assistant-response-v1`` (reference
ops/dpo_data.py:13-88).  `collate_pairs` interleaves chosen/rejected rows and returns an
``active`` mask for padding pairs of a short final batch.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..utils.io import digest
from .sft import DATA_FORMAT, IGNORE_INDEX, collate, encode_messages, renderer_sha256, supervised_count

MASK_FORMAT = "warpstate-final-assistant-response-v1"
BRANCHES = ("chosen", "rejected")


def encode_pair(row: dict, tokenizer, max_length: int | None) -> dict:
    prompt = row.get("prompt")
    if not isinstance(prompt, list) or not prompt or prompt[-1].get("role") not in ("user", "tool"):
        raise ValueError("DPO requires a nonempty shared prompt ending user/tool")
    has_bos = int(0 <= tokenizer.bos_id() < tokenizer.vocab_size())
    out = {}
    for name in BRANCHES:
        response = row.get(name)
        if not isinstance(response, list) or len(response) != 1 or response[0].get("role") != "assistant":
            raise ValueError("DPO requires exactly one final assistant response per branch")
        whole = encode_messages(prompt + response, tokenizer, max_length=max_length)
        tail = encode_messages(response, tokenizer)
        prefix = len(whole["input_ids"]) - len(tail["input_ids"]) + has_bos
        if whole["input_ids"][prefix:] != tail["input_ids"][has_bos:]:
            raise ValueError("Response segmentation differs from the frozen SFT renderer")
        whole["labels"][:prefix] = [IGNORE_INDEX] * prefix
        if supervised_count(whole) == 0:
            raise ValueError("Preference branch has no response targets")
        out[name] = whole
    if out["chosen"]["input_ids"] == out["rejected"]["input_ids"]:
        raise ValueError("Chosen and rejected responses must differ")
    return out


def collate_pairs(records, sequence_length: int, pad_id: int):
    """Rows 2i / 2i+1 are the chosen / rejected branch of pair i; ``None`` pairs are inactive."""
    rows = [record[b] if record is not None else None for record in records for b in BRANCHES]
    x, y = collate(rows, sequence_length, pad_id)
    return x, y, torch.tensor([record is not None for record in records], dtype=torch.bool)


def pair_tokens(record: dict) -> int:
    return sum(len(record[b]["input_ids"]) - 1 for b in BRANCHES)


def pair_targets(record: dict) -> int:
    return sum(supervised_count(record[b]) for b in BRANCHES)


def load_data(data_dir, tokenizer, tokenizer_hash: str, sequence_length: int):
    directory = Path(data_dir)
    manifest_path = directory / "manifest.json"
    manifest = json.loads(manifest_path.read_text())
    if manifest.get("format") != DATA_FORMAT or manifest.get("complete") is not True:
        raise ValueError("Posttraining data is not complete")
    if manifest.get("tokenizer_sha256") != tokenizer_hash:
        raise ValueError("Prepared data tokenizer hash differs")
    if manifest.get("renderer_sha256") != renderer_sha256():
        raise ValueError("Prepared data renderer hash differs")
    if manifest.get("max_length") != sequence_length:
        raise ValueError("Prepared data max_length differs from sequence_length")
    splits = []
    for filename in ("dpo_train.jsonl", "dpo_val.jsonl"):
        path = directory / filename
        info = manifest.get("outputs", {}).get(filename)
        if not info or not path.is_file() or digest(path) != info.get("sha256"):
            raise ValueError(f"Missing or changed prepared file: {filename}")
        records, tokens_total, targets_total = [], 0, 0
        with path.open() as stream:
            for number, line in enumerate(stream, 1):
                row = json.loads(line)
                encoded = encode_pair(row, tokenizer, sequence_length)
                for b in BRANCHES:
                    tokens, targets = len(encoded[b]["input_ids"]), supervised_count(encoded[b])
                    if row.get("tokens", {}).get(b) != tokens or row.get("supervised_tokens", {}).get(b) != targets:
                        raise ValueError(f"{filename}:{number}: token metadata differs")
                    tokens_total += tokens
                    targets_total += targets
                records.append(encoded)
                if number % 10000 == 0:
                    print(json.dumps(dict(event="data_validation", file=filename, rows=number)), flush=True)
        if not records or len(records) != info.get("rows"):
            raise ValueError(f"{filename}: empty data or row count mismatch")
        if tokens_total != info.get("tokens") or targets_total != info.get("supervised_tokens"):
            raise ValueError(f"{filename}: manifest token totals differ")
        splits.append(records)
    return splits[0], splits[1], manifest, digest(manifest_path)
