"""Preparation of SFT / DPO data directories (JSONL + ``manifest.json``).

The reference bundle refers to a ``prepare_posttrain_data.py`` that it does not ship; this is
the tool that produces what its loaders verify (reference posttrain.py:117-156,
ops/dpo_data.py:37-78): every row carries its exact token and supervised-token counts, every file
its SHA-256 / rows / totals, and the manifest the tokenizer hash, renderer hash and
``max_length``.  Hold-out split: a row goes to validation iff
``sha256(json of the row)[:8] % val_modulus == 0``.  Rows that fail to render or exceed
``max_length`` are dropped and counted (never truncated).
"""
from __future__ import annotations

import argparse
import hashlib
import json
from pathlib import Path

from ..utils.io import atomic_json, digest
from . import dpo as DP
from . import sft as S


def _is_val(row: dict, modulus: int) -> bool:
    h = hashlib.sha256(json.dumps(row, sort_keys=True, ensure_ascii=False).encode()).digest()
    return int.from_bytes(h[:8], "little") % modulus == 0


def _write(path: Path, rows) -> dict:
    tokens = targets = 0
    with path.open("w") as f:
        for row, t, s in rows:
            f.write(json.dumps(row, ensure_ascii=False) + "\n")
            tokens += t
            targets += s
    return {"sha256": digest(path), "rows": len(rows), "tokens": tokens, "supervised_tokens": targets}


def prepare(out_dir: Path, tokenizer_path: Path, max_length: int, sft_rows=None, dpo_rows=None,
            val_modulus: int = 20) -> dict:
    import sentencepiece as spm
    sp = spm.SentencePieceProcessor(model_file=str(tokenizer_path))
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    outputs, dropped = {}, {"sft": 0, "dpo": 0}
    if sft_rows is not None:
        split = {"sft_train.jsonl": [], "sft_val.jsonl": []}
        for row in sft_rows:
            try:
                enc = S.encode_messages(row["messages"], sp, max_length=max_length)
            except (ValueError, KeyError):
                dropped["sft"] += 1
                continue
            tokens, targets = len(enc["input_ids"]), S.supervised_count(enc)
            record = {"messages": row["messages"], "tokens": tokens, "supervised_tokens": targets}
            split["sft_val.jsonl" if _is_val(row, val_modulus) else "sft_train.jsonl"].append((record, tokens, targets))
        if not split["sft_val.jsonl"] and len(split["sft_train.jsonl"]) > 1:
            split["sft_val.jsonl"].append(split["sft_train.jsonl"].pop())
        for name, rows in split.items():
            outputs[name] = _write(out_dir / name, rows)
    if dpo_rows is not None:
        split = {"dpo_train.jsonl": [], "dpo_val.jsonl": []}
        for row in dpo_rows:
            try:
                enc = DP.encode_pair(row, sp, max_length)
            except (ValueError, KeyError, AttributeError):
                dropped["dpo"] += 1
                continue
            tokens = {b: len(enc[b]["input_ids"]) for b in DP.BRANCHES}
            targets = {b: S.supervised_count(enc[b]) for b in DP.BRANCHES}
            record = {"prompt": row["prompt"], "chosen": row["chosen"], "rejected": row["rejected"],
                      "tokens": tokens, "supervised_tokens": targets}
            split["dpo_val.jsonl" if _is_val(row, val_modulus) else "dpo_train.jsonl"].append(
                (record, sum(tokens.values()), sum(targets.values())))
        if not split["dpo_val.jsonl"] and len(split["dpo_train.jsonl"]) > 1:
            split["dpo_val.jsonl"].append(split["dpo_train.jsonl"].pop())
        for name, rows in split.items():
            outputs[name] = _write(out_dir / name, rows)
    manifest = {"format": S.DATA_FORMAT, "complete": True, "tokenizer_sha256": digest(tokenizer_path),
                "renderer_sha256": S.renderer_sha256(), "renderer_format": S.RENDER_FORMAT,
                "mask_format": DP.MASK_FORMAT, "max_length": max_length, "outputs": outputs, "dropped": dropped}
    atomic_json(out_dir / "manifest.json", manifest)
    return manifest


def _read_jsonl(path):
    if path is None:
        return None
    with Path(path).open() as f:
        return [json.loads(line) for line in f if line.strip()]


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--out-dir", type=Path, required=True)
    p.add_argument("--tokenizer", type=Path, required=True)
    p.add_argument("--max-length", type=int, default=2048)
    p.add_argument("--sft", type=Path, help="JSONL of {'messages': [...]}")
    p.add_argument("--dpo", type=Path, help="JSONL of {'prompt': [...], 'chosen': [...], 'rejected': [...]}")
    p.add_argument("--val-modulus", type=int, default=20)
    a = p.parse_args(argv)
    manifest = prepare(a.out_dir, a.tokenizer, a.max_length, _read_jsonl(a.sft), _read_jsonl(a.dpo), a.val_modulus)
    print(json.dumps({"event": "prepared", "outputs": manifest["outputs"], "dropped": manifest["dropped"]}))


if __name__ == "__main__":
    main()
