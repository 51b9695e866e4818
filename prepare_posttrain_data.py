#!/usr/bin/env python3
"""Prepare SFT / DPO data: render, validate and publish JSONL files with a manifest.

Input: JSONL conversations (``{"messages": [...]}``) for SFT and preference pairs
(``{"prompt": [...], "chosen": "...", "rejected": "..."}``) for DPO.  Output directory receives
``sft_train.jsonl``, ``sft_val.jsonl`` (and ``dpo_train.jsonl``, ``dpo_val.jsonl`` when pairs are
given) plus ``manifest.json`` (``warpstate-posttrain-data-v1``) carrying the tokenizer hash, the
renderer hash, ``max_length`` and per-file SHA-256 / row / token counts that training verifies
by exact re-encoding (reference posttrain.py:117-156, ops/dpo_data.py:37-78).  Conversations
longer than ``--max-length`` are dropped and counted, never truncated.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from warpstate_ai_b200.data.prepare_posttrain import main  # noqa: E402

if __name__ == "__main__":
    main()
