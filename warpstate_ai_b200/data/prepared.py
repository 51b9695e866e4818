"""Reading a prepared post-training data directory (``manifest.json`` + JSON-lines splits).

The directory format is the reference's ``warpstate-posttrain-data-v1`` (reference
ops/posttrain_data.py:103-147, ops/dpo_data.py:37-78): the manifest is complete, names the tokenizer
and renderer hashes and the maximum length it was prepared for, and lists every split with its
SHA-256, row count and token totals; every row carries its own token counts.  A loader re-encodes every
row and refuses the directory on the first disagreement.

`PreparedDirectory` is that contract once, for SFT conversations and DPO pairs alike: the two loaders
pass a row encoder and a function that measures an encoded record.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable

from ..utils.io import digest

DATA_FORMAT = "warpstate-posttrain-data-v1"


class PreparedDirectory:
    def __init__(self, data_dir, tokenizer_hash: str, renderer_hash: str, sequence_length: int):
        self.directory = Path(data_dir)
        self.manifest_path = self.directory / "manifest.json"
        self.manifest = json.loads(self.manifest_path.read_text())
        expected = (("format", DATA_FORMAT, "is not prepared post-training data"),
                    ("complete", True, "was not finished by its preparation run"),
                    ("tokenizer_sha256", tokenizer_hash, "was prepared with another tokenizer"),
                    ("renderer_sha256", renderer_hash, "was prepared with another version of the renderer"),
                    ("max_length", sequence_length, "was prepared for another sequence length"))
        for key, want, complaint in expected:
            if self.manifest.get(key) != want:
                raise ValueError(f"{self.directory} {complaint} (manifest '{key}')")

    def manifest_digest(self) -> str:
        return digest(self.manifest_path)

    def split(self, filename: str, encode: Callable[[dict, int], object],
              measure: Callable[[dict, object], tuple[int, int] | None], progress_every: int = 0) -> list:
        """Encoded records of one split.  ``encode(row, line_number)`` renders a row; ``measure(row, record)``
        returns its ``(tokens, supervised tokens)`` after checking them against the row's own counts (it
        returns ``None`` when they disagree)."""
        entry = self.manifest.get("outputs", {}).get(filename)
        path = self.directory / filename
        if not entry or not path.is_file() or digest(path) != entry.get("sha256"):
            raise ValueError(f"{filename} is missing from {self.directory} or differs from its manifest entry")
        records, tokens, supervised = [], 0, 0
        with path.open() as lines:
            for number, line in enumerate(lines, 1):
                row = json.loads(line)
                record = encode(row, number)
                counts = measure(row, record)
                if counts is None:
                    raise ValueError(f"{filename}:{number}: the row's token counts do not match its encoding")
                tokens += counts[0]
                supervised += counts[1]
                records.append(record)
                if progress_every and number % progress_every == 0:
                    print(json.dumps({"event": "data_validation", "file": filename, "rows": number}), flush=True)
        if not records or len(records) != entry.get("rows"):
            raise ValueError(f"{filename}: no rows, or not the {entry.get('rows')} rows its manifest promises")
        if (tokens, supervised) != (entry.get("tokens"), entry.get("supervised_tokens")):
            raise ValueError(f"{filename}: token totals differ from the manifest")
        return records
