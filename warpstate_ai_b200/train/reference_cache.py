"""Scores of the frozen DPO reference model, computed once and kept on disk.

The cache directory (format ``warpstate-dpo-reference-v1``, the reference's layout, reference
dpo.py:100-128, 224-329) holds ``train.npy`` / ``val.npy`` -- float64 ``[pairs, 2]`` response log-probability
sums of (chosen, rejected) -- and a ``manifest.json`` binding them to an *identity*: hashes of the weights,
the data, the tokenizer, the renderer and the scoring sources, the settings that affect scoring, and the
world size.  While it is being built it holds ``identity.json`` and one resumable ``<split>-rank-<r>.npz``
shard per rank (identity hash, batches done, pair indices, scores).

`ReferenceScoreCache` has three verbs: `verify` (an existing cache answers this identity), `score`
(this rank's shards, resumable, interruptible between batches) and `merge` (rank 0 turns complete shards into
the sealed arrays).  `build` strings them together for a multi-rank job.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
import time
from pathlib import Path

import numpy as np

from ..utils.io import atomic_json, digest

CACHE_FORMAT = "warpstate-dpo-reference-v1"
SPLITS = ("train", "val")


def identity_digest(identity) -> str:
    text = json.dumps(identity, sort_keys=True, separators=(",", ":"), allow_nan=False)
    return hashlib.sha256(text.encode()).hexdigest()


def atomic_array(path, array) -> None:
    staging = Path(f"{path}.tmp")
    with staging.open("wb") as stream:
        np.save(stream, array, allow_pickle=False)
        stream.flush()
        os.fsync(stream.fileno())
    os.replace(staging, path)


class Shard:
    """One rank's scores of one split: batches ``rank, rank + world, ...`` of ``mb`` pairs each."""

    def __init__(self, path: Path, tag: str, rows: int, mb: int, rank: int, world: int):
        self.path, self.tag, self.rows, self.mb = path, tag, rows, mb
        self.starts = list(range(rank * mb, rows, world * mb))
        self.done = 0
        self.indices: list[int] = []
        self.scores: list = []
        if path.exists():
            with np.load(path, allow_pickle=False) as stored:
                if str(stored["identity"]) != tag:
                    raise ValueError(f"{path.name} belongs to a cache with another identity")
                self.done = int(stored["batches"])
                self.indices, self.scores = stored["indices"].tolist(), stored["scores"].tolist()
            if self.indices != [i for b in range(self.done) for i in self.batch(b)] or len(self.scores) != len(self.indices):
                raise ValueError(f"{path.name} does not continue where its batch counter says")

    def batch(self, number: int) -> list[int]:
        begin = self.starts[number]
        return list(range(begin, min(begin + self.mb, self.rows)))

    def add(self, number: int, values) -> None:
        self.indices.extend(self.batch(number))
        self.scores.extend(values.tolist())
        self.done = number + 1

    def write(self) -> None:
        staging = Path(f"{self.path}.tmp")
        with staging.open("wb") as stream:
            np.savez(stream, identity=self.tag, batches=self.done, indices=np.asarray(self.indices, dtype=np.int64),
                     scores=np.asarray(self.scores, dtype=np.float64).reshape(-1, 2))
            stream.flush()
            os.fsync(stream.fileno())
        os.replace(staging, self.path)


class ReferenceScoreCache:
    def __init__(self, directory, identity: dict, sizes):
        self.directory, self.identity, self.sizes = Path(directory), identity, tuple(sizes)
        self.tag = identity_digest(identity)

    @property
    def sealed(self) -> bool:
        return (self.directory / "manifest.json").exists()

    # ------------------------------------------------------------------ verify
    def verify(self):
        """-> (train scores, validation scores, SHA-256 of the manifest); raises ValueError on any mismatch."""
        manifest_path = self.directory / "manifest.json"
        manifest = json.loads(manifest_path.read_text())
        stated = (manifest.get("format"), manifest.get("complete"), manifest.get("identity"), manifest.get("identity_sha256"))
        if stated != (CACHE_FORMAT, True, self.identity, self.tag):
            raise ValueError(f"the reference cache in {self.directory} was built for another fixed-reference identity "
                             "or was never completed")
        arrays = []
        for split, rows in zip(SPLITS, self.sizes):
            path = self.directory / f"{split}.npy"
            entry = manifest.get("files", {}).get(path.name, {})
            if not path.is_file() or path.is_symlink() or entry.get("rows") != rows or digest(path) != entry.get("sha256"):
                raise ValueError(f"{path.name} is missing or is not the file its cache manifest describes")
            scores = np.load(path, allow_pickle=False, mmap_mode="r")
            if scores.dtype != np.float64 or scores.shape != (rows, 2) or not np.isfinite(scores).all():
                raise ValueError(f"{path.name} does not hold finite float64 scores of {rows} pairs")
            arrays.append(scores)
        return arrays[0], arrays[1], digest(manifest_path)

    # ------------------------------------------------------------------ score
    def claim(self, rank: int) -> None:
        """Bind a cache under construction to this identity (rank 0 writes the marker)."""
        self.directory.mkdir(parents=True, exist_ok=True)
        marker = self.directory / "identity.json"
        if marker.exists() and json.loads(marker.read_text()) != self.identity:
            raise ValueError(f"{self.directory} holds a partial cache of another identity")
        if rank == 0:
            atomic_json(marker, self.identity)

    def score(self, records, score_batch, mb: int, rank: int, world: int, should_stop, report_every: int = 128) -> bool:
        """Fill this rank's shards.  ``score_batch(rows) -> float64 [len(rows), 2]``.  ``should_stop()`` is
        called once per global batch on every rank alike (it may be a collective).  False = interrupted."""
        began = time.monotonic()
        for split, rows in zip(SPLITS, records):
            shard = Shard(self.directory / f"{split}-rank-{rank}.npz", self.tag, len(rows), mb, rank, world)
            for number in range(math.ceil(len(rows) / (world * mb))):
                if should_stop():
                    shard.write()
                    return False
                if number < shard.done or number >= len(shard.starts):
                    continue
                values = score_batch([rows[i] for i in shard.batch(number)])
                if not np.isfinite(values).all():
                    raise RuntimeError("the frozen reference produced a non-finite score")
                shard.add(number, values)
                if shard.done % report_every == 0 or shard.done == len(shard.starts):
                    shard.write()
                    print(json.dumps(dict(event="reference_progress", rank=rank, split=split, batches=shard.done,
                                          total_batches=len(shard.starts), scored_pairs=len(shard.scores),
                                          elapsed_seconds=time.monotonic() - began)), flush=True)
            shard.write()
        return True

    # ------------------------------------------------------------------ merge
    def merge(self, world: int) -> None:
        files = {}
        for split, rows in zip(SPLITS, self.sizes):
            table = np.full((rows, 2), np.nan, dtype=np.float64)
            filled = np.zeros(rows, dtype=np.bool_)
            for owner in range(world):
                with np.load(self.directory / f"{split}-rank-{owner}.npz", allow_pickle=False) as part:
                    if str(part["identity"]) != self.tag:
                        raise ValueError(f"the {split} shard of rank {owner} has another identity")
                    where = part["indices"]
                    if filled[where].any():
                        raise ValueError(f"the {split} shard of rank {owner} repeats pairs of another shard")
                    table[where] = part["scores"]
                    filled[where] = True
            if not (filled.all() and np.isfinite(table).all()):
                raise ValueError(f"the {split} shards do not cover every pair")
            path = self.directory / f"{split}.npy"
            atomic_array(path, table)
            files[path.name] = dict(sha256=digest(path), rows=rows)
        atomic_json(self.directory / "manifest.json", dict(format=CACHE_FORMAT, complete=True, identity=self.identity,
                                                           identity_sha256=self.tag, files=files))

    def build(self, records, score_batch, mb: int, rank: int, world: int, should_stop, barrier):
        """Score, merge on rank 0, verify everywhere.  Returns `verify()`'s result, or None when interrupted."""
        self.claim(rank)
        barrier()
        if not self.score(records, score_batch, mb, rank, world, should_stop):
            return None
        barrier()
        if rank == 0:
            self.merge(world)
        barrier()
        return self.verify()
