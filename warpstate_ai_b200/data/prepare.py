"""Corpus preparation: stream documents, tokenise them with SentencePiece and write little-endian
uint16 ``train.bin`` / ``val.bin`` with a commit log that makes an interrupted run resume byte for byte.

What the files must look like (the reference's recipe, run_40b.py:227-344, is the format):

* each document is encoded on its own and ends with EOS;
* a document is held out for validation iff the first 8 bytes (little endian) of the SHA-256 of its
  text are divisible by 1000; held-out documents never reach the training file;
* ``manifest.json`` carries the signature of the request (recipe, dataset, revision, token budgets,
  tokenizer hash, dtype, hold-out rule), the resolved source revision and the SHA-256 of both files;
  training refuses a directory whose manifest does not answer the request.

How this module writes them:

* `SplitFile` is one token file with a *committed length*; opening it discards whatever lies beyond;
* `CommitLog` is the small pickled record (``prepare-state.pkl``) of committed lengths, document count,
  source revision and the dataset iterator's own state, replaced atomically;
* `CorpusWriter` pulls batches of documents, routes each to its split until the split's budget is
  full, and commits (fsync the files, then replace the log) every `COMMIT_TOKENS` tokens and when asked
  to stop.  A crash between the two halves of a commit loses at most uncommitted bytes.

The HuggingFace ``datasets`` / ``huggingface_hub`` packages are imported only by `prepare` (training
does not need them; tests substitute small fakes).
"""
from __future__ import annotations

import hashlib
import itertools
import json
import os
import pickle
import shutil
import time
from pathlib import Path

from ..utils.io import atomic_write, digest

RECIPE = 1          # version of the file format below; run_40b.py:22 writes the same number, so either side reads the other's corpus
COMMIT_TOKENS = 8_000_000
HOLDOUT_RULE = "sha256(raw-text) modulo 1000 == 0; train excludes all holdout documents"
SPLITS = ("train", "val")
TOKEN_BYTES = 2


def data_signature(a) -> dict:
    return {"recipe": RECIPE, "dataset": a.dataset, "config": a.dataset_config, "requested_revision": a.revision,
            "train_tokens": a.train_tokens, "val_tokens": a.val_tokens, "tokenizer_sha256": digest(a.tokenizer),
            "dtype": "<u2", "holdout": HOLDOUT_RULE}


def is_holdout(text: str) -> bool:
    head = hashlib.sha256(text.encode("utf-8")).digest()[:8]
    return int.from_bytes(head, "little") % 1000 == 0


def _data_dir(a) -> Path:
    return Path(a.work_dir) / "data"


def _publish_manifest(directory: Path, signature: dict, revision, documents: int, datasets_version: str,
                      source_url: str) -> dict:
    manifest = {"signature": signature, "source_revision": revision, "complete": True, "documents_read": documents,
                "datasets_version": datasets_version,
                "sha256": {split: digest(directory / f"{split}.bin") for split in SPLITS}, "source_url": source_url}
    atomic_write(directory / "manifest.json", lambda f: f.write(json.dumps(manifest, indent=2).encode()))
    return manifest


def check_manifest(a) -> dict:
    """The manifest of ``<work_dir>/data`` if it answers the request ``a``; raises ValueError otherwise."""
    directory = _data_dir(a)
    manifest = json.loads((directory / "manifest.json").read_text())
    if not manifest["complete"] or manifest["signature"] != data_signature(a):
        raise ValueError("the prepared corpus was made for other settings or another tokenizer")
    budgets = {"train": a.train_tokens, "val": a.val_tokens}
    for split in SPLITS:
        path = directory / f"{split}.bin"
        if path.stat().st_size != budgets[split] * TOKEN_BYTES:
            raise ValueError(f"{path.name} does not hold exactly {budgets[split]} tokens")
        if getattr(a, "verify_data", False) and digest(path) != manifest["sha256"][split]:
            raise ValueError(f"{path.name} does not match the checksum in its manifest")
    return manifest


class SplitFile:
    """A token file opened at its committed length (bytes beyond it are dropped)."""

    def __init__(self, path: Path, committed_tokens: int):
        self.path = path
        size = committed_tokens * TOKEN_BYTES
        if not path.exists():
            if committed_tokens:
                raise RuntimeError(f"{path.name}: {committed_tokens} tokens were committed but the file is gone")
            path.touch()
        if path.stat().st_size < size:
            raise RuntimeError(f"{path.name} is shorter than its committed length")
        self.handle = path.open("r+b")
        self.handle.truncate(size)
        self.handle.seek(size)

    def append(self, tokens) -> None:
        self.handle.write(tokens.tobytes())

    def sync(self) -> None:
        self.handle.flush()
        os.fsync(self.handle.fileno())

    def close(self) -> None:
        self.handle.close()


class CommitLog:
    """``prepare-state.pkl``: {signature, datasets_version, train, val, revision, iterator, documents}."""

    def __init__(self, path: Path):
        self.path = path
        self.record: dict | None = None

    def load(self) -> bool:
        if not self.path.exists():
            return False
        with self.path.open("rb") as stream:
            self.record = pickle.load(stream)
        return True

    def start(self, signature: dict, datasets_version: str, revision) -> None:
        self.record = {"signature": signature, "datasets_version": datasets_version, "train": 0, "val": 0,
                       "revision": revision, "iterator": None, "documents": 0}
        self.write()

    def write(self) -> None:
        atomic_write(self.path, lambda stream: pickle.dump(self.record, stream, protocol=pickle.HIGHEST_PROTOCOL))

    def written(self) -> int:
        return sum(self.record[split] for split in SPLITS)


class CorpusWriter:
    def __init__(self, directory: Path, log: CommitLog, budgets: dict, tokenizer, dataset, workers: int,
                 documents_per_batch: int):
        self.log, self.budgets, self.tokenizer, self.dataset = log, budgets, tokenizer, dataset
        self.workers, self.batch = workers, documents_per_batch
        self.files = {split: SplitFile(directory / f"{split}.bin", log.record[split]) for split in SPLITS}
        if log.record["iterator"] is not None:
            dataset.load_state_dict(log.record["iterator"])
        self.documents = iter(dataset)

    def close(self) -> None:
        closer = getattr(self.documents, "close", None)
        if closer is not None:
            closer()
        for f in self.files.values():
            f.close()

    def full(self) -> bool:
        return all(self.log.record[split] >= self.budgets[split] for split in SPLITS)

    def commit(self) -> None:
        for f in self.files.values():
            f.sync()
        self.log.record["iterator"] = self.dataset.state_dict()
        self.log.write()

    def take_batch(self) -> None:
        """Route one batch of documents; raises when the source is exhausted."""
        import numpy as np
        rows = list(itertools.islice(self.documents, self.batch))
        if not rows:
            self.commit()
            raise RuntimeError("the source ran out of documents before the token budget was met "
                               "(repeating it silently would duplicate data)")
        texts = [row["text"] for row in rows]
        encoded = self.tokenizer.encode(texts, out_type=int, num_threads=self.workers)
        eos = self.tokenizer.eos_id()
        record = self.log.record
        for text, ids in zip(texts, encoded):
            record["documents"] += 1
            if not text.strip():
                continue
            split = "val" if is_holdout(text) else "train"
            room = self.budgets[split] - record[split]
            if room > 0:
                piece = np.asarray((ids + [eos])[:room], dtype="<u2")
                self.files[split].append(piece)
                record[split] += len(piece)

    def run(self, stop_requested) -> bool:
        """True when both budgets are full; False when stopped (after a commit)."""
        begun_at, begun_with = time.monotonic(), self.log.written()
        since_commit = begun_with
        while not self.full():
            self.take_batch()
            now = self.log.written()
            stopping = bool(stop_requested())
            if stopping or now - since_commit >= COMMIT_TOKENS:
                self.commit()
                since_commit = now
                rate = (now - begun_with) / max(time.monotonic() - begun_at, 1)
                r = self.log.record
                print(f"prepared train={r['train']:,}/{self.budgets['train']:,}, val={r['val']:,}; {rate:,.0f} tokens/s",
                      flush=True)
            if stopping:
                return False
        self.commit()
        return True


def prepare(a, stop_requested=lambda: False) -> bool:
    """Returns True when the corpus is complete, False when stopped after a commit."""
    import datasets
    import sentencepiece as spm
    from huggingface_hub import HfApi

    directory = _data_dir(a)
    directory.mkdir(parents=True, exist_ok=True)
    if (directory / "manifest.json").exists():
        check_manifest(a)
        print("The corpus is already complete for this request and tokenizer.", flush=True)
        return True
    signature = data_signature(a)
    tokenizer = spm.SentencePieceProcessor(model_file=str(a.tokenizer))
    if tokenizer.vocab_size() > 1 << 16 or tokenizer.eos_id() < 0:
        raise ValueError("the tokenizer must fit uint16 token ids and define EOS")
    log = CommitLog(directory / "prepare-state.pkl")
    if log.load():
        if (log.record["signature"], log.record["datasets_version"]) != (signature, datasets.__version__):
            raise ValueError("an unfinished preparation with other settings or another datasets version lives in "
                             f"{directory}; finish it in its own environment or pick another work directory")
    else:
        if any((directory / f"{split}.bin").exists() for split in SPLITS):
            raise RuntimeError(f"{directory} holds token files but no preparation state; not overwriting them")
        log.start(signature, datasets.__version__, HfApi().dataset_info(a.dataset, revision=a.revision).sha)
    budgets = {"train": a.train_tokens, "val": a.val_tokens}
    still_needed = TOKEN_BYTES * (sum(budgets.values()) - log.written())
    headroom = 0 if getattr(a, "test_small_gpu", False) else 70 << 30      # room for checkpoints later
    if shutil.disk_usage(directory).free < still_needed + headroom:
        raise RuntimeError(f"need {(still_needed + headroom) / 2 ** 30:.1f} GiB of free disk for the rest of the corpus "
                           "and the checkpoints")
    revision = log.record["revision"]
    stream = datasets.load_dataset(a.dataset, name=a.dataset_config, split="train", streaming=True, revision=revision)
    print(f"Preparing {a.dataset}/{a.dataset_config} at {revision}; resuming train={log.record['train']:,}, "
          f"val={log.record['val']:,}", flush=True)
    writer = CorpusWriter(directory, log, budgets, tokenizer, stream, a.workers, a.documents_per_batch)
    try:
        finished = writer.run(stop_requested)
    finally:
        writer.close()
    if not finished:
        return False
    _publish_manifest(directory, signature, revision, log.record["documents"], datasets.__version__,
                      "https://huggingface.co/datasets/" + a.dataset)
    check_manifest(a)
    print("Prepared exactly the requested token counts.", flush=True)
    return True


def write_synthetic_corpus(work_dir: Path, tokenizer: Path, train_tokens: int, val_tokens: int, vocab: int,
                           seed: int = 0, dataset: str = "synthetic/uniform", config: str = "none",
                           revision: str = "0") -> dict:
    """A complete ``data/`` directory of uniform-random tokens with a valid manifest, for tests
    and benchmarks that have no network (same file layout and manifest schema as `prepare`)."""
    import numpy as np
    from types import SimpleNamespace

    request = SimpleNamespace(dataset=dataset, dataset_config=config, revision=revision, train_tokens=train_tokens,
                              val_tokens=val_tokens, tokenizer=Path(tokenizer), work_dir=Path(work_dir))
    directory = _data_dir(request)
    directory.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    for split, count in zip(SPLITS, (train_tokens, val_tokens)):
        rng.integers(0, vocab, size=count, dtype=np.uint16).astype("<u2").tofile(directory / f"{split}.bin")
    return _publish_manifest(directory, data_signature(request), revision, 0, "none", "synthetic")
