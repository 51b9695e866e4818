"""Corpus preparation: stream documents, tokenise with SentencePiece, write little-endian uint16
``train.bin`` / ``val.bin`` with a resumable, commit-based protocol.

Behavioural contract of the reference (run_40b.py:227-344):

* every document is encoded separately and terminated with EOS;
* a document belongs to the validation split iff ``int(sha256(text)[:8], little) % 1000 == 0``;
  training never sees hold-out documents;
* progress is committed every 8 M tokens: token files are fsynced, then the dataset iterator
  state and the token counts are published atomically; on restart uncommitted bytes are
  truncated away, so an interrupted preparation resumes byte-identically;
* the final ``manifest.json`` records the signature (recipe, dataset, revision, token budgets,
  tokenizer hash, dtype, hold-out rule) and the SHA-256 of both files; training refuses data
  whose manifest does not match the requested settings.

The HuggingFace `datasets` / `huggingface_hub` packages are imported only inside `prepare`
(they are not needed for training and can be replaced by a fake module in tests).
"""
from __future__ import annotations

import contextlib
import hashlib
import itertools
import json
import os
import pickle
import shutil
import time
from pathlib import Path

from ..utils.io import atomic_write, digest

RECIPE = "fineweb-edu-sentencepiece-uint16-v1"
COMMIT_TOKENS = 8_000_000
HOLDOUT_RULE = "sha256(raw-text) modulo 1000 == 0; train excludes all holdout documents"


def data_signature(a) -> dict:
    return {"recipe": RECIPE, "dataset": a.dataset, "config": a.dataset_config, "requested_revision": a.revision,
            "train_tokens": a.train_tokens, "val_tokens": a.val_tokens, "tokenizer_sha256": digest(a.tokenizer),
            "dtype": "<u2", "holdout": HOLDOUT_RULE}


def is_holdout(text: str) -> bool:
    return int.from_bytes(hashlib.sha256(text.encode("utf-8")).digest()[:8], "little") % 1000 == 0


def check_manifest(a) -> dict:
    directory = a.work_dir / "data"
    manifest = json.loads((directory / "manifest.json").read_text())
    if manifest["signature"] != data_signature(a) or not manifest["complete"]:
        raise ValueError("Prepared dataset does not match requested settings/tokenizer")
    for split, count in (("train", a.train_tokens), ("val", a.val_tokens)):
        if (directory / f"{split}.bin").stat().st_size != count * 2:
            raise ValueError("Invalid token file size: " + split)
        if getattr(a, "verify_data", False) and digest(directory / f"{split}.bin") != manifest["sha256"][split]:
            raise ValueError("Dataset checksum mismatch: " + split)
    return manifest


def prepare(a, stop_requested=lambda: False) -> bool:
    """Returns True when the corpus is complete, False when stopped after a commit."""
    import datasets
    import numpy as np
    import sentencepiece as spm
    from huggingface_hub import HfApi

    directory = a.work_dir / "data"
    directory.mkdir(parents=True, exist_ok=True)
    if (directory / "manifest.json").exists():
        check_manifest(a)
        print("Dataset already complete and matches this tokenizer.", flush=True)
        return True
    signature = data_signature(a)
    sp = spm.SentencePieceProcessor(model_file=str(a.tokenizer))
    if sp.vocab_size() > 65536 or sp.eos_id() < 0:
        raise ValueError("Need a uint16-compatible tokenizer with EOS")
    progress = directory / "prepare-state.pkl"

    def publish(state):
        atomic_write(progress, lambda f: pickle.dump(state, f, protocol=pickle.HIGHEST_PROTOCOL))

    if progress.exists():
        with progress.open("rb") as f:
            state = pickle.load(f)
        if state["signature"] != signature or state["datasets_version"] != datasets.__version__:
            raise ValueError("Preparation settings/version changed; use the original environment or a different "
                             "work directory")
    else:
        if any((directory / f"{s}.bin").exists() for s in ("train", "val")):
            raise RuntimeError("Token files without preparation state: refusing to overwrite")
        state = {"signature": signature, "datasets_version": datasets.__version__, "train": 0, "val": 0,
                 "revision": HfApi().dataset_info(a.dataset, revision=a.revision).sha, "iterator": None,
                 "documents": 0}
        publish(state)
    budget = {"train": a.train_tokens, "val": a.val_tokens}
    remaining = 2 * (a.train_tokens + a.val_tokens - state["train"] - state["val"])
    reserve = 0 if getattr(a, "test_small_gpu", False) else 70 * 1024 ** 3
    if shutil.disk_usage(directory).free < remaining + reserve:
        raise RuntimeError(f"Need {(remaining + reserve) / 1024 ** 3:.1f} GiB free for remaining data and checkpoints")
    ds = datasets.load_dataset(a.dataset, name=a.dataset_config, split="train", streaming=True,
                               revision=state["revision"])
    print(f"Preparing {a.dataset}/{a.dataset_config} at {state['revision']}; "
          f"resuming train={state['train']:,}, val={state['val']:,}", flush=True)
    if state["iterator"] is not None:
        ds.load_state_dict(state["iterator"])
    iterator = iter(ds)
    with contextlib.ExitStack() as stack:
        stack.callback(lambda: getattr(iterator, "close", lambda: None)())
        files = {}
        for split in ("train", "val"):
            path = directory / f"{split}.bin"
            if not path.exists() and state[split]:
                raise RuntimeError("Missing committed data: " + split)
            f = stack.enter_context(path.open("r+b" if path.exists() else "w+b"))
            if path.stat().st_size < state[split] * 2:
                raise RuntimeError("Truncated committed data: " + split)
            f.truncate(state[split] * 2)  # drop bytes written after the last commit
            f.seek(state[split] * 2)
            files[split] = f

        def commit():
            for f in files.values():
                f.flush()
                os.fsync(f.fileno())
            state["iterator"] = ds.state_dict()
            publish(state)

        last_commit = start_count = state["train"] + state["val"]
        started = time.monotonic()
        while any(state[s] < budget[s] for s in budget):
            rows = list(itertools.islice(iterator, a.documents_per_batch))
            if not rows:
                commit()
                raise RuntimeError("Source exhausted before the requested token budget; do not repeat it silently")
            texts = [row["text"] for row in rows]
            for text, ids in zip(texts, sp.encode(texts, out_type=int, num_threads=a.workers)):
                state["documents"] += 1
                if not text.strip():
                    continue
                split = "val" if is_holdout(text) else "train"
                room = budget[split] - state[split]
                if room <= 0:
                    continue
                tokens = np.asarray((ids + [sp.eos_id()])[:room], dtype="<u2")
                files[split].write(tokens.tobytes())
                state[split] += len(tokens)
            count = state["train"] + state["val"]
            stopping = stop_requested()
            if stopping or count - last_commit >= COMMIT_TOKENS:
                commit()
                last_commit = count
                print(f"prepared train={state['train']:,}/{a.train_tokens:,}, val={state['val']:,}; "
                      f"{(count - start_count) / max(time.monotonic() - started, 1):,.0f} tokens/s", flush=True)
            if stopping:
                return False
        commit()
    manifest = {"signature": signature, "source_revision": state["revision"], "complete": True,
                "documents_read": state["documents"], "datasets_version": datasets.__version__,
                "sha256": {s: digest(directory / f"{s}.bin") for s in ("train", "val")},
                "source_url": "https://huggingface.co/datasets/" + a.dataset}
    atomic_write(directory / "manifest.json", lambda f: f.write(json.dumps(manifest, indent=2).encode()))
    check_manifest(a)
    print("Prepared the exact requested token counts.", flush=True)
    return True


def write_synthetic_corpus(work_dir: Path, tokenizer: Path, train_tokens: int, val_tokens: int, vocab: int,
                           seed: int = 0, dataset: str = "synthetic/uniform", config: str = "none",
                           revision: str = "0") -> dict:
    """A complete ``data/`` directory of uniform-random tokens with a valid manifest, for tests
    and benchmarks that have no network (same file layout and manifest schema as `prepare`)."""
    import numpy as np
    from types import SimpleNamespace

    directory = Path(work_dir) / "data"
    directory.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    for split, count in (("train", train_tokens), ("val", val_tokens)):
        rng.integers(0, vocab, size=count, dtype=np.uint16).astype("<u2").tofile(directory / f"{split}.bin")
    a = SimpleNamespace(dataset=dataset, dataset_config=config, revision=revision, train_tokens=train_tokens,
                        val_tokens=val_tokens, tokenizer=Path(tokenizer), work_dir=Path(work_dir))
    manifest = {"signature": data_signature(a), "source_revision": revision, "complete": True, "documents_read": 0,
                "datasets_version": "none", "sha256": {s: digest(directory / f"{s}.bin") for s in ("train", "val")},
                "source_url": "synthetic"}
    atomic_write(directory / "manifest.json", lambda f: f.write(json.dumps(manifest, indent=2).encode()))
    return manifest
