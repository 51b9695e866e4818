"""The frozen-reference score cache of DPO (`train/reference_cache.py`): sharded scoring, resume, merge, verification.

Layout and guarantees as in the reference (dpo.py:100-128, 224-329); the scorer here is a pure function of the record,
so that any split over ranks and any interruption must reproduce the same table.
"""
import json

import numpy as np
import pytest

from warpstate_ai_b200.train.reference_cache import CACHE_FORMAT, ReferenceScoreCache, Shard, identity_digest
from warpstate_ai_b200.utils.io import digest

IDENTITY = {"weights": "aa", "data": "bb", "settings": {"objective": "length-normalized-dpo", "max_tokens": 64}, "world": 2}
TRAIN = [{"id": i} for i in range(11)]
VAL = [{"id": 100 + i} for i in range(3)]


def expected(records):
    return np.array([[-(r["id"] + 0.25), -(2 * r["id"] + 0.5)] for r in records], dtype=np.float64).reshape(-1, 2)


def score_batch(rows):
    return expected(rows)


def never():
    return False


def run_ranks(directory, world, mb, identity=IDENTITY, should_stop=never, scorer=score_batch):
    caches = [ReferenceScoreCache(directory, identity, (len(TRAIN), len(VAL))) for _ in range(world)]
    finished = []
    for rank, cache in enumerate(caches):
        cache.claim(rank)
    for rank, cache in enumerate(caches):
        finished.append(cache.score((TRAIN, VAL), scorer, mb, rank, world, should_stop, report_every=2))
    return caches, finished


@pytest.mark.parametrize("world, mb", [(1, 4), (2, 2), (3, 2), (2, 16), (4, 1)])
def test_any_split_over_ranks_gives_the_same_sealed_table(tmp_path, capsys, world, mb):
    caches, finished = run_ranks(tmp_path / "cache", world, mb)
    assert finished == [True] * world and not caches[0].sealed
    caches[0].merge(world)
    assert caches[0].sealed
    for cache in caches:
        train, val, manifest_hash = cache.verify()
        assert np.array_equal(train, expected(TRAIN)) and np.array_equal(val, expected(VAL))
        assert train.dtype == np.float64 and manifest_hash == digest(tmp_path / "cache" / "manifest.json")
    manifest = json.loads((tmp_path / "cache" / "manifest.json").read_text())
    assert manifest["format"] == CACHE_FORMAT and manifest["complete"] is True
    assert manifest["identity_sha256"] == identity_digest(IDENTITY)
    assert manifest["files"]["train.npy"] == {"sha256": digest(tmp_path / "cache" / "train.npy"), "rows": 11}
    events = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert events and all(e["event"] == "reference_progress" for e in events)
    last_of_rank0 = [e for e in events if e["rank"] == 0 and e["split"] == "train"][-1]
    assert last_of_rank0["batches"] == last_of_rank0["total_batches"]


def test_build_runs_claim_score_merge_verify(tmp_path):
    marks = []
    cache = ReferenceScoreCache(tmp_path / "cache", IDENTITY, (len(TRAIN), len(VAL)))
    train, val, _ = cache.build((TRAIN, VAL), score_batch, 4, 0, 1, never, lambda: marks.append("barrier"))
    assert marks == ["barrier"] * 3
    assert np.array_equal(train, expected(TRAIN)) and np.array_equal(val, expected(VAL))
    assert json.loads((tmp_path / "cache" / "identity.json").read_text()) == IDENTITY


def test_an_interrupted_rank_resumes_without_scoring_a_pair_twice(tmp_path):
    scored = []

    def counting(rows):
        scored.extend(r["id"] for r in rows)
        return expected(rows)

    calls = {"n": 0}

    def stop_on_third_batch():
        calls["n"] += 1
        return calls["n"] == 3

    cache = ReferenceScoreCache(tmp_path / "cache", IDENTITY, (len(TRAIN), len(VAL)))
    cache.claim(0)
    assert cache.score((TRAIN, VAL), counting, 2, 0, 1, stop_on_third_batch, report_every=100) is False
    assert scored == [0, 1, 2, 3]                                       # two batches, then the stop was honoured
    kept = Shard(tmp_path / "cache" / "train-rank-0.npz", cache.tag, len(TRAIN), 2, 0, 1)
    assert kept.done == 2 and kept.indices == [0, 1, 2, 3]
    assert cache.build((TRAIN, VAL), counting, 2, 0, 1, never, lambda: None) is not None
    assert sorted(scored) == sorted([r["id"] for r in TRAIN + VAL])     # everything once, nothing twice
    train, val, _ = cache.verify()
    assert np.array_equal(train, expected(TRAIN)) and np.array_equal(val, expected(VAL))


def test_build_returns_none_when_interrupted(tmp_path):
    cache = ReferenceScoreCache(tmp_path / "cache", IDENTITY, (len(TRAIN), len(VAL)))
    assert cache.build((TRAIN, VAL), score_batch, 2, 0, 1, lambda: True, lambda: None) is None
    assert not cache.sealed


def test_a_non_finite_score_stops_the_build(tmp_path):
    def broken(rows):
        values = expected(rows)
        values[0, 1] = np.nan
        return values

    cache = ReferenceScoreCache(tmp_path / "cache", IDENTITY, (len(TRAIN), len(VAL)))
    cache.claim(0)
    with pytest.raises(RuntimeError, match="non-finite"):
        cache.score((TRAIN, VAL), broken, 2, 0, 1, never)


def test_another_identity_neither_resumes_nor_verifies(tmp_path):
    caches, _ = run_ranks(tmp_path / "cache", 2, 2)
    other_identity = dict(IDENTITY, weights="cc")
    other = ReferenceScoreCache(tmp_path / "cache", other_identity, (len(TRAIN), len(VAL)))
    with pytest.raises(ValueError, match="partial cache of another identity"):
        other.claim(0)
    with pytest.raises(ValueError, match="another identity"):
        other.score((TRAIN, VAL), score_batch, 2, 0, 2, never)
    with pytest.raises(ValueError, match="another identity"):
        other.merge(2)
    caches[0].merge(2)
    with pytest.raises(ValueError, match="another fixed-reference identity"):
        other.verify()
    assert identity_digest(IDENTITY) != identity_digest(other_identity)
    assert identity_digest({"b": 1, "a": 2}) == identity_digest({"a": 2, "b": 1})       # key order does not matter
    with pytest.raises(ValueError):
        identity_digest({"x": float("nan")})


def test_merge_needs_every_pair_exactly_once(tmp_path):
    directory = tmp_path / "cache"
    caches, _ = run_ranks(directory, 2, 2)
    # rank 1's shard replaced by a copy of rank 0's: repeated pairs
    (directory / "train-rank-1.npz").write_bytes((directory / "train-rank-0.npz").read_bytes())
    with pytest.raises(ValueError, match="repeats pairs"):
        caches[0].merge(2)
    # a world of one more rank than scored: a shard is missing altogether
    caches, _ = run_ranks(tmp_path / "second", 2, 2)
    with pytest.raises(FileNotFoundError):
        caches[0].merge(3)
    # a shard that stopped early leaves holes
    directory = tmp_path / "third"
    cache = ReferenceScoreCache(directory, IDENTITY, (len(TRAIN), len(VAL)))
    cache.claim(0)
    calls = {"n": 0}

    def stop_late():
        calls["n"] += 1
        return calls["n"] == 4

    cache.score((TRAIN, VAL), score_batch, 2, 0, 1, stop_late)
    Shard(directory / "val-rank-0.npz", cache.tag, len(VAL), 2, 0, 1).write()
    with pytest.raises(ValueError, match="do not cover every pair"):
        cache.merge(1)
    assert not cache.sealed


@pytest.mark.parametrize("damage", ["flip", "truncate", "swap", "link", "incomplete", "nan"])
def test_a_sealed_cache_that_was_touched_is_refused(tmp_path, damage):
    directory = tmp_path / "cache"
    caches, _ = run_ranks(directory, 1, 4)
    cache = caches[0]
    cache.merge(1)
    cache.verify()
    train = directory / "train.npy"
    manifest_path = directory / "manifest.json"
    if damage == "flip":
        raw = bytearray(train.read_bytes())
        raw[-1] ^= 1
        train.write_bytes(bytes(raw))
    elif damage == "truncate":
        np.save(train, expected(TRAIN)[:-1])
    elif damage == "swap":
        train.write_bytes((directory / "val.npy").read_bytes())
    elif damage == "link":
        moved = tmp_path / "elsewhere.npy"
        train.rename(moved)
        train.symlink_to(moved)
    elif damage == "incomplete":
        manifest = json.loads(manifest_path.read_text())
        manifest["complete"] = False
        manifest_path.write_text(json.dumps(manifest))
    else:   # a table that is consistent with its manifest but holds a non-finite score
        table = expected(TRAIN)
        table[3, 0] = np.inf
        np.save(train, table)
        manifest = json.loads(manifest_path.read_text())
        manifest["files"]["train.npy"]["sha256"] = digest(train)
        manifest_path.write_text(json.dumps(manifest))
    with pytest.raises(ValueError):
        cache.verify()


def test_a_shard_whose_counter_and_contents_disagree_is_refused(tmp_path):
    path = tmp_path / "train-rank-0.npz"
    good = Shard(path, "tag", 10, 2, 0, 2)
    assert good.starts == [0, 4, 8] and good.batch(2) == [8, 9]
    good.add(0, expected([{"id": 0}, {"id": 1}]))
    good.write()
    again = Shard(path, "tag", 10, 2, 0, 2)
    assert again.done == 1 and again.indices == [0, 1] and np.array_equal(np.asarray(again.scores), expected([{"id": 0}, {"id": 1}]))
    with pytest.raises(ValueError, match="another identity"):
        Shard(path, "other", 10, 2, 0, 2)
    with pytest.raises(ValueError, match="does not continue"):
        Shard(path, "tag", 10, 2, 1, 2)             # the same file read as another rank's
    np.savez(path, identity="tag", batches=2, indices=np.array([0, 1]), scores=expected([{"id": 0}, {"id": 1}]))
    with pytest.raises(ValueError, match="does not continue"):
        Shard(path, "tag", 10, 2, 0, 2)
