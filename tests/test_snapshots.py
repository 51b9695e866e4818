"""Sealed inference exports (`serve/snapshots.py`): what is published, what is refused, what survives a replaced source.

Guarantees restated from the reference (chat.py:37-151); the fixture is a hand-made training checkpoint of a tiny model.
"""
import json
import os
from dataclasses import asdict
from pathlib import Path

import pytest
import torch

from warpstate_ai_b200.ckpt.formats import CHAT_FORMAT, SERVER_FORMAT
from warpstate_ai_b200.config import WarpStateConfig
from warpstate_ai_b200.models.warpstate import WarpStateLM
from warpstate_ai_b200.serve import snapshots as S
from warpstate_ai_b200.utils.io import digest

TOK = Path(__file__).resolve().parents[1] / "tokenizer.model"


def tiny_config():
    return WarpStateConfig(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=4,
                           gradient_checkpointing=False, parallel_memory=True)


def training_checkpoint(step=7, tokens=112, seed=0):
    torch.manual_seed(seed)
    cfg = tiny_config()
    model = WarpStateLM(cfg)
    return {"format": SERVER_FORMAT, "signature": {"data": {"signature": {"tokenizer_sha256": digest(TOK)}}},
            "config": asdict(cfg), "model": model.state_dict(), "optimizer": {"state": {0: {"exp_avg": torch.ones(3)}}},
            "step": step, "tokens_seen": tokens, "val_loss": 10.25}


@pytest.fixture()
def run(tmp_path):
    source = tmp_path / "run" / "latest.pt"
    source.parent.mkdir()
    state = training_checkpoint()
    torch.save(state, source)
    return tmp_path, source, state


def test_export_holds_the_model_only_and_is_sealed_read_only(run):
    tmp, source, state = run
    before = digest(source)
    store = S.SnapshotStore(tmp / "snaps", TOK)
    exported = store.export(source)
    assert exported.name == "model.pt" and exported.parent.parent == tmp / "snaps" and exported.parent.name.startswith("step-7-")
    assert oct(exported.stat().st_mode & 0o777) == "0o444"
    assert digest(source) == before and not source.with_name("snapshot.json").exists()     # the source is only read
    payload = torch.load(exported, map_location="cpu", weights_only=False)
    assert "optimizer" not in payload and "signature" not in payload
    assert payload["format"] == CHAT_FORMAT and payload["inference_only"] is True
    assert (payload["step"], payload["tokens_seen"], payload["val_loss"]) == (7, 112, 10.25)
    for key, value in state["model"].items():
        assert torch.equal(payload["model"][key], value)
    seal = json.loads(exported.with_name("snapshot.json").read_text())
    assert seal["snapshot_sha256"] == digest(exported) and seal["snapshot_bytes"] == exported.stat().st_size
    st = source.stat()
    assert seal["source"] == {"path": str(source.resolve()), "device": st.st_dev, "inode": st.st_ino, "size": st.st_size,
                              "mtime_ns": st.st_mtime_ns}
    assert seal["tokenizer_sha256"] == digest(TOK)
    assert sorted(p.name for p in exported.parent.iterdir()) == ["model.pt", "snapshot.json"]   # no staging file left
    again = store.export(source)                                                           # every export is its own folder
    assert again != exported and again.parent.parent == exported.parent.parent


def test_loaded_model_is_strict_fp32_eval_and_steps_like_its_forward(run):
    tmp, source, state = run
    store = S.SnapshotStore(tmp / "snaps", TOK)
    model, processor, metadata = store.load(store.export(source))
    assert "model" not in metadata and metadata["step"] == 7
    assert not model.training and not any(p.requires_grad for p in model.parameters())
    assert {p.device.type for p in model.parameters()} == {"cpu"} and {b.device.type for b in model.buffers()} <= {"cpu"}
    assert processor.vocab_size() == model.cfg.vocab_size
    tokens = torch.tensor([[3, 4, 5, 6, 7, 8, 9, 10]])                                     # two 4-token chunks
    caches = model.init_generation_cache(1, torch.device("cpu"), torch.float32)
    stepped = torch.cat([model.step(tokens[:, i:i + 1], caches) for i in range(tokens.shape[1])], dim=1)
    torch.testing.assert_close(stepped, model(tokens), rtol=2e-5, atol=2e-6)


def test_export_keeps_the_version_it_opened_when_the_trainer_publishes_a_new_one(run, monkeypatch):
    tmp, source, state = run
    newer = tmp / "run" / "next.pt"
    torch.save(training_checkpoint(step=8, tokens=128, seed=1), newer)
    real_load = S.PinnedFile.load

    def load_then_replace(self):
        os.replace(newer, source)               # the trainer renames a new checkpoint over the path meanwhile
        return real_load(self)

    monkeypatch.setattr(S.PinnedFile, "load", load_then_replace)
    exported = S.SnapshotStore(tmp / "snaps", TOK).export(source)
    payload = torch.load(exported, map_location="cpu", weights_only=False)
    assert payload["step"] == 7                                                            # the pinned version, complete
    for key, value in state["model"].items():
        assert torch.equal(payload["model"][key], value)
    assert torch.load(source, map_location="cpu", weights_only=False)["step"] == 8


def test_a_source_rewritten_in_place_publishes_nothing(run, monkeypatch):
    tmp, source, _ = run
    real_load = S.PinnedFile.load

    def load_then_append(self):
        loaded = real_load(self)
        with open(source, "ab") as stream:      # same inode, new size: not a rename-published file
            stream.write(b"tail")
        return loaded

    monkeypatch.setattr(S.PinnedFile, "load", load_then_append)
    with pytest.raises(RuntimeError, match="changed while it was being exported"):
        S.SnapshotStore(tmp / "snaps", TOK).export(source)
    assert not list((tmp / "snaps").rglob("model.pt")) and not list((tmp / "snaps").rglob("snapshot.json"))


def test_resolve_uses_a_sealed_export_as_it_is(run, monkeypatch):
    tmp, source, _ = run
    store = S.SnapshotStore(tmp / "snaps", TOK)
    exported = store.export(source)
    elsewhere = S.SnapshotStore(tmp / "unused", TOK)
    monkeypatch.setattr(S.SnapshotStore, "export", lambda self, path: pytest.fail("a sealed export must not be exported again"))
    assert elsewhere.resolve(exported) == exported
    assert not (tmp / "unused").exists()
    with pytest.raises(ValueError, match="no such checkpoint file"):
        elsewhere.resolve(tmp / "missing.pt")


def test_an_export_without_its_seal_is_neither_loaded_nor_resealed(run):
    tmp, source, _ = run
    store = S.SnapshotStore(tmp / "snaps", TOK)
    exported = store.export(source)
    exported.with_name("snapshot.json").unlink()
    with pytest.raises(ValueError, match="snapshot.json is missing"):
        store.load(exported)
    with pytest.raises(ValueError, match="already an inference export"):
        S.SnapshotStore(tmp / "unused", TOK).resolve(exported)
    assert not (tmp / "unused").exists()


@pytest.mark.parametrize("seal", ["[]", "{}", '{"snapshot_sha256": 5}', '{"snapshot_sha256": "0000"}'])
def test_a_seal_that_does_not_vouch_for_the_file_is_refused(run, seal):
    tmp, source, _ = run
    store = S.SnapshotStore(tmp / "snaps", TOK)
    exported = store.export(source)
    exported.with_name("snapshot.json").chmod(0o644)
    exported.with_name("snapshot.json").write_text(seal)
    with pytest.raises(ValueError, match="not a snapshot seal|does not match its seal"):
        store.load(exported)
    assert store.resolve(exported) == exported          # resolving does not replace it either


def test_malformed_seal_text_is_an_error_not_a_bypass(run):
    tmp, source, _ = run
    store = S.SnapshotStore(tmp / "snaps", TOK)
    exported = store.export(source)
    exported.with_name("snapshot.json").chmod(0o644)
    exported.with_name("snapshot.json").write_text("{")
    with pytest.raises(ValueError):
        store.load(exported)


def test_wrong_tokenizer_is_refused_at_export_and_at_load(run, tmp_path):
    tmp, source, state = run
    other = tmp_path / "other.model"
    other.write_bytes(TOK.read_bytes() + b"\0")
    with pytest.raises(ValueError, match="tokenizer file is not the one"):
        S.SnapshotStore(tmp / "snaps", other).export(source)
    exported = S.SnapshotStore(tmp / "snaps", TOK).export(source)
    with pytest.raises(ValueError, match="tokenizer SHA256"):
        S.SnapshotStore(tmp / "snaps", other).load(exported)


@pytest.mark.parametrize("damage", ["missing", "extra", "dtype"])
def test_state_dict_must_fit_exactly(run, damage):
    tmp, source, state = run
    model = dict(state["model"])
    if damage == "missing":
        model.pop("final_norm.weight")
    elif damage == "extra":
        model["module.embed.weight"] = model["embed.weight"].clone()
    else:
        model["final_norm.weight"] = model["final_norm.weight"].to(torch.bfloat16)
    torch.save(dict(state, model=model), source)
    store = S.SnapshotStore(tmp / "snaps", TOK)
    exported = store.export(source)
    with pytest.raises((RuntimeError, ValueError), match="final_norm|module.embed|FP32"):
        store.load(exported)


@pytest.mark.parametrize("name", ["latest.pt.tmp", "latest.bin"])
def test_only_finished_regular_checkpoints_are_opened(run, name):
    tmp, source, _ = run
    odd = source.with_name(name)
    odd.write_bytes(source.read_bytes())
    with pytest.raises(ValueError, match="regular .pt checkpoint"):
        S.SnapshotStore(tmp / "snaps", TOK).export(odd)
    link = source.with_name("link.pt")
    link.symlink_to(source)
    with pytest.raises(ValueError, match="regular .pt checkpoint"):
        S.SnapshotStore(tmp / "snaps", TOK).export(link)
    assert not (tmp / "snaps").exists()


def test_other_formats_are_not_training_checkpoints(run):
    tmp, source, state = run
    torch.save(dict(state, format="warpstate-posttrain-v1"), source)
    with pytest.raises(ValueError, match="expected a warpstate-server-v1"):
        S.SnapshotStore(tmp / "snaps", TOK).export(source)
