"""Model configuration, checkpoint-format helpers and the host-side file utilities.

Contracts: the configuration's fields and JSON form (reference warpstate/config.py:12-46), the production model's size
(2,005,111,424 parameters in 256 tensors), canonical state-dict keys (reference test_training_execution.py:417-418),
the ``warpstate-server-v1`` key set (reference run_40b.py:680-686), atomic publication and the pipeline lock
(reference run_40b.py:211-224).
"""
import json
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from warpstate_ai_b200.ckpt import formats as F
from warpstate_ai_b200.config import WarpStateConfig, warpstate_2b, warpstate_smoke
from warpstate_ai_b200.models.warpstate import WarpStateLM
from warpstate_ai_b200.utils import io as IO

ROOT = Path(__file__).resolve().parents[1]
TOK = ROOT / "tokenizer.model"


# ------------------------------------------------------------------------------------------- configuration
def test_production_configuration_has_the_documented_size():
    cfg = warpstate_2b()
    cfg.validate()
    with torch.device("meta"):
        model = WarpStateLM(cfg)
    assert model.num_parameters() == 2_005_111_424
    keys = list(model.state_dict())
    assert len(keys) == 256 == 9 * 28 + 4
    assert {k for k in keys if not k.startswith("cores.")} == {"depth_scale", "depth_bias", "embed.weight", "final_norm.weight"}
    assert {k.split(".", 2)[2] for k in keys if k.startswith("cores.0.")} == {
        "fast_decay_logit", "slow_decay_logit", "memory_mix_logit", "norm1.weight", "in_proj.weight", "out_proj.weight",
        "norm2.weight", "ffn.up_gate.weight", "ffn.down.weight"}
    shapes = {k: tuple(v.shape) for k, v in model.state_dict().items()}
    assert shapes["cores.3.in_proj.weight"] == (5 * 2048, 2048) and shapes["cores.3.ffn.up_gate.weight"] == (2 * 7168, 2048)
    assert shapes["depth_scale"] == (28, 2048) and shapes["cores.0.fast_decay_logit"] == (32,)
    assert cfg.head_dim == 64


def test_configuration_round_trips_through_json_and_rejects_nonsense(tmp_path):
    cfg = warpstate_smoke()
    path = tmp_path / "cfg.json"
    cfg.to_json(path)
    assert WarpStateConfig.from_json(path) == cfg and json.loads(path.read_text()) == cfg.to_dict()
    assert WarpStateConfig(**vars(cfg)) == cfg                                    # checkpoints store vars(cfg)
    assert (WarpStateConfig().d_model, WarpStateConfig().n_cores, WarpStateConfig().logical_depth) == (1280, 4, 16)
    with pytest.raises(TypeError, match=r"unknown WarpStateConfig fields: \['n_layers'\]"):
        WarpStateConfig.from_dict({"n_layers": 3})
    for bad, message in ((dict(d_model=100, n_heads=3), "divisible by n_heads"), (dict(n_cores=4, logical_depth=2), "at least n_cores"),
                         (dict(chunk_size=0), "must be positive"), (dict(d_model=30, n_heads=2), "head_dim must be even")):
        with pytest.raises(AssertionError, match=message):
            WarpStateConfig.from_dict(bad)


# ------------------------------------------------------------------------------------------- checkpoint helpers
class Wrapper(torch.nn.Module):
    def __init__(self, inner, name):
        super().__init__()
        setattr(self, name, inner)


def test_state_dict_keys_lose_every_wrapper_prefix():
    cfg = WarpStateConfig(vocab_size=64, d_model=16, n_heads=2, n_cores=1, logical_depth=1, ffn_hidden=24, chunk_size=4)
    model = WarpStateLM(cfg)
    plain = F.clean_state_dict(model)
    assert list(plain) == list(model.state_dict())
    wrapped = Wrapper(Wrapper(model, "_orig_mod"), "module")
    assert list(wrapped.state_dict())[0].startswith("module._orig_mod.")
    cleaned = F.clean_state_dict(wrapped)
    assert list(cleaned) == list(plain) and all(cleaned[k] is plain[k] or torch.equal(cleaned[k], plain[k]) for k in plain)
    model.cores[0] = Wrapper(model.cores[0], "_orig_mod")                         # a compiled core inside the model
    assert list(F.clean_state_dict(model)) == list(plain)


def test_rng_capture_and_restore_cover_all_three_generators():
    F.seed_everything(123)
    state = F.capture_rng()
    first = (torch.rand(3), np.random.rand(3), random.random())
    F.restore_rng(state)
    second = (torch.rand(3), np.random.rand(3), random.random())
    assert torch.equal(first[0], second[0]) and np.array_equal(first[1], second[1]) and first[2] == second[2]
    assert state["cuda"].numel() == 0                                             # no device: an empty placeholder
    F.seed_everything(123)
    assert torch.equal(torch.rand(3), first[0])
    F.seed_everything(124)
    assert not torch.equal(torch.rand(3), first[0])


def test_server_checkpoint_has_the_reference_key_set_and_loads_strictly(tmp_path):
    cfg = WarpStateConfig(vocab_size=64, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=4)
    model = WarpStateLM(cfg)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-3)
    rng = F.capture_rng()
    state = F.server_state(signature={"s": 1}, origin={"o": 2}, history=[{"h": 3}], cfg=cfg, model=model, optimizer=optimizer,
                           step=5, tokens_seen=640, val_loss=None, val_step=None, val_tokens=None, rng_by_rank=[rng, rng])
    assert set(state) == {"format", "signature", "origin", "execution_history", "config", "model", "optimizer", "step",
                          "tokens_seen", "val_loss", "val_step", "val_tokens", "rng_by_rank", "rng_torch", "rng_cuda",
                          "rng_numpy", "rng_python"}
    assert state["format"] == "warpstate-server-v1" and state["config"] == vars(cfg) and state["config"] is not vars(cfg)
    assert state["rng_torch"] is rng["torch"] and len(state["rng_by_rank"]) == 2 and len(state["rng_cuda"]) == 1
    given = {"only": torch.zeros(1)}
    assert F.server_state(signature={}, origin={}, history=[], cfg=cfg, model=model, optimizer=optimizer, step=0, tokens_seen=0,
                          val_loss=None, val_step=None, val_tokens=None, rng_by_rank=[rng], model_state=given)["model"] is given
    path = tmp_path / "latest.pt"
    torch.save(state, path)
    loaded = F.load_checkpoint(path)
    rebuilt, rebuilt_cfg = F.model_from_checkpoint(loaded, torch.device("cpu"))
    assert rebuilt_cfg == cfg and all(torch.equal(a, b) for a, b in zip(rebuilt.parameters(), model.parameters()))
    loaded["model"].pop("embed.weight")
    with pytest.raises(RuntimeError, match="embed.weight"):
        F.model_from_checkpoint(loaded, torch.device("cpu"))


def test_stage_exports_are_verifiable_and_tamper_evident(tmp_path):
    cfg = WarpStateConfig(vocab_size=64, d_model=16, n_heads=2, n_cores=1, logical_depth=1, ffn_hidden=24, chunk_size=4)
    checkpoint = {"config": vars(cfg).copy(), "model": WarpStateLM(cfg).state_dict(), "step": 9, "tokens_seen": 90, "origin": {"base": 1}}
    meta = F.export_chat_snapshot(checkpoint, tmp_path / "export", TOK, {"path": "x"}, stage="sft")
    assert meta["stage"] == "sft" and meta["format"] == "warpstate-chat-v1" and meta["step"] == 9
    assert F.verify_chat_snapshot(tmp_path / "export", TOK) == meta
    payload = torch.load(tmp_path / "export/model.pt", weights_only=False)
    assert payload["origin"] == {"base": 1} and payload["inference_only"] is True and "optimizer" not in payload
    plain = F.export_chat_snapshot(checkpoint, tmp_path / "plain", TOK, {"path": "x"})
    assert "stage" not in plain and "stage" not in torch.load(tmp_path / "plain/model.pt", weights_only=False)
    other = tmp_path / "other.model"
    other.write_bytes(b"not the tokenizer")
    with pytest.raises(ValueError, match="Tokenizer does not match"):
        F.verify_chat_snapshot(tmp_path / "export", other)
    with open(tmp_path / "export/model.pt", "ab") as stream:
        stream.write(b"!")
    with pytest.raises(ValueError, match="does not match snapshot.json"):
        F.verify_chat_snapshot(tmp_path / "export")


# ------------------------------------------------------------------------------------------- files and locks
def test_atomic_write_publishes_whole_files_or_nothing(tmp_path):
    target = tmp_path / "state.json"
    IO.atomic_json(target, {"a": 1})
    assert json.loads(target.read_text()) == {"a": 1} and [p.name for p in tmp_path.iterdir()] == ["state.json"]

    def fails_half_way(stream):
        stream.write(b'{"a": 2, ')
        raise OSError("disk full")

    with pytest.raises(OSError, match="disk full"):
        IO.atomic_write(target, fails_half_way)
    assert json.loads(target.read_text()) == {"a": 1} and [p.name for p in tmp_path.iterdir()] == ["state.json"]
    with pytest.raises(KeyboardInterrupt):                                       # an interrupt cleans up too
        IO.atomic_write(target, lambda stream: (_ for _ in ()).throw(KeyboardInterrupt()))
    assert [p.name for p in tmp_path.iterdir()] == ["state.json"]
    IO.atomic_json(target, {"a": 3}, indent=None)
    assert target.read_text() == '{"a": 3}'


def test_digests_and_json_lines(tmp_path):
    blob = tmp_path / "blob"
    blob.write_bytes(b"abc" * 1000)
    assert IO.digest(blob) == IO.digest(blob, block=7) == IO.digest_bytes(b"abc" * 1000)
    assert IO.digest_bytes(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    log = tmp_path / "events.jsonl"
    IO.append_jsonl(log, {"step": 1})
    IO.append_jsonl(log, {"step": 2, "loss": 0.5})
    assert [json.loads(line) for line in log.read_text().splitlines()] == [{"step": 1}, {"step": 2, "loss": 0.5}]
    stamp = IO.utc_timestamp()
    assert len(stamp) == 20 and stamp[10] == "T" and stamp.endswith("Z")


TRY_LOCK = """
import sys
from warpstate_ai_b200.utils import io as IO
try:
    with IO.process_lock(sys.argv[1], shared=sys.argv[2] == "shared"):
        print("acquired")
except IO.LockHeld as error:
    print(f"held: {error}")
"""


def attempt(path, shared):
    """Another process tries to take the lock, without waiting, and says how it went."""
    run = subprocess.run([sys.executable, "-c", TRY_LOCK, str(path), "shared" if shared else "exclusive"], cwd=ROOT,
                         capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stderr
    return run.stdout.strip()


def test_pipeline_lock_is_exclusive_for_pretraining_and_shared_among_post_training_ranks(tmp_path):
    path = tmp_path / "control" / "pipeline.lock"
    with IO.process_lock(path):                                                   # the pretraining job
        assert attempt(path, shared=True).startswith("held:") and attempt(path, shared=False).startswith("held:")
    assert attempt(path, shared=False) == "acquired"                             # released with the context
    with IO.process_lock(path, shared=True):                                      # a post-training rank
        assert attempt(path, shared=True) == "acquired"                          # its sibling ranks may join
        assert "is locked by another process" in attempt(path, shared=False)     # the base job may not start


def test_a_child_that_inherited_the_descriptor_keeps_the_lock(tmp_path):
    path = tmp_path / "pipeline.lock"
    with IO.process_lock(path, shared=True) as handle:
        # a worker started with the lock's descriptor, as the launcher passes it on; it lives until its stdin closes
        orphan = subprocess.Popen([sys.executable, "-c", "import sys; sys.stdin.read()"], stdin=subprocess.PIPE,
                                  pass_fds=[handle.fileno()])
    try:
        # the context is over, but the orphaned worker still holds the open file description
        assert attempt(path, shared=False).startswith("held:")
    finally:
        orphan.stdin.close()
        orphan.wait(30)
    assert attempt(path, shared=False) == "acquired"
