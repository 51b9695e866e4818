"""Where a pretraining run starts from and what it demands of the machine (`train/startup.py`;
rules of the reference: run_40b.py:442-456, 459-520, 805-840).  CUDA queries are replaced by fakes: nothing here needs,
or touches, a GPU."""
import json
from argparse import Namespace
from dataclasses import asdict
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

from warpstate_ai_b200.ckpt.formats import SERVER_FORMAT
from warpstate_ai_b200.config import WarpStateConfig
from warpstate_ai_b200.models.warpstate import WarpStateLM
from warpstate_ai_b200.train import startup as S

TOK = Path(__file__).resolve().parents[1] / "tokenizer.model"
GIB = 1 << 30


def tiny(**changes):
    values = dict(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=4,
                  gradient_checkpointing=False, parallel_memory=True)
    values.update(changes)
    return WarpStateConfig(**values)


def arguments(tmp_path, **changes):
    values = dict(work_dir=tmp_path / "work", from_scratch=False, weights=None, config=tmp_path / "cfg.json", tokenizer=TOK,
                  seq_len=8, device="cpu", local_rank=0, test_small_gpu=True, vram_limit_gib=None, vram_headroom_gib=2.0)
    values.update(changes)
    (tmp_path / "work").mkdir(exist_ok=True)
    return Namespace(**values)


def save_checkpoint(path, cfg=None, **extra):
    cfg = cfg or tiny()
    path.parent.mkdir(parents=True, exist_ok=True)
    torch.save({"format": SERVER_FORMAT, "config": asdict(cfg), "model": WarpStateLM(cfg).state_dict(), **extra}, path)
    return path


# ------------------------------------------------------------------------------------------- start points
def test_the_runs_own_checkpoint_wins_over_every_other_way_to_start(tmp_path):
    a = arguments(tmp_path, from_scratch=True, weights=tmp_path / "elsewhere.pt")
    save_checkpoint(a.work_dir / "run/latest.pt", step=3)
    start = S.StartPoint.resolve(a)
    assert (start.kind, start.source) == ("resume", a.work_dir / "run/latest.pt") and start.checkpoint["step"] == 3
    assert start.config(a) == tiny() and start.legacy_masters() is None
    assert "checkpoint=" not in repr(start) and "tensor" not in repr(start)     # a 2 B state dict is not for printing


def test_a_foreign_latest_file_is_not_resumed(tmp_path):
    a = arguments(tmp_path)
    path = save_checkpoint(a.work_dir / "run/latest.pt")
    torch.save(dict(torch.load(path, weights_only=False), format="warpstate-posttrain-v1"), path)
    with pytest.raises(ValueError, match="is not a warpstate-server-v1 checkpoint"):
        S.StartPoint.resolve(a)


def test_first_launch_needs_weights_or_an_explicit_fresh_start(tmp_path):
    with pytest.raises(ValueError, match="needs --weights"):
        S.StartPoint.resolve(arguments(tmp_path))
    with pytest.raises(ValueError, match="needs --weights"):
        S.StartPoint.resolve(arguments(tmp_path, weights=tmp_path / "absent.pt"))
    empty = tmp_path / "empty.pt"
    torch.save({"config": asdict(tiny())}, empty)
    with pytest.raises(ValueError, match="holds no WarpState model state dict"):
        S.StartPoint.resolve(arguments(tmp_path, weights=empty))
    fresh = S.StartPoint.resolve(arguments(tmp_path, from_scratch=True))
    assert (fresh.kind, fresh.source, fresh.checkpoint) == ("scratch", None, {})


def test_initial_weights_bring_their_configuration_or_take_the_given_one(tmp_path):
    cfg = tiny(ffn_hidden=40)
    a = arguments(tmp_path, weights=save_checkpoint(tmp_path / "init.pt", cfg))
    a.config.write_text(json.dumps(asdict(tiny())))                               # ignored: the checkpoint has its own
    start = S.StartPoint.resolve(a)
    assert start.kind == "weights" and start.config(a).ffn_hidden == 40
    bare = tmp_path / "bare.pt"
    torch.save({"model": WarpStateLM(tiny()).state_dict()}, bare)
    start = S.StartPoint.resolve(arguments(tmp_path, weights=bare))
    assert start.config(a) == tiny()                                             # falls back to --config
    a.config.write_text(json.dumps(dict(asdict(tiny()), n_heads=3)))
    with pytest.raises((AssertionError, ValueError), match="divisible by n_heads"):
        start.config(a)                                                          # 16 is not divisible by 3 heads


def test_models_are_built_from_the_checkpoint_or_from_the_seed(tmp_path, capsys):
    cfg = tiny()
    a = arguments(tmp_path, weights=save_checkpoint(tmp_path / "init.pt", cfg))
    start = S.StartPoint.resolve(a)
    model = start.build_model(cfg, seed=0)
    for name, tensor in start.checkpoint["model"].items():
        assert torch.equal(model.state_dict()[name], tensor)
    assert all(p.dtype == torch.float32 and p.device.type == "cpu" for p in model.parameters())
    scratch = S.StartPoint("scratch", None)
    torch.manual_seed(4)
    one = scratch.build_model(cfg, seed=4)
    torch.manual_seed(4)
    two = scratch.build_model(cfg, seed=4)
    assert "fresh FP32 weights from seed 4" in capsys.readouterr().out
    assert all(torch.equal(p, q) for p, q in zip(one.parameters(), two.parameters()))


def test_legacy_offload_masters_are_preferred_only_when_initialising(tmp_path):
    masters = [torch.zeros(2), torch.ones(3)]
    state = {"optimizer": {"kind": "cpu_offload_adamw", "masters": masters}, "model": {}}
    assert S.StartPoint("weights", tmp_path / "w.pt", state).legacy_masters() is masters
    assert S.StartPoint("resume", tmp_path / "w.pt", state).legacy_masters() is None
    assert S.StartPoint("weights", tmp_path / "w.pt", {"optimizer": {"state": {}}, "model": {}}).legacy_masters() is None


# ------------------------------------------------------------------------------------------- fit and preflight
def test_model_must_fit_tokenizer_and_sequence_length(tmp_path):
    a = arguments(tmp_path)
    S.check_fit(tiny(), a)
    with pytest.raises(ValueError, match="1000 vocabulary rows, the tokenizer 32768"):
        S.check_fit(tiny(vocab_size=1000), a)
    with pytest.raises(ValueError, match="--seq-len 10 is not a multiple of the model's chunk size 4"):
        S.check_fit(tiny(), arguments(tmp_path, seq_len=10))


def test_preflight_accepts_the_test_model_and_rejects_what_cannot_train(tmp_path, capsys):
    a = arguments(tmp_path, weights=save_checkpoint(tmp_path / "init.pt"))
    S.preflight(a)
    assert "initial weights" in capsys.readouterr().out
    with pytest.raises(ValueError, match="this package trains the ~2.005 B WarpState architecture"):
        S.preflight(arguments(tmp_path, weights=a.weights, test_small_gpu=False))
    damaged = torch.load(a.weights, weights_only=False)
    damaged["model"].pop("final_norm.weight")
    torch.save(damaged, tmp_path / "damaged.pt")
    with pytest.raises(RuntimeError, match="final_norm.weight"):
        S.preflight(arguments(tmp_path, weights=tmp_path / "damaged.pt"))
    legacy = torch.load(a.weights, weights_only=False)
    legacy["optimizer"] = {"kind": "cpu_offload_adamw", "masters": [torch.zeros(1)]}
    torch.save(legacy, tmp_path / "legacy.pt")
    with pytest.raises(ValueError, match="FP32 masters of the legacy optimizer state"):
        S.preflight(arguments(tmp_path, weights=tmp_path / "legacy.pt"))


def test_full_size_window_brackets_the_production_parameter_count():
    assert 2_005_000_000 in S.FULL_SIZE and 2_000_000_000 in S.FULL_SIZE and 2_020_000_000 in S.FULL_SIZE
    assert 1_999_999_999 not in S.FULL_SIZE and 2_020_000_001 not in S.FULL_SIZE


# ------------------------------------------------------------------------------------------- device rules (faked)
def fake_cuda(monkeypatch, *, available=True, bf16=True, total=180 * GIB, free=170 * GIB, name="B200"):
    calls = []
    monkeypatch.setattr(torch.cuda, "is_available", lambda: available)
    monkeypatch.setattr(torch.cuda, "is_bf16_supported", lambda: bf16)
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda device: SimpleNamespace(name=name, total_memory=total))
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device: (free, total))
    monkeypatch.setattr(torch.cuda, "set_per_process_memory_fraction", lambda fraction, device: calls.append((fraction, device)))
    return calls


def test_cpu_runs_ask_nothing_of_the_machine(tmp_path, monkeypatch):
    fake_cuda(monkeypatch, available=False)
    device, name, total = S.require_device(arguments(tmp_path))
    assert (device, name, total) == (torch.device("cpu"), "cpu", 0)
    S.cap_device_memory(arguments(tmp_path, vram_limit_gib=10.0))                  # a cap means nothing on the CPU


def test_the_training_preset_needs_a_bf16_gpu_of_80_gib(tmp_path, monkeypatch):
    fake_cuda(monkeypatch, available=False)
    with pytest.raises(RuntimeError, match="BF16 support is required"):
        S.require_device(arguments(tmp_path, device="cuda"))
    fake_cuda(monkeypatch, bf16=False)
    with pytest.raises(RuntimeError, match="BF16 support is required"):
        S.require_device(arguments(tmp_path, device="cuda"))
    fake_cuda(monkeypatch, total=48 * GIB, name="L40S")
    with pytest.raises(RuntimeError, match="L40S has 48 GiB; the training preset needs 80 GiB or more"):
        S.require_device(arguments(tmp_path, device="cuda", test_small_gpu=False))
    device, name, total = S.require_device(arguments(tmp_path, device="cuda", test_small_gpu=True, local_rank=3))
    assert (device, name, total) == (torch.device("cuda", 3), "L40S", 48 * GIB)
    fake_cuda(monkeypatch)
    assert S.require_device(arguments(tmp_path, device="cuda", test_small_gpu=False))[2] == 180 * GIB


def test_allocator_cap_is_installed_only_when_cap_plus_headroom_is_free(tmp_path, monkeypatch, capsys):
    calls = fake_cuda(monkeypatch, total=180 * GIB, free=160 * GIB)
    S.cap_device_memory(arguments(tmp_path, device="cuda"))                        # no limit asked: nothing happens
    assert calls == []
    S.cap_device_memory(arguments(tmp_path, device="cuda", vram_limit_gib=150.0, vram_headroom_gib=8.0, local_rank=1))
    assert calls == [(150 / 180, torch.device("cuda", 1))]
    assert "capped at 150.00 GiB (160.00 GiB were free)" in capsys.readouterr().out
    with pytest.raises(RuntimeError, match="needs 162.00 GiB but the device has 160.00 GiB free of 180.00"):
        S.cap_device_memory(arguments(tmp_path, device="cuda", vram_limit_gib=150.0, vram_headroom_gib=12.0))
    with pytest.raises(RuntimeError, match="needs 200.00 GiB"):
        S.cap_device_memory(arguments(tmp_path, device="cuda", vram_limit_gib=200.0, vram_headroom_gib=0.0))
    assert len(calls) == 1                                                         # a refused cap installs nothing
