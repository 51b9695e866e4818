"""The pretraining command line on CPU: continuous vs split-and-resumed runs are bitwise equal,
flag cross-validation, resume signatures, corpus preparation interrupt/resume.

The fixture is the reference's 73-token corpus (updates of 32, 32 and 9 tokens, so the final
update has fewer tokens than one micro-batch; test_server.py:79-125,
test_training_execution.py:385-543).
"""
import json
import os
import sys
import types
from pathlib import Path

import numpy as np
import pytest
import torch

from warpstate_ai_b200.data import prepare as P
from warpstate_ai_b200.data.tokens import batches, update_slices
from warpstate_ai_b200.train import pretrain as T
from warpstate_ai_b200.train.signature import check_resume_signature

ROOT = Path(__file__).resolve().parents[1]
TOKENIZER = ROOT / "tokenizer.model"


def tiny_config(path: Path):
    cfg = dict(vocab_size=32768, d_model=16, n_heads=2, n_cores=2, logical_depth=2, ffn_hidden=24, chunk_size=4,
               dropout=0.0, rms_eps=1e-5, gradient_checkpointing=False, parallel_memory=True, loss_chunk_size=16)
    path.write_text(json.dumps(cfg))
    return path


def base_args(work: Path, config: Path, extra=()):
    return ["--from-scratch", "--work-dir", str(work), "--config", str(config), "--tokenizer", str(TOKENIZER),
            "--stage", "train", "--device", "cpu", "--test-small-gpu", "--train-tokens", "73", "--val-tokens", "64",
            "--seq-len", "8", "--micro-batch", "2", "--grad-accum", "2", "--warmup-steps", "2", "--lr", "1e-3",
            "--min-lr", "1e-4", "--eval-every", "1", "--eval-batches", "2", "--save-every", "1",
            "--no-activation-checkpointing", "--dataset", "synthetic/uniform", "--dataset-config", "none",
            "--revision", "0", *extra]


def make_work(tmp_path: Path, name: str):
    work = tmp_path / name
    P.write_synthetic_corpus(work, TOKENIZER, 73, 64, 32768, seed=5)
    return work


def load(work: Path):
    return torch.load(work / "run/latest.pt", weights_only=False)


def assert_same_checkpoint(a, b):
    assert a["step"] == b["step"] and a["tokens_seen"] == b["tokens_seen"]
    assert list(a["model"].keys()) == list(b["model"].keys())
    assert not any(k.startswith(("module.", "_orig_mod.")) for k in a["model"])
    for k in a["model"]:
        assert torch.equal(a["model"][k], b["model"][k]), k
    for i in a["optimizer"]["state"]:
        for f in ("step", "exp_avg", "exp_avg_sq"):
            assert torch.equal(a["optimizer"]["state"][i][f], b["optimizer"]["state"][i][f]), (i, f)
    assert torch.equal(a["rng_torch"], b["rng_torch"])
    assert a["rng_python"] == b["rng_python"]


@pytest.mark.parametrize("async_ckpt", [False, True])
def test_continuous_and_resumed_runs_are_bitwise_equal(tmp_path, monkeypatch, async_ckpt):
    monkeypatch.setattr(T, "STOP", False)
    config = tiny_config(tmp_path / "cfg.json")
    extra = ["--async-checkpoint"] if async_ckpt else []
    cont = make_work(tmp_path, "cont")
    T.main(base_args(cont, config, extra))
    full = load(cont)
    assert full["step"] == 3 and full["tokens_seen"] == 73 and full["format"] == "warpstate-server-v1"
    split = make_work(tmp_path, "split")
    T.main(base_args(split, config, extra + ["--max-steps", "1"]))
    assert load(split)["step"] == 1
    T.main(base_args(split, config, extra + ["--stop-at-step", "2"]))
    assert load(split)["step"] == 2
    T.main(base_args(split, config, extra))
    assert_same_checkpoint(full, load(split))
    metrics = [json.loads(line) for line in (cont / "run/metrics.jsonl").read_text().splitlines()]
    assert [m["step"] for m in metrics] == [1, 2, 3] and metrics[-1]["tokens"] == 73
    assert {"loss", "lr", "grad_norm", "tokens_per_second", "val_loss", "gpu_memory"} <= set(metrics[0])
    assert (cont / "run/settings.json").exists() and (cont / "run/validation.jsonl").exists()


def test_resume_rejects_changed_objective_and_accepts_reconfigure(tmp_path, monkeypatch):
    monkeypatch.setattr(T, "STOP", False)
    config = tiny_config(tmp_path / "cfg.json")
    work = make_work(tmp_path, "w")
    T.main(base_args(work, config, ["--max-steps", "1"]))
    with pytest.raises(ValueError, match="Resume settings/data differ"):
        T.main(base_args(work, config, ["--lr", "2e-3"]))
    args = base_args(work, config)
    i = args.index("--micro-batch")
    args[i + 1] = "1"
    args[args.index("--grad-accum") + 1] = "4"
    with pytest.raises(ValueError, match="Resume settings/data differ"):
        T.main(args)
    T.main(args + ["--reconfigure"])
    ckpt = load(work)
    assert ckpt["step"] == 3 and len(ckpt["execution_history"]) == 1
    assert ckpt["execution_history"][0]["from"]["micro_batch"] == 2


def test_signature_rules():
    base = {"settings": {"seq_len": 8, "micro_batch": 2, "grad_accum": 2, "train_tokens": 73, "lr": 1e-3, "min_lr": 1e-4,
                         "warmup_steps": 2, "weight_decay": 0.1, "seed": 1, "activation_checkpointing": False,
                         "loss_chunk_size": 16, "compile": False, "world_size": 1}, "data": {"x": 1}}
    same = json.loads(json.dumps(base))
    assert check_resume_signature(base, same) is False
    two = json.loads(json.dumps(base))
    two["settings"].update(world_size=2, grad_accum=1, loss_mode="compiled-full")
    with pytest.raises(ValueError):
        check_resume_signature(base, two)
    assert check_resume_signature(base, two, reconfigure=True) is True
    bad = json.loads(json.dumps(two))
    bad["settings"]["grad_accum"] = 2  # global tokens per update would double
    with pytest.raises(ValueError, match="global tokens per update"):
        check_resume_signature(base, bad, reconfigure=True)
    other_data = json.loads(json.dumps(base))
    other_data["data"] = {"x": 2}
    with pytest.raises(ValueError):
        check_resume_signature(base, other_data, reconfigure=True)


@pytest.mark.parametrize("flags", [
    ["--min-lr", "1"], ["--micro-batch", "0"], ["--ddp-bucket-cap-mb", "-1"], ["--val-tokens", "100"],
    ["--shard-params", "stream", "--shard-optimizer"], ["--bootstrap", "--no-bootstrap"], ["--vram-limit-gib", "0"],
    ["--stage", "sometimes"],
])
def test_invalid_settings_are_rejected(flags):
    with pytest.raises(SystemExit):
        T.arguments(["--from-scratch", *flags])


def test_reference_execution_flags_are_accepted_recorded_and_reported(capsys):
    """The reference's execution experiments have no counterpart to switch here: any combination parses, the
    values reach the resume signature, and rank 0 says once per flag that it changes nothing and why."""
    from warpstate_ai_b200.train.signature import train_signature
    a = T.arguments(["--from-scratch", "--compile", "--compile-core", "--compile-mode", "reduce-overhead",
                     "--gradient-mode", "compiled-autograd", "--ddp-batched-grad-copy", "--backward-layout", "paired",
                     "--cache-core-weight-casts", "--activation-mode", "swiglu", "--overlap-swap-collectives"])
    out = capsys.readouterr().out
    for flag in ("--compile-mode reduce-overhead", "--backward-layout paired", "--gradient-mode compiled-autograd"):
        assert f"note: {flag} has no effect here" in out
    settings = train_signature(a, {"x": 1})["settings"]
    assert settings["gradient_mode"] == "compiled-autograd" and settings["compile_mode"] == "reduce-overhead"
    assert settings["cache_core_weight_casts"] is True and settings["ddp_batched_grad_copy"] is True
    quiet = T.arguments(["--from-scratch"])
    assert "no effect" not in capsys.readouterr().out and quiet.ddp_bucket_cap_mb == 0.0


def test_bucket_cap_merges_small_cores_and_splits_large_buckets():
    import torch
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.optim.arena import ParamArena
    from warpstate_ai_b200.parallel.grad_sync import CollectiveGradSync
    cfg = WarpStateConfig(vocab_size=64, d_model=32, n_heads=2, n_cores=4, logical_depth=4, ffn_hidden=48, chunk_size=8,
                          gradient_checkpointing=False)
    per_core = ParamArena(WarpStateLM(cfg), device=torch.device("cpu"))
    assert len(per_core.buckets) == 5                                      # tail + one per core
    core_bytes = 4 * (per_core.buckets[1].stop - per_core.buckets[1].start)
    merged = ParamArena(WarpStateLM(cfg), device=torch.device("cpu"), bucket_cap_bytes=2 * core_bytes)
    assert len(merged.buckets) == 3                                        # tail + two pairs of cores
    sync = CollectiveGradSync(torch.device("cpu"), 2, 0, bucket_cap_bytes=4 * 1024)
    sync.attach(merged, WarpStateLM(cfg))
    assert sync.core_bucket == {0: 1, 2: 2}                                # the lowest core of a bucket completes it
    for b in merged.buckets:
        pieces = sync.pieces_of(b.index)
        assert pieces[0][0] == b.start and sum(c for _, c in pieces) == b.stop - b.start
        assert all(c <= 1024 and c % 4 == 0 for _, c in pieces)
        assert all(pieces[i][0] + pieces[i][1] == pieces[i + 1][0] for i in range(len(pieces) - 1))


def test_bootstrap_builds_an_environment_and_re_executes(monkeypatch, tmp_path):
    """--bootstrap with pip, venv and exec replaced by recorders: the sequence of commands, and the command line
    that is re-executed inside the environment."""
    import subprocess
    calls = []
    monkeypatch.setattr(T, "ROOT", tmp_path)
    (tmp_path / "launch").mkdir()
    (tmp_path / "launch/requirements-training.txt").write_text("torch\n")

    def fake_run(cmd, check=True):
        calls.append(cmd)
        if cmd[1:3] == ["-m", "venv"]:
            (tmp_path / ".server-venv/bin").mkdir(parents=True)
            (tmp_path / ".server-venv/bin/python").write_text("")

    monkeypatch.setattr(subprocess, "run", fake_run)
    monkeypatch.setattr(subprocess, "check_output", lambda cmd, text=True: "torch==0\n")
    executed = {}
    monkeypatch.setattr(T.os, "execv", lambda path, argv: executed.update(path=path, argv=argv))
    monkeypatch.setattr(sys, "argv", ["run_40b.py", "--from-scratch", "--bootstrap", "--seq-len", "256"])
    a = T.arguments(["--from-scratch", "--bootstrap", "--seq-len", "256"])
    T.bootstrap(a)
    assert [c[1:4] for c in calls][:2] == [["-m", "venv", str(tmp_path / ".server-venv")], ["-m", "pip", "install"]]
    assert (tmp_path / ".server-venv/warpstate-deps-v1.json").exists()
    assert executed["argv"][-1] == "--no-bootstrap" and "--bootstrap" not in executed["argv"]
    assert executed["argv"][3:6] == ["--from-scratch", "--seq-len", "256"]
    calls.clear()
    T.bootstrap(T.arguments(["--from-scratch"]))      # off by default: nothing happens
    assert calls == []


def test_accepted_flag_combinations():
    a = T.arguments(["--from-scratch", "--compile-core", "--compile-mode", "max-autotune-no-cudagraphs",
                     "--loss-mode", "compiled-full", "--no-activation-checkpointing", "--async-checkpoint"])
    assert a.async_checkpoint and a.loss_mode == "compiled-full" and a.kernels == "sm100a"
    a = T.arguments(["--from-scratch", "--no-async-checkpoint", "--device", "cpu"])
    assert not a.async_checkpoint and a.kernels == "pytorch"


@pytest.mark.parametrize("world", [1, 2, 3])
def test_update_slices_partition_the_update(world):
    for target in (1, 31, 32, 73, 200):
        covered = []
        for rank in range(world):
            for offset, valid in update_slices(target, 16, world, rank):
                covered.extend(range(offset, offset + valid))
        assert sorted(covered) == list(range(target))
        counts = {len(list(update_slices(target, 16, world, r))) for r in range(world)}
        assert len(counts) == 1  # every rank runs the same number of iterations, even when empty


def test_batches_wrap_and_mask():
    data = np.arange(10, dtype=np.uint16)
    x, y = batches(data, 7, 2, 3, 4, torch.device("cpu"))
    assert x.tolist() == [[7, 8, 9], [0, 1, 2]]
    assert y.tolist() == [[8, 9, 0], [1, -100, -100]]


def test_prepare_interrupt_and_resume_is_byte_identical(tmp_path, monkeypatch):
    docs = [{"text": f"document number {i} " + "lorem ipsum " * (i % 7 + 1)} for i in range(400)]

    class FakeStream:
        def __init__(self):
            self.position = 0

        def __iter__(self):
            while self.position < len(docs):
                self.position += 1
                yield docs[self.position - 1]

        def state_dict(self):
            return {"position": self.position}

        def load_state_dict(self, state):
            self.position = state["position"]

    fake_datasets = types.SimpleNamespace(__version__="fake-1", load_dataset=lambda *a, **k: FakeStream())
    fake_hub = types.SimpleNamespace(HfApi=lambda: types.SimpleNamespace(
        dataset_info=lambda name, revision: types.SimpleNamespace(sha="deadbeef")))
    monkeypatch.setitem(sys.modules, "datasets", fake_datasets)
    monkeypatch.setitem(sys.modules, "huggingface_hub", fake_hub)
    monkeypatch.setattr(P, "COMMIT_TOKENS", 200)

    def args(work):
        return types.SimpleNamespace(work_dir=work, tokenizer=TOKENIZER, dataset="d", dataset_config="c", revision="main",
                                     train_tokens=1500, val_tokens=0, workers=1, documents_per_batch=7,
                                     test_small_gpu=True, verify_data=True)

    holdout = sum(P.is_holdout(d["text"]) for d in docs)
    one = args(tmp_path / "one")
    one.val_tokens = 5 if holdout else 0
    if one.val_tokens == 0:
        one.val_tokens = 0
    # uninterrupted
    a = args(tmp_path / "a")
    a.val_tokens = 0
    b = args(tmp_path / "b")
    b.val_tokens = 0
    for ns in (a, b):
        ns.val_tokens = 0
    assert P.prepare(a) is True
    calls = {"n": 0}

    def stop_after_three():
        calls["n"] += 1
        return calls["n"] == 3

    assert P.prepare(b, stop_requested=stop_after_three) is False
    partial = (b.work_dir / "data/train.bin").stat().st_size
    assert 0 < partial < 3000
    with (b.work_dir / "data/train.bin").open("ab") as f:
        f.write(b"\xff" * 10)  # uncommitted garbage after an interruption
    assert P.prepare(b) is True
    assert (a.work_dir / "data/train.bin").read_bytes() == (b.work_dir / "data/train.bin").read_bytes()
    assert P.check_manifest(b)["complete"] is True
    with pytest.raises(ValueError):
        b.train_tokens = 1499
        P.check_manifest(b)
