"""Checkpoint / resume through the GPU path of the pretraining CLI (fused kernels, gradient arena, in-kernel
gradient synchronisation), as child processes of ``run_40b.py``:

* a run split into three launches (pause after one update, pause at step two, finish) ends bit-identical to
  the uninterrupted run -- model, AdamW moments and step counts, RNG streams -- with the synchronous and with
  the asynchronous checkpoint writer, on one GPU and on two (where the last update leaves the second rank
  short of data);
* a run started on one GPU and continued on two with ``--reconfigure`` (same global tokens per update) stays
  within the reference's tolerances of its reconfiguration test (reference test_training_execution.py:546-570:
  model rtol 0.01 / atol 2e-5, moments rtol 0.03 / atol 2e-7);
* the same split with fully sharded parameters resumes from the unsharded checkpoint it wrote.

The CPU counterpart (plain PyTorch path) is tests/test_pretrain_cli.py.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from warpstate_ai_b200.data import prepare as P

ROOT = Path(__file__).resolve().parents[1]
TOKENIZER = ROOT / "tokenizer.model"
pytestmark = pytest.mark.gpu
needs_two_gpus = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                    reason="needs two CUDA devices")
TRAIN_TOKENS, VAL_TOKENS, SEQ = 1300, 600, 256


def write_config(path: Path) -> Path:
    # the smallest geometry the kernels take: head_dim 64, chunk 128
    path.write_text(json.dumps(dict(vocab_size=32768, d_model=128, n_heads=2, n_cores=2, logical_depth=2, ffn_hidden=256,
                                    chunk_size=128, dropout=0.0, rms_eps=1e-5, gradient_checkpointing=False,
                                    parallel_memory=True, loss_chunk_size=128)))
    return path


def launch(work: Path, config: Path, gpus: int, extra=(), grad_accum: int = 2, port: int = 29621):
    arguments = ["--from-scratch", "--work-dir", str(work), "--config", str(config), "--tokenizer", str(TOKENIZER),
                 "--stage", "train", "--device", "cuda", "--test-small-gpu", "--train-tokens", str(TRAIN_TOKENS),
                 "--val-tokens", str(VAL_TOKENS), "--seq-len", str(SEQ), "--micro-batch", "1", "--grad-accum",
                 str(grad_accum), "--warmup-steps", "2", "--lr", "1e-3", "--min-lr", "1e-4", "--eval-every", "1",
                 "--eval-batches", "2", "--save-every", "1", "--no-activation-checkpointing", "--dataset",
                 "synthetic/uniform", "--dataset-config", "none", "--revision", "0", *extra]
    command = [sys.executable]
    if gpus > 1:
        command += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
                    "--master-port", str(port)]
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    done = subprocess.run(command + [str(ROOT / "run_40b.py"), *arguments], env=env, capture_output=True, text=True,
                          timeout=600)
    assert done.returncode == 0, (done.stdout[-2000:], done.stderr[-3000:])


def work_dir(tmp_path: Path, name: str) -> Path:
    work = tmp_path / name
    P.write_synthetic_corpus(work, TOKENIZER, TRAIN_TOKENS, VAL_TOKENS, 32768, seed=5)
    return work


def load(work: Path):
    return torch.load(work / "run/latest.pt", weights_only=False)


def assert_bitwise(a, b):
    assert (a["step"], a["tokens_seen"]) == (b["step"], b["tokens_seen"])
    assert list(a["model"]) == list(b["model"])
    for name in a["model"]:
        assert torch.equal(a["model"][name], b["model"][name]), name
    assert a["optimizer"]["state"].keys() == b["optimizer"]["state"].keys()
    for index, entry in a["optimizer"]["state"].items():
        for key in ("step", "exp_avg", "exp_avg_sq"):
            assert torch.equal(entry[key], b["optimizer"]["state"][index][key]), (index, key)
    for mine, theirs in zip(a["rng_by_rank"], b["rng_by_rank"]):
        assert torch.equal(mine["torch"], theirs["torch"]) and torch.equal(mine["cuda"], theirs["cuda"])
        assert mine["python"] == theirs["python"]


def split_then_finish(tmp_path, config, gpus, extra, name, grad_accum=2):
    work = work_dir(tmp_path, name)
    launch(work, config, gpus, [*extra, "--max-steps", "1"], grad_accum)
    assert load(work)["step"] == 1
    launch(work, config, gpus, [*extra, "--stop-at-step", "2"], grad_accum)
    launch(work, config, gpus, extra, grad_accum)
    return load(work)


@pytest.mark.parametrize("writer", ["sync", "async"])
def test_one_gpu_split_run_is_bitwise_equal_to_continuous(tmp_path, writer):
    config = write_config(tmp_path / "cfg.json")
    extra = ["--async-checkpoint"] if writer == "async" else []
    whole = work_dir(tmp_path, "whole")
    launch(whole, config, 1, extra)
    full = load(whole)
    assert full["step"] == 3 and full["tokens_seen"] == TRAIN_TOKENS
    assert json.loads((whole / "run/settings.json").read_text())["runtime"]["kernels"] == "sm100a"
    assert_bitwise(full, split_then_finish(tmp_path, config, 1, extra, "split"))


def test_one_gpu_sharded_layout_resumes_from_its_unsharded_checkpoint(tmp_path):
    config = write_config(tmp_path / "cfg.json")
    extra = ["--shard-params", "stream"]
    whole = work_dir(tmp_path, "whole")
    launch(whole, config, 1, extra)
    full = load(whole)
    assert full["model"]["cores.0.in_proj.weight"].shape == (640, 128)       # unsharded, reference keys
    assert_bitwise(full, split_then_finish(tmp_path, config, 1, extra, "split"))


@pytest.mark.multigpu
@needs_two_gpus
@pytest.mark.parametrize("writer", ["sync", "async"])
def test_two_gpu_split_run_is_bitwise_equal_to_continuous(tmp_path, writer):
    config = write_config(tmp_path / "cfg.json")
    extra = ["--async-checkpoint"] if writer == "async" else []
    whole = work_dir(tmp_path, "whole")
    launch(whole, config, 2, extra)
    full = load(whole)
    # 1024 tokens per update on two ranks: the second update has 276 tokens, 20 of them on the second rank
    assert full["step"] == 2 and full["tokens_seen"] == TRAIN_TOKENS and len(full["rng_by_rank"]) == 2
    work = work_dir(tmp_path, "split")
    launch(work, config, 2, [*extra, "--max-steps", "1"])
    launch(work, config, 2, extra)
    assert_bitwise(full, load(work))


@pytest.mark.multigpu
@needs_two_gpus
def test_one_to_two_gpu_reconfiguration_preserves_training_state(tmp_path):
    config = write_config(tmp_path / "cfg.json")
    serial = work_dir(tmp_path, "serial")
    launch(serial, config, 1, grad_accum=4)                    # 1024 tokens per update on one GPU
    expected = load(serial)
    moved = work_dir(tmp_path, "moved")
    launch(moved, config, 1, ["--max-steps", "1"], grad_accum=4)
    launch(moved, config, 2, ["--reconfigure"], grad_accum=2)  # the same 1024 tokens per update on two
    actual = load(moved)
    assert (actual["step"], actual["tokens_seen"]) == (expected["step"], expected["tokens_seen"]) == (2, TRAIN_TOKENS)
    assert actual["signature"]["settings"]["world_size"] == 2 and len(actual["rng_by_rank"]) == 2
    assert len(actual["execution_history"]) == 1
    for name, value in actual["model"].items():
        torch.testing.assert_close(value, expected["model"][name], rtol=0.01, atol=2e-5)
    for index, entry in actual["optimizer"]["state"].items():
        for key in ("exp_avg", "exp_avg_sq"):
            torch.testing.assert_close(entry[key], expected["optimizer"]["state"][index][key], rtol=0.03, atol=2e-7)
