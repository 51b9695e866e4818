"""`bench.py` on the CPU: the flags and defaults of its contract, the JSON line both arms print, the stream length and the
reference arm's answer when the reference is not installed.  Nothing here needs a GPU (no timed region is entered)."""
import importlib.util
import json
import sys
from argparse import Namespace
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture()
def bench(monkeypatch):
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def arguments(**changes):
    values = dict(gpus=1, steps=4, warmup=3, impl="ours", model="2b", micro_batch=8, grad_accum=4, seq_len=2048)
    values.update(changes)
    return Namespace(**values)


def test_defaults_are_the_headline_configuration(bench, monkeypatch):
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    monkeypatch.delenv("WARPSTATE_REF_COMPILE_MODE", raising=False)
    a = bench.parse()
    assert (a.gpus, a.impl, a.model, a.micro_batch, a.grad_accum, a.seq_len) == (1, "ours", "2b", 8, 4, 2048)
    assert a.warmup >= 3 and a.steps >= 1                                      # at least three untimed warm-up steps
    assert a.shard_params == "off" and not a.shard_optimizer and not a.activation_checkpointing and not a.bf16_residuals
    assert a.ref_compile_mode == "max-autotune-no-cudagraphs"
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "8", "--steps", "20", "--warmup", "5", "--impl", "reference"])
    a = bench.parse()
    assert (a.gpus, a.steps, a.warmup, a.impl) == (8, 20, 5, "reference")
    cfg = bench.model_config("2b")
    assert (cfg.d_model, cfg.n_cores, cfg.ffn_hidden, cfg.vocab_size, cfg.gradient_checkpointing) == (2048, 28, 7168, 32768, False)


@pytest.mark.parametrize("world", [1, 8])
def test_both_arms_print_the_same_workload_description(bench, capsys, world):
    clocks = {"sm_mhz": 1350.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"]}
    a = arguments(gpus=world)
    bench.emit(a, 0, world, 80000.0 * world, 819.2, 80100.0 * world, clocks, 57100, "ours",
               {"grad_sync": "fused-nvls"}, {"last_loss": 10.6}, 1048576 * world, 12 * world)
    bench.emit(a, 0, world, 64000.0 * world, 1024.0, 63900.0 * world, clocks, 0, "reference",
               {"compile_mode": "max-autotune-no-cudagraphs"}, {"last_loss": 10.7}, 1048576 * world, 8 * world)
    ours, reference = (json.loads(line) for line in capsys.readouterr().out.splitlines())
    assert ours["config"] == reference["config"]                               # the workload; settings live in "arm"
    assert ours["metric"] == reference["metric"] == "train tokens/sec @2.005B seq2048 (max over ranks)"
    assert (ours["impl"], reference["impl"]) == ("ours", "reference") and ours["arm"] != reference["arm"]
    config = ours["config"]
    assert config["global_batch"] == 32 * world and config["tokens_per_update"] == 65536 * world
    assert config["parallelism"] == f"dp{world}" and config["seq_len"] == 2048 and config["model"] == "warpstate-2.005B"
    assert "L2" in config["l2"] and "pinned-host" in config["e2e_region"]
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert key in ours, key
    assert ours["n_gpus"] == world and ours["higher_is_better"] is True and ours["scaling"] == "weak" and ours["dtype"] == "bf16"
    assert ours["vs_baseline"] == pytest.approx(80000.0 * world / 72499.0)
    assert ours["e2e"] == {"value": 80100.0 * world, "unit": "tokens/s", "h2d_bytes_per_step": 1048576 * world,
                           "d2h_bytes_per_step": 12 * world}
    assert ours["clocks"] == clocks and ours["gpu_launches"] == 57100 and "synthetic" in ours["data"]


def test_only_rank_zero_prints_and_the_smoke_model_has_no_baseline(bench, capsys):
    bench.emit(arguments(), 3, 8, 1.0, 1.0, 1.0, {}, 1, "ours", {}, {}, 0, 0)
    assert capsys.readouterr().out == ""
    bench.emit(arguments(model="smoke"), 0, 1, 5000.0, 1.0, 5000.0, {}, 1, "ours", {}, {}, 0, 0)
    line = json.loads(capsys.readouterr().out)
    assert line["vs_baseline"] is None and line["config"]["model"] == "warpstate-smoke" and "smoke" in line["metric"]


def test_the_token_stream_gives_every_update_its_own_window(bench):
    a = arguments(steps=20, warmup=5)
    update = 8 * 2048 * 4
    assert bench.stream_tokens(a, 1) == update * (5 + 2 * 20) + 1             # warm-up, device-timed and end-to-end regions
    assert bench.stream_tokens(a, 8) == 8 * update * 45 + 1


def test_reference_arm_says_so_when_the_reference_is_not_installed(bench, capsys, tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    before = list(sys.path)
    bench.run_reference(arguments(impl="reference"))
    assert json.loads(capsys.readouterr().out) == {"impl": "reference", "unavailable": "baseline/_ref is not installed"}
    assert sys.path == before                                                  # and it has not touched the import path


def test_more_gpus_than_processes_is_a_launch_error(bench, monkeypatch):
    import torch
    for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(name, raising=False)
    monkeypatch.setattr(torch.cuda, "set_device", lambda index: pytest.fail("no device may be touched before the check"))
    with pytest.raises(SystemExit, match="launch with torch.distributed.run"):
        bench.dist_setup(arguments(gpus=4))
