"""The production-shaped training validation harness (`bench/validate_training.py`).

CPU: the harness itself on a small shape -- every arm is the FP32 PyTorch definition there, so every comparison must be
exact and the checkpoint continuation byte-identical.  GPU: the real thing, one production-shaped core (d_model 2048,
32 heads, FFN 7168, sequence 2048) trained by the PyTorch definition and by the fused kernel path, judged against
the declared tolerance table; on two GPUs each arm also synchronises gradients its own way.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def run_harness(out: Path, *flags, gpus: int = 1, port: int = 29641):
    command = [sys.executable]
    if gpus > 1:
        command += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
                    "--master-port", str(port)]
    command += ["-m", "warpstate_ai_b200.bench.validate_training", "--output-dir", str(out), *flags]
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    done = subprocess.run(command, env=env, cwd=ROOT, capture_output=True, text=True, timeout=1500)
    report = json.loads((out / "report.json").read_text()) if (out / "report.json").exists() else None
    return done, report


def test_harness_logic_on_cpu(tmp_path):
    done, report = run_harness(tmp_path / "v", "--shape", "small", "--seq-len", "256", "--micro-batch", "1", "--device", "cpu")
    assert done.returncode == 0, done.stderr[-2000:]
    assert report["passed"] and report["resumed_byte_identical"] and report["failures"] == []
    assert report["worst"] == {"gradient": 0.0, "moment": 0.0, "parameter": 0.0}
    assert len(report["losses"]["fused"]) == 3 and any(k.startswith("gradient:cores.0.in_proj") for k in report["fused_vs_exact"])
    again, _ = run_harness(tmp_path / "v", "--shape", "small", "--seq-len", "256", "--micro-batch", "1", "--device", "cpu")
    assert again.returncode != 0          # the output directory must be fresh


@pytest.mark.gpu
def test_production_shaped_core_fused_against_pytorch_definition(tmp_path):
    done, report = run_harness(tmp_path / "v", "--cores", "1", "--micro-batch", "2")
    assert report is not None, (done.stdout[-2000:], done.stderr[-3000:])
    assert report["passed"] and done.returncode == 0, (report["worst"], report["failures"][:10], report["losses"])
    assert report["resumed_byte_identical"]
    assert report["fixture"]["seq_len"] == 2048
    # no further from the FP32 definition than PyTorch's own BF16 path is (declared margin 1.5), and small in itself
    assert report["worst"]["gradient"] <= max(0.005, 1.5 * report["worst_stock"]["gradient"]) and report["worst"]["gradient"] < 0.02


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two CUDA devices")
def test_production_shaped_core_on_two_gpus(tmp_path):
    done, report = run_harness(tmp_path / "v", "--cores", "1", "--micro-batch", "1", gpus=2)
    assert report is not None, (done.stdout[-2000:], done.stderr[-3000:])
    assert report["passed"] and report["passed_on_every_rank"] and done.returncode == 0, (report["worst"], report["failures"][:10])
