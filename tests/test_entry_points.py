"""The entry points a user of the reference expects at the repository root and as modules: they start, describe their
flags and exit 0 on ``--help``; every benchmark and tool module offers ``main``."""
import importlib
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
ROOT_SCRIPTS = {"run_40b.py": "--stage", "posttrain.py": "--config", "dpo.py": "--reference-cache-dir", "chat.py": "--snapshot",
                "prepare_posttrain_data.py": "--max-length"}
TOOLS = ["bench.train_bench", "bench.gemm_bench", "bench.grad_accum_bench", "bench.tune_gemm", "bench.decode_bench",
         "bench.profile_step", "bench.comm_profile", "bench.compare_runs", "bench.kernel_case", "bench.sharded_linear_bench",
         "bench.allreduce_bench", "bench.dpo_bench", "bench.decode_anatomy", "bench.validate_training",
         "analysis.loss_forecast", "orchestration.launcher", "orchestration.handoff", "orchestration.preflight",
         "orchestration.archive_dpo", "orchestration.transfer", "serve.posttrain_chat", "train.evaluate_snapshot",
         "data.prepare_posttrain"]


@pytest.mark.parametrize("script, flag", sorted(ROOT_SCRIPTS.items()))
def test_root_scripts_describe_their_flags(script, flag):
    run = subprocess.run([sys.executable, str(ROOT / script), "--help"], capture_output=True, text=True, timeout=180, cwd=ROOT)
    assert run.returncode == 0, run.stderr[-2000:]
    assert "usage:" in run.stdout and flag in run.stdout and "Traceback" not in run.stderr


@pytest.mark.parametrize("name", TOOLS)
def test_tools_are_importable_modules_with_a_main(name):
    module = importlib.import_module(f"warpstate_ai_b200.{name}")
    assert callable(getattr(module, "main", None)), name
    assert (module.__doc__ or "").strip(), f"{name} says nothing about itself"


REFERENCE = ROOT / "baseline" / "_ref"
SAME_FLAGS = ["posttrain.py", "dpo.py", "chat.py", "ops/posttrain_chat.py", "ops/launch_training.py", "ops/transfer_artifacts.py",
              "ops/posttrain_handoff.py", "ops/dpo_handoff.py", "ops/compare_communication_benchmarks.py",
              "ops/analyze_communication_profile.py", "ops/evaluate_sft_snapshot.py", "ops/archive_dpo.py",
              "ops/loss_curve_forecast.py", "ops/posttrain_preflight.py", "ops/dpo_preflight.py", "ops/benchmark_training.py",
              "ops/benchmark_gemm.py", "ops/benchmark_gradient_accumulation.py", "ops/tune_matmul.py", "ops/prepare_data.py", "run_40b.py"]


def _flags(script, cwd):
    import re
    run = subprocess.run([sys.executable, script, "--help"], capture_output=True, text=True, cwd=cwd, timeout=300)
    assert run.returncode == 0, (script, str(cwd), run.stderr[-1500:])
    return set(re.findall(r"(?<![\w-])--[a-z][a-z0-9-]*", run.stdout))


def test_every_flag_of_the_reference_entry_points_exists_here():
    """``--help`` of each script at the reference's path, here and in the installed reference: no flag of the reference
    is missing (this framework adds some of its own)."""
    if not (REFERENCE / "posttrain.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    from concurrent.futures import ThreadPoolExecutor
    jobs = [(script, where) for script in SAME_FLAGS for where in (ROOT, REFERENCE)]
    with ThreadPoolExecutor(max_workers=8) as pool:
        found = dict(zip(jobs, pool.map(lambda job: _flags(*job), jobs)))
    for script in SAME_FLAGS:
        missing = found[(script, REFERENCE)] - found[(script, ROOT)]
        assert not missing, (script, sorted(missing))
