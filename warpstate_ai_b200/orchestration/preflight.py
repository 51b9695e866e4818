"""GPU preflight gate run by the handoff guardians before a long SFT / DPO job.

A tiny fixture (d_model 32, a handful of conversations / preference pairs whose last global batch
leaves ranks with masked rows) is trained twice with the real entry point on the real devices:
continuously, and split after one update and resumed.  The gate accepts only if both runs
finish, model / optimizer agree within ``rtol 1e-5`` (counters and cursors exactly), and -- for
DPO -- the first evaluation loss equals ln 2 (policy == reference) and the frozen initialisation
file is unchanged.  The report (``report.json``) is what the guardian verifies
(reference ops/posttrain_preflight.py:30-268, ops/dpo_preflight.py:202-204).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
from pathlib import Path

import torch

from ..utils.io import atomic_json, digest
from .launcher import PACKAGE

TOKENIZER = PACKAGE / "tokenizer.model"


def fixture_rows(n: int):
    sft = [{"messages": [{"role": "user", "content": f"Count to {i}."},
                         {"role": "assistant", "content": " ".join(str(k) for k in range(1, i + 2))}]} for i in range(n)]
    dpo = [{"prompt": [{"role": "user", "content": f"Name the number after {i}."}],
            "chosen": [{"role": "assistant", "content": str(i + 1)}],
            "rejected": [{"role": "assistant", "content": f"Perhaps {i + 5}, or something else."}]} for i in range(n)]
    return sft, dpo


def build_fixture(root: Path, stage: str, processes: int, base_work_dir: Path | None = None) -> dict:
    """Model export, prepared data and plan of the gate's tiny run.  With ``base_work_dir`` the plan names the
    pretraining job's work directory, so the trainer children hold its pipeline lock (shared) while they run."""
    from .. import WarpStateConfig, WarpStateLM
    from ..ckpt.formats import export_chat_snapshot
    from ..data.prepare_posttrain import prepare
    root.mkdir(parents=True, exist_ok=True)
    tok = root / "tokenizer.model"
    tok.write_bytes(TOKENIZER.read_bytes())
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=32768, d_model=256, n_heads=4, n_cores=1, logical_depth=2, ffn_hidden=256,
                          chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    model = WarpStateLM(cfg)
    export_chat_snapshot({"config": vars(cfg).copy(), "model": model.state_dict(), "step": 1, "tokens_seen": 1,
                          "val_loss": 0.0, "origin": {"step": 1, "tokens_seen": 1}}, root / "init", tok,
                         {"path": "preflight-fixture"}, stage="sft" if stage == "dpo" else None)
    sft, dpo = fixture_rows(5 * processes + 1)
    prepare(root / "data", tok, 128, sft_rows=sft, dpo_rows=dpo, val_modulus=4)
    training = {"sequence_length": 128, "micro_batch": 2, "grad_accum": 1, "lr": 1e-3, "eval_every": 1,
                "save_every": 1, "eval_batches": 1, "workers": 1, "max_steps": 3}
    if stage == "dpo":
        training.update(beta=0.5, head_chunk_size=64)
        plan = {"format": "warpstate-dpo-plan-v1", "stage": "dpo", "training": training}
    else:
        plan = {"format": "warpstate-posttrain-plan-v1", "stage": "sft", "training": training}
    if base_work_dir is not None:
        from .launcher import workspace_root
        plan["handoff"] = {"base_work_dir": str(Path(base_work_dir).resolve().relative_to(workspace_root()))}
    (root / "plan.json").write_text(json.dumps(plan))
    return {"tokenizer": tok, "weights": root / "init/model.pt", "data": root / "data", "plan": root / "plan.json"}


def run_trainer(stage: str, fx: dict, work: Path, processes: int, device: str, extra=(), cache: Path | None = None) -> None:
    script = PACKAGE / ("dpo.py" if stage == "dpo" else "posttrain.py")
    command = [sys.executable, "-B"]
    if processes > 1:
        command += ["-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes", "1",
                    "--nproc-per-node", str(processes)]
    command += [str(script), "--config", str(fx["plan"]), "--work-dir", str(work), "--data-dir", str(fx["data"]),
                "--weights", str(fx["weights"]), "--tokenizer", str(fx["tokenizer"]), "--device", device, *extra]
    if stage == "dpo":
        command += ["--reference-cache-dir", str(cache)]
    env = dict(os.environ, PYTHONPATH=str(PACKAGE) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    subprocess.run(command, check=True, env=env)


def compare(a: dict, b: dict, rtol: float = 1e-5, atol: float = 1e-6) -> None:
    for key in ("step", "sample_cursor", "tokens_seen"):
        if a[key] != b[key]:
            raise ValueError(f"resumed run differs in {key}: {a[key]} vs {b[key]}")
    for name in a["model"]:
        if not torch.allclose(a["model"][name], b["model"][name], rtol=rtol, atol=atol):
            raise ValueError(f"resumed run differs in model tensor {name}")
    for index, entry in a["optimizer"]["state"].items():
        for field in ("exp_avg", "exp_avg_sq"):
            if not torch.allclose(entry[field], b["optimizer"]["state"][index][field], rtol=rtol, atol=atol):
                raise ValueError(f"resumed run differs in optimizer state {index}.{field}")


def run(stage: str, work: Path, processes: int, device: str, base_work_dir: Path | None = None,
        prepare_only: bool = False) -> dict:
    os.environ.setdefault("WARPSTATE_WORKSPACE", str(work.resolve()))
    root = work.resolve()
    fx = build_fixture(root / "fixture", stage, processes, base_work_dir)
    if prepare_only:                      # the fixture alone, made on the CPU; nothing is launched
        return {"prepared": True, "stage": stage, "processes": processes, **{key: str(path) for key, path in fx.items()},
                "weights_sha256": digest(fx["weights"])}
    base_hash = digest(fx["weights"])
    run_trainer(stage, fx, root / "continuous", processes, device, cache=root / "cache-a")
    run_trainer(stage, fx, root / "split", processes, device, extra=("--max-steps", "1"), cache=root / "cache-b")
    run_trainer(stage, fx, root / "split", processes, device, cache=root / "cache-b")
    a = torch.load(root / "continuous/latest.pt", map_location="cpu", weights_only=False)
    b = torch.load(root / "split/latest.pt", map_location="cpu", weights_only=False)
    compare(a, b)
    events = [json.loads(line) for line in (root / "continuous/metrics.jsonl").read_text().splitlines()]
    first_eval = next(e for e in events if e["event"] == "validation")
    report = {"format": f"warpstate-{'dpo' if stage == 'dpo' else 'posttrain'}-preflight-v1", "accepted": True,
              "processes": processes, "device": device, "bf16_compute": device == "cuda" or True,
              "fp32_parameters_and_adam": all(t.dtype == torch.float32 for t in a["model"].values() if t.is_floating_point()),
              "steps": a["step"], "initial_validation_loss": first_eval["val_loss"],
              "generator_sha256": digest(__file__)}
    if stage == "dpo":
        if abs(first_eval["val_loss"] - math.log(2.0)) > 1e-4:
            raise ValueError(f"initial DPO loss {first_eval['val_loss']} is not ln 2")
        report["frozen_reference_unchanged"] = digest(fx["weights"]) == base_hash
        if not report["frozen_reference_unchanged"]:
            raise ValueError("the frozen initialisation changed during the preflight")
    return report


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--stage", choices=["sft", "dpo"], default="sft")
    p.add_argument("--work-dir", type=Path, required=True)
    p.add_argument("--processes", type=int, default=2)
    p.add_argument("--device", choices=["cuda", "cpu"], default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--base-work-dir", type=Path,
                   help="work directory of the pretraining job: the gate's trainers then hold its pipeline lock (shared)")
    p.add_argument("--prepare-only", action="store_true", help="create the fixture on the CPU and stop; never launches training")
    a = p.parse_args(argv)
    if a.base_work_dir is not None:
        from .launcher import workspace_root
        if not a.base_work_dir.is_dir() or not a.base_work_dir.resolve().is_relative_to(workspace_root()):
            p.error("--base-work-dir must be an existing directory inside the workspace")
    a.work_dir.mkdir(parents=True, exist_ok=True)
    if a.prepare_only:
        print(json.dumps(run(a.stage, a.work_dir, a.processes, a.device, a.base_work_dir, prepare_only=True)), flush=True)
        return 0
    try:
        report = run(a.stage, a.work_dir, a.processes, a.device, a.base_work_dir)
    except BaseException as error:  # noqa: BLE001
        atomic_json(a.work_dir / "report.json", {"accepted": False, "error": f"{type(error).__name__}: {error}"})
        raise
    atomic_json(a.work_dir / "report.json", report)
    print(json.dumps(report), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
