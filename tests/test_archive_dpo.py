"""Sealed archive of a completed DPO run and its chat copy (reference test_archive_dpo.py): a tiny
CPU DPO run to completion, archive, verify, idempotence, tamper and stale-state rejection."""
import json
import os
from pathlib import Path

import pytest
import torch

from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
from warpstate_ai_b200.ckpt.formats import export_chat_snapshot
from warpstate_ai_b200.data.prepare_posttrain import prepare
from warpstate_ai_b200.orchestration import archive_dpo as AD
from warpstate_ai_b200.train import dpo as DPO

ROOT = Path(__file__).resolve().parents[1]


def pairs(n):
    return [{"prompt": [{"role": "user", "content": f"What follows {i}?"}],
             "chosen": [{"role": "assistant", "content": str(i + 1)}],
             "rejected": [{"role": "assistant", "content": f"maybe {i + 3} or so"}]} for i in range(n)]


@pytest.fixture(scope="module")
def finished_run(tmp_path_factory):
    root = tmp_path_factory.mktemp("dpo-archive") / "ws"
    root.mkdir()
    old = os.environ.get("WARPSTATE_WORKSPACE")
    os.environ["WARPSTATE_WORKSPACE"] = str(root)
    try:
        tok = root / "tokenizer.model"
        tok.write_bytes((ROOT / "tokenizer.model").read_bytes())
        torch.manual_seed(0)
        cfg = WarpStateConfig(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24,
                              chunk_size=8, gradient_checkpointing=False, parallel_memory=True)
        ckpt = {"config": vars(cfg).copy(), "model": WarpStateLM(cfg).state_dict(), "step": 4, "tokens_seen": 400,
                "val_loss": 9.0, "origin": {"step": 7, "tokens_seen": 700}}
        export_chat_snapshot(ckpt, root / "sft-export", tok, {"path": "test"}, stage="sft")
        prepare(root / "data", tok, 64, dpo_rows=pairs(14), val_modulus=5)
        plan = root / "plan.json"
        plan.write_text(json.dumps({
            "format": "warpstate-dpo-plan-v1", "stage": "dpo", "sft": {"step": 4, "tokens_seen": 400},
            "training": {"sequence_length": 64, "micro_batch": 2, "grad_accum": 2, "lr": 1e-3, "eval_every": 2,
                         "save_every": 2, "eval_batches": 2, "workers": 1, "beta": 0.5, "head_chunk_size": 16},
            "handoff": {"processes": 1, "work_dir": "dpo", "data_dir": "data", "tokenizer": "tokenizer.model"}}))
        DPO.STOP = False
        DPO.main(["--config", str(plan), "--data-dir", str(root / "data"), "--weights", str(root / "sft-export/model.pt"),
                  "--tokenizer", str(tok), "--device", "cpu", "--reference-cache-dir", str(root / "dpo/reference-cache"),
                  "--work-dir", str(root / "dpo/run")])
        yield root, tok, plan
    finally:
        if old is None:
            os.environ.pop("WARPSTATE_WORKSPACE", None)
        else:
            os.environ["WARPSTATE_WORKSPACE"] = old


def build(root, tok, plan, name="final"):
    return AD.archive_dpo(root / "dpo/run", root / "data", root / "dpo/reference-cache", tok, plan, root / "archives" / name, "rev")


def test_archive_verify_idempotent_and_chat_copy(finished_run):
    root, tok, plan = finished_run
    meta = build(root, tok, plan)
    archive = root / "archives/final"
    assert meta["stage"] == "dpo" and {p.name for p in archive.iterdir()} == set(AD.FILES) | {"SHA256SUMS"}
    assert all(not (p.stat().st_mode & 0o222) for p in archive.iterdir())
    again = build(root, tok, plan)  # verifies, does not rewrite
    assert again["snapshot_sha256"] == meta["snapshot_sha256"]
    metadata, entries = AD.verify_dpo_archive(archive)
    full = torch.load(archive / "checkpoint.pt", weights_only=False)
    assert full["completed"] is True and full["optimizer"]["state"] and metadata["step"] == full["step"]
    model = AD.chat_copy(archive, root / "chat/dpo-final")
    assert model.exists() and model.stat().st_ino != (archive / "model.pt").stat().st_ino
    assert AD.chat_copy(archive, root / "chat/dpo-final") == model
    assert AD.main(["--chat-copy", str(root / "chat/second"), "--archive", str(archive)]) == 0
    # the sealed chat copy loads in the chat CLI's snapshot verifier
    from warpstate_ai_b200.ckpt.formats import verify_chat_snapshot
    assert verify_chat_snapshot(root / "chat/dpo-final", tok)["stage"] == "dpo"


def test_tampered_or_extended_archive_is_rejected(finished_run):
    root, tok, plan = finished_run
    build(root, tok, plan, "victim")
    victim = root / "archives/victim"
    os.chmod(victim, 0o755)
    (victim / "extra.txt").write_text("x")
    os.chmod(victim, 0o555)
    with pytest.raises(ValueError, match="unexpected files"):
        AD.verify_dpo_archive(victim)
    os.chmod(victim, 0o755)
    (victim / "extra.txt").unlink()
    os.chmod(victim / "evaluation.json", 0o644)
    report = json.loads((victim / "evaluation.json").read_text())
    report["reward_accuracy"] = 0.123
    (victim / "evaluation.json").write_text(json.dumps(report))
    os.chmod(victim / "evaluation.json", 0o444)
    os.chmod(victim, 0o555)
    with pytest.raises(ValueError, match="checksum mismatch"):
        AD.verify_dpo_archive(victim)
    with pytest.raises(ValueError, match="differs from the source checkpoint"):
        AD.verify_dpo_archive(root / "archives/final", expected_checkpoint_hash="0" * 64)


def test_incomplete_or_capped_runs_are_not_archived(finished_run):
    root, tok, plan = finished_run
    ckpt = torch.load(root / "dpo/run/latest.pt", weights_only=False)
    reports = [json.loads((root / "dpo/run" / n).read_text()) for n in ("evaluation.json", "completion.json", "settings.json")]
    data = json.loads((root / "data/manifest.json").read_text())
    ref = json.loads((root / "dpo/reference-cache/manifest.json").read_text())
    p = json.loads(plan.read_text())
    AD.validate_state(ckpt, *reports, data, ref, p)
    with pytest.raises(ValueError, match="step cap"):
        capped = json.loads(plan.read_text())
        capped["training"]["max_steps"] = 2
        AD.validate_state(ckpt, *reports, data, ref, capped)
    with pytest.raises(ValueError, match="fully completed"):
        AD.validate_state(dict(ckpt, step=ckpt["step"] - 1), *reports, data, ref, p)
    with pytest.raises(ValueError, match="completion report"):
        AD.validate_state(ckpt, reports[0], dict(reports[1], val_loss=0.0), reports[2], data, ref, p)
    with pytest.raises(ValueError, match="fixed-reference identity"):
        AD.validate_state(ckpt, *reports, data, dict(ref, identity=dict(ref["identity"], world_size=2)), p)


def test_guardian_records_travel_with_the_archive_and_the_layout_is_the_reference_one(finished_run):
    root, tok, plan = finished_run
    without = root / "archives/final"
    if not without.exists():
        build(root, tok, plan)
    for name in AD.GUARDIAN_RECORDS:                       # this run had no guardian: the archive says so
        assert json.loads((without / name).read_text()) == AD.NO_GUARDIAN
    records = {"control/execution.json": {"format": "execution", "processes": 1}, "control/handoff.json": {"phase": "complete"},
               "preflight/report.json": {"passed": True, "ranks": 1}}
    for leaf, content in records.items():
        path = root / "dpo" / leaf
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(content))
    build(root, tok, plan, name="guarded")
    guarded = root / "archives/guarded"
    for name, leaf in AD.GUARDIAN_RECORDS.items():
        assert json.loads((guarded / name).read_text()) == records[leaf]
        assert (guarded / name).stat().st_ino != (root / "dpo" / leaf).stat().st_ino      # an independent copy
    AD.verify_dpo_archive(guarded)
    listing = [line.split("  ", 1)[1] for line in (guarded / "SHA256SUMS").read_text().splitlines()]
    assert listing == list(AD.FILES)
    reference_list = ROOT / "baseline" / "_ref" / "ops" / "archive_dpo.py"
    if reference_list.exists():                            # the file list of the reference's archive, read as text
        import ast
        tree = ast.parse(reference_list.read_text())
        files = next(ast.literal_eval(node.value) for node in tree.body
                     if isinstance(node, ast.Assign) and getattr(node.targets[0], "id", "") == "FILES")
        assert tuple(files) == AD.FILES


def test_a_guarded_run_is_archived_only_after_its_guardian_is_done(tmp_path, monkeypatch):
    from warpstate_ai_b200.orchestration import handoff as H
    work = tmp_path / "dpo"
    (work / "control").mkdir(parents=True)
    asked = []

    def status(socket_path, program):
        asked.append((Path(socket_path), program))
        return state

    monkeypatch.setattr(H, "process_status", status)
    section = {"supervisor_socket": "control/supervisor.sock"}
    AD.guardian_done(tmp_path, {"work_dir": "dpo"}, work, "warpstate-dpo")            # no guardian in the plan: nothing to ask
    assert asked == []
    state = {"statename": "RUNNING"}
    with pytest.raises(ValueError, match="must have exited successfully"):
        AD.guardian_done(tmp_path, section, work, "warpstate-dpo")
    state = {"statename": "EXITED", "exitstatus": 3}
    with pytest.raises(ValueError, match="must have exited successfully"):
        AD.guardian_done(tmp_path, section, work, "warpstate-dpo")
    state = {"statename": "EXITED", "exitstatus": 0}
    with pytest.raises(ValueError, match="has not completed its final integrity checks"):
        AD.guardian_done(tmp_path, section, work, "warpstate-dpo")                    # no journal yet
    (work / "control/handoff.json").write_text(json.dumps({"phase": "paused"}))
    with pytest.raises(ValueError, match="has not completed"):
        AD.guardian_done(tmp_path, section, work, "warpstate-dpo")
    (work / "control/handoff.json").write_text(json.dumps({"phase": "complete"}))
    AD.guardian_done(tmp_path, section, work, "my-dpo-program")
    assert asked[-1] == (tmp_path / "control/supervisor.sock", "my-dpo-program")
