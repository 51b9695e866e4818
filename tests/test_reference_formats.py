"""Files written by one implementation are read by the other: plan documents, the DPO reference-score cache and sealed
chat exports, with the reference imported as a library from ``baseline/_ref`` (skipped where it is not installed)."""
import importlib
import json
from dataclasses import asdict
from pathlib import Path

import numpy as np
import pytest
import torch

from test_reference_parity import REF, reference_import_path

TOK = Path(__file__).resolve().parents[1] / "tokenizer.model"


@pytest.fixture(scope="module")
def ref():
    if not (REF / "posttrain.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    with reference_import_path():
        return {name: importlib.import_module(name) for name in ("posttrain", "dpo", "chat")}


# ------------------------------------------------------------------------------------------- plan documents
TRAINING_SECTIONS = [
    {}, {"lr": 2e-5, "min_lr": 2e-6, "max_steps": 7}, {"lr": 1, "warmup_ratio": 0}, {"sequence_length": 4096, "micro_batch": 1, "grad_accum": 64},
    {"compile_core": False, "bf16_residuals": False, "gradient_checkpointing": True, "deterministic": False},
    # refused by both
    {"lr": 0}, {"lr": -1e-5}, {"min_lr": 1e-3}, {"lr": "1e-5"}, {"lr": float("inf")}, {"clip_grad_norm": 0}, {"weight_decay": -0.1},
    {"warmup_ratio": 1}, {"warmup_ratio": True}, {"warmup_ratio": -0.1}, {"micro_batch": 0}, {"micro_batch": 2.0}, {"epochs": True},
    {"max_steps": 0}, {"max_steps": 1.5}, {"seed": -1}, {"seed": 1.0}, {"compile_core": 1}, {"deterministic": "yes"},
    {"unknown_key": 1}, {"workers": 0}, {"eval_every": None},
]


def verdict(load, document, path):
    path.write_text(json.dumps(document))
    try:
        return load(path)[1]
    except ValueError:
        return "refused"


@pytest.mark.parametrize("training", TRAINING_SECTIONS, ids=lambda t: ",".join(f"{k}={v}" for k, v in t.items()) or "defaults")
def test_plans_mean_the_same_to_both(ref, tmp_path, training):
    from warpstate_ai_b200.train.plans import DPO_PLAN, SFT_PLAN
    sft = {"format": "warpstate-posttrain-plan-v1", "stage": "sft", "training": training}
    assert verdict(SFT_PLAN.read, sft, tmp_path / "a.json") == verdict(ref["posttrain"].load_plan, sft, tmp_path / "b.json")
    dpo = {"format": "warpstate-dpo-plan-v1", "stage": "dpo", "training": training}
    mine, theirs = verdict(DPO_PLAN.read, dpo, tmp_path / "c.json"), verdict(ref["dpo"].load_plan, dpo, tmp_path / "d.json")
    if theirs == "refused":
        assert mine == "refused"
    else:
        assert {k: mine[k] for k in theirs} == theirs and set(mine) - set(theirs) == {"reference_mode"}


def test_stage_specific_keys_and_wrong_documents(ref, tmp_path):
    from warpstate_ai_b200.train.plans import DPO_PLAN, SFT_PLAN
    cases = [({"loss_mode": "full"}, "sft"), ({"loss_mode": "fused"}, "sft"), ({"beta": 0.1, "objective": "summed-dpo"}, "dpo"),
             ({"beta": 0}, "dpo"), ({"objective": "ipo"}, "dpo"), ({"head_chunk_size": 0}, "dpo"), ({"beta": 0.1}, "sft"), ({"loss_mode": "full"}, "dpo")]
    for training, stage in cases:
        schema, load, plan_format = ((SFT_PLAN, ref["posttrain"].load_plan, "warpstate-posttrain-plan-v1") if stage == "sft"
                                     else (DPO_PLAN, ref["dpo"].load_plan, "warpstate-dpo-plan-v1"))
        document = {"format": plan_format, "stage": stage, "training": training}
        mine, theirs = verdict(schema.read, document, tmp_path / "m.json"), verdict(load, document, tmp_path / "t.json")
        assert (mine == "refused") == (theirs == "refused"), (training, stage)
        if theirs != "refused":
            assert {k: mine[k] for k in theirs} == theirs
    for document in ({}, {"format": "warpstate-dpo-plan-v1", "stage": "sft"}, {"format": "warpstate-posttrain-plan-v1", "stage": "dpo"}):
        assert verdict(SFT_PLAN.read, document, tmp_path / "m.json") == verdict(ref["posttrain"].load_plan, document, tmp_path / "t.json") == "refused"
        assert verdict(DPO_PLAN.read, document, tmp_path / "m.json") == verdict(ref["dpo"].load_plan, document, tmp_path / "t.json") == "refused"


# ------------------------------------------------------------------------------------------- DPO reference cache
def test_a_score_cache_written_here_is_accepted_by_the_reference(ref, tmp_path):
    from warpstate_ai_b200.train.reference_cache import ReferenceScoreCache
    identity = {"format": "warpstate-dpo-reference-v1", "weights_sha256": "aa", "data_sha256": "bb", "settings": {"micro_batch": 2},
                "dropout": 0.0, "world_size": 2}
    train = [{"id": i} for i in range(9)]
    val = [{"id": 50 + i} for i in range(4)]
    score = lambda rows: np.array([[-1.5 * r["id"] - 0.25, -0.5 * r["id"] - 3.0] for r in rows], dtype=np.float64).reshape(-1, 2)
    caches = [ReferenceScoreCache(tmp_path / "cache", identity, (9, 4)) for _ in range(2)]
    for rank, cache in enumerate(caches):
        cache.claim(rank)
        assert cache.score((train, val), score, 2, rank, 2, lambda: False)
    caches[0].merge(2)
    mine = caches[0].verify()
    theirs = ref["dpo"].validate_cache(tmp_path / "cache", identity, (9, 4))
    assert np.array_equal(mine[0], theirs[0]) and np.array_equal(mine[1], theirs[1]) and mine[2] == theirs[2]
    assert np.array_equal(theirs[0], score(train)) and theirs[1].dtype == np.float64
    with pytest.raises(ValueError):
        ref["dpo"].validate_cache(tmp_path / "cache", dict(identity, weights_sha256="cc"), (9, 4))
    with pytest.raises(ValueError):
        ref["dpo"].validate_cache(tmp_path / "cache", identity, (9, 5))
    table = np.load(tmp_path / "cache" / "val.npy")
    table[0, 0] += 1.0
    np.save(tmp_path / "cache" / "val.npy", table)
    for check in (caches[0].verify, lambda: ref["dpo"].validate_cache(tmp_path / "cache", identity, (9, 4))):
        with pytest.raises(ValueError):
            check()


# ------------------------------------------------------------------------------------------- chat exports
def training_checkpoint(path):
    from warpstate_ai_b200.ckpt.formats import SERVER_FORMAT
    from warpstate_ai_b200.config import WarpStateConfig
    from warpstate_ai_b200.models.warpstate import WarpStateLM
    from warpstate_ai_b200.utils.io import digest
    torch.manual_seed(5)
    cfg = WarpStateConfig(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=4,
                          gradient_checkpointing=False, parallel_memory=True)
    model = WarpStateLM(cfg)
    with torch.no_grad():
        model.depth_scale.normal_(0, 0.1)
        model.depth_bias.normal_(0, 0.1)
    path.parent.mkdir(parents=True, exist_ok=True)
    torch.save({"format": SERVER_FORMAT, "signature": {"data": {"signature": {"tokenizer_sha256": digest(TOK)}}}, "config": asdict(cfg),
                "model": model.state_dict(), "optimizer": {"state": {}}, "step": 7, "tokens_seen": 112, "val_loss": 9.5}, path)
    return model


def stepped_logits(model, ids):
    caches = model.init_generation_cache(1, torch.device("cpu"), torch.float32)
    with torch.no_grad():
        return torch.cat([model.step(ids[:, i:i + 1], caches) for i in range(ids.shape[1])], dim=1)


def test_exports_of_either_implementation_load_in_the_other(ref, tmp_path):
    from warpstate_ai_b200.serve.snapshots import SnapshotStore
    source = tmp_path / "run" / "latest.pt"
    trained = training_checkpoint(source)
    ids = torch.randint(0, 32768, (1, 10))
    wanted = stepped_logits(trained.eval(), ids)
    store = SnapshotStore(tmp_path / "ours", TOK)
    exported_here = store.export(source)
    exported_there = ref["chat"].capture_latest(source, TOK, tmp_path / "theirs")
    # same layout on disk, same sealed fields
    seal_here, seal_there = (json.loads(p.with_name("snapshot.json").read_text()) for p in (exported_here, exported_there))
    assert set(seal_here) == set(seal_there)
    for key in ("format", "inference_only", "config", "step", "tokens_seen", "val_loss", "tokenizer_sha256", "source"):
        assert seal_here[key] == seal_there[key], key
    payload_here, payload_there = (torch.load(p, weights_only=False) for p in (exported_here, exported_there))
    assert set(payload_here) == set(payload_there) and "optimizer" not in payload_here
    # each loader accepts the other's export and the model computes the same logits
    model_a, _, meta_a = ref["chat"].load_model(exported_here, TOK)
    model_b, _, meta_b = store.load(exported_there)
    assert meta_a["step"] == meta_b["step"] == 7
    assert torch.allclose(stepped_logits(model_a, ids), wanted, rtol=1e-5, atol=1e-6)
    assert torch.allclose(stepped_logits(model_b, ids), wanted, rtol=1e-5, atol=1e-6)
    assert ref["chat"].resolve_snapshot(exported_here, TOK, tmp_path / "unused") == exported_here
    assert store.resolve(exported_there) == exported_there and not (tmp_path / "unused").exists()
    # and both refuse the other's export once it is tampered with
    exported_here.chmod(0o644)
    with open(exported_here, "ab") as stream:
        stream.write(b"x")
    with pytest.raises(ValueError):
        ref["chat"].load_model(exported_here, TOK)
    exported_there.chmod(0o644)
    with open(exported_there, "ab") as stream:
        stream.write(b"x")
    with pytest.raises(ValueError):
        store.load(exported_there)


# ------------------------------------------------------------------------------------------- training checkpoints
def test_a_checkpoint_of_this_trainer_is_a_reference_checkpoint(ref, tmp_path):
    """`run_40b.py --device cpu` here, then the reference's own readers: its chat export, its model, its optimizer."""
    from warpstate_ai_b200.data import prepare as P
    from warpstate_ai_b200.train import pretrain as T
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(dict(vocab_size=32768, d_model=16, n_heads=2, n_cores=2, logical_depth=4, ffn_hidden=24, chunk_size=4,
                                        gradient_checkpointing=False, parallel_memory=True)))
    work = tmp_path / "work"
    P.write_synthetic_corpus(work, TOK, 73, 64, 32768, seed=1)
    T.STOP = False
    T.main(["--from-scratch", "--work-dir", str(work), "--config", str(cfg_path), "--tokenizer", str(TOK), "--stage", "train",
            "--device", "cpu", "--test-small-gpu", "--train-tokens", "73", "--val-tokens", "64", "--seq-len", "8", "--micro-batch", "2",
            "--grad-accum", "2", "--warmup-steps", "1", "--max-steps", "2", "--eval-batches", "1", "--no-activation-checkpointing",
            "--dataset", "synthetic/uniform", "--dataset-config", "none", "--revision", "0"])
    latest = work / "run" / "latest.pt"
    checkpoint = torch.load(latest, weights_only=False)
    assert checkpoint["format"] == "warpstate-server-v1" and checkpoint["step"] == 2
    with reference_import_path():
        run_40b = importlib.import_module("run_40b")
        warpstate = importlib.import_module("warpstate")
    # the reference's resume check reads the stored signature (its keys are all there; ours are extra settings)
    assert run_40b.check_resume_signature(checkpoint["signature"], checkpoint["signature"]) is False
    for key in ("seq_len", "micro_batch", "grad_accum", "train_tokens", "lr", "min_lr", "warmup_steps", "weight_decay", "seed",
                "activation_checkpointing", "loss_chunk_size", "compile", "world_size", "loss_mode", "ddp_bucket_cap_mb"):
        assert key in checkpoint["signature"]["settings"], key
    # model and optimizer state load into the reference's classes, parameter for parameter
    model = warpstate.WarpStateLM(warpstate.WarpStateConfig(**checkpoint["config"]))
    model.load_state_dict(checkpoint["model"], strict=True)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1.0, betas=(0.5, 0.5))
    optimizer.load_state_dict(checkpoint["optimizer"])
    group = optimizer.param_groups[0]
    assert group["betas"] == (0.9, 0.95) and group["eps"] == 1e-8 and len(group["params"]) == len(list(model.parameters()))
    for parameter in model.parameters():
        state = optimizer.state[parameter]
        assert state["exp_avg"].shape == parameter.shape == state["exp_avg_sq"].shape and float(state["step"]) == 2.0
    assert any(float(optimizer.state[p]["exp_avg"].abs().sum()) > 0 for p in model.parameters())
    for key in ("rng_by_rank", "rng_torch", "rng_cuda", "rng_numpy", "rng_python", "tokens_seen", "val_loss", "origin", "execution_history"):
        assert key in checkpoint, key
    # and its chat probe exports and loads it
    exported = ref["chat"].capture_latest(latest, TOK, tmp_path / "snaps")
    probe, _, metadata = ref["chat"].load_model(exported, TOK)
    assert metadata["step"] == 2 and metadata["tokens_seen"] == checkpoint["tokens_seen"]
    ids = torch.randint(0, 32768, (1, 6))
    assert torch.allclose(stepped_logits(probe, ids), stepped_logits(model.eval(), ids), rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------------------------------- a finished DPO run and its archive
def test_a_dpo_run_of_this_trainer_satisfies_the_reference_archive_verifier(ref, tmp_path, monkeypatch):
    """A tiny DPO run to completion with this trainer; the reference's own validator of run records and its verifier of
    sealed archives accept what was written.  (The one concession: its table of defaults is told about
    ``reference_mode``, the setting this framework adds to the plan.)"""
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.ckpt.formats import export_chat_snapshot
    from warpstate_ai_b200.data.prepare_posttrain import prepare
    from warpstate_ai_b200.orchestration import archive_dpo as AD
    from warpstate_ai_b200.train import dpo as DPO
    from warpstate_ai_b200.utils.io import digest
    root = tmp_path / "ws"
    root.mkdir()
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(root))
    tok = root / "tokenizer.model"
    tok.write_bytes(TOK.read_bytes())
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=8,
                          gradient_checkpointing=False, parallel_memory=True)
    sft = {"config": vars(cfg).copy(), "model": WarpStateLM(cfg).state_dict(), "step": 4, "tokens_seen": 400, "assistant_tokens_seen": 90,
           "val_loss": 9.0, "origin": {"step": 7, "tokens_seen": 700}}
    exported = export_chat_snapshot(sft, root / "sft-export", tok, {"path": "test"}, stage="sft")
    assert exported["assistant_tokens_seen"] == 90 and exported["inference_only"] is True and exported["origin"] == sft["origin"]
    pairs = [{"prompt": [{"role": "user", "content": f"What follows {i}?"}], "chosen": [{"role": "assistant", "content": str(i + 1)}],
              "rejected": [{"role": "assistant", "content": f"maybe {i + 3} or so"}]} for i in range(14)]
    prepare(root / "data", tok, 64, dpo_rows=pairs, val_modulus=5)
    plan = {"format": "warpstate-dpo-plan-v1", "stage": "dpo",
            "sft": {"step": 4, "tokens_seen": 400, "base_step": 7, "base_tokens_seen": 700, "tokenizer_sha256": digest(tok)},
            "training": {"sequence_length": 64, "micro_batch": 2, "grad_accum": 2, "lr": 1e-3, "eval_every": 2, "save_every": 2,
                         "eval_batches": 2, "workers": 1, "beta": 0.5, "head_chunk_size": 16},
            "handoff": {"processes": 1, "work_dir": "dpo", "data_dir": "data", "tokenizer": "tokenizer.model",
                        "data_manifest_sha256": digest(root / "data/manifest.json")}}
    plan_path = root / "plan.json"
    plan_path.write_text(json.dumps(plan))
    monkeypatch.setattr(DPO, "STOP", False)
    DPO.main(["--config", str(plan_path), "--data-dir", str(root / "data"), "--weights", str(root / "sft-export/model.pt"),
              "--tokenizer", str(tok), "--device", "cpu", "--reference-cache-dir", str(root / "dpo/reference-cache"),
              "--work-dir", str(root / "dpo/run")])
    run = root / "dpo/run"
    with reference_import_path():
        theirs = importlib.import_module("ops.archive_dpo")
    monkeypatch.setattr(theirs, "DEFAULTS", dict(theirs.DEFAULTS, reference_mode="cached"))
    read = lambda path: json.loads(Path(path).read_text())
    checkpoint = torch.load(run / "latest.pt", weights_only=False)
    counters = theirs.validate_state(checkpoint, read(run / "evaluation.json"), read(run / "completion.json"), read(run / "settings.json"),
                                     read(root / "data/manifest.json"), read(root / "dpo/reference-cache/manifest.json"), plan)
    assert counters["step"] == checkpoint["step"] == 2 and counters["response_tokens_seen"] == checkpoint["response_tokens_seen"]
    AD.archive_dpo(run, root / "data", root / "dpo/reference-cache", tok, plan_path, root / "archives/final", "rev")
    metadata, entries = theirs.verify_dpo_archive(root / "archives/final", expected_checkpoint_hash=digest(run / "latest.pt"))
    mine, my_entries = AD.verify_dpo_archive(root / "archives/final")
    assert metadata == mine and entries == my_entries and metadata["stage"] == "dpo" and metadata["response_tokens_seen"] == 77
    with pytest.raises(ValueError):
        theirs.verify_dpo_archive(root / "archives/final", expected_checkpoint_hash="0" * 64)


def test_an_sft_run_of_this_trainer_satisfies_the_reference_archive_verifier(ref, tmp_path, monkeypatch):
    """A tiny SFT run to completion, sealed by this framework's SFT -> DPO guardian; the reference's verifier of SFT
    archives accepts it.  (The one concession: the reference insists on the RNG state of exactly two ranks; this run has
    one, so its validator is shown the list twice.)"""
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.ckpt.formats import export_chat_snapshot
    from warpstate_ai_b200.data.prepare_posttrain import prepare
    from warpstate_ai_b200.orchestration import archive as A
    from warpstate_ai_b200.orchestration import handoff as H
    from warpstate_ai_b200.train import sft as SFT
    from warpstate_ai_b200.utils.io import digest
    root = tmp_path / "ws"
    root.mkdir()
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(root))
    tok = root / "tokenizer.model"
    tok.write_bytes(TOK.read_bytes())
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=8,
                          gradient_checkpointing=False, parallel_memory=True)
    base = {"config": vars(cfg).copy(), "model": WarpStateLM(cfg).state_dict(), "step": 7, "tokens_seen": 700, "val_loss": 9.9}
    export_chat_snapshot(base, root / "base", tok, {"path": "test"})
    rows = [{"messages": [{"role": "user", "content": f"What is {i} plus {i + 1}?"}, {"role": "assistant", "content": f"It is {2 * i + 1}."}]}
            for i in range(12)]
    prepare(root / "data", tok, 64, sft_rows=rows, val_modulus=5)
    sft_plan = {"format": "warpstate-posttrain-plan-v1", "stage": "sft", "base": {"step": 7, "tokens_seen": 700, "tokenizer_sha256": digest(tok)},
                "training": {"sequence_length": 64, "micro_batch": 2, "grad_accum": 2, "lr": 1e-3, "eval_every": 2, "save_every": 2,
                             "eval_batches": 2, "workers": 1}}
    (root / "sft-plan.json").write_text(json.dumps(sft_plan))
    monkeypatch.setattr(SFT, "STOP", False)
    SFT.main(["--config", str(root / "sft-plan.json"), "--data-dir", str(root / "data"), "--weights", str(root / "base/model.pt"),
              "--tokenizer", str(tok), "--device", "cpu", "--work-dir", str(root / "sft/run")])
    latest = root / "sft/run/latest.pt"
    done = torch.load(latest, weights_only=False)
    manifest = json.loads((root / "data/manifest.json").read_text())
    dpo_plan = {"format": "warpstate-dpo-plan-v1", "stage": "dpo",
                "sft": {"step": done["step"], "tokens_seen": done["tokens_seen"], "tokenizer_sha256": digest(tok),
                        "train_rows": manifest["outputs"]["sft_train.jsonl"]["rows"], "assistant_tokens_seen": done["assistant_tokens_seen"],
                        "validation_rows": manifest["outputs"]["sft_val.jsonl"]["rows"], "raw_archive_sha256": done["signature"]["base_sha256"],
                        "base_step": 7, "base_tokens_seen": 700},
                "training": {"sequence_length": 64}, "handoff": {"data_manifest_sha256": digest(root / "data/manifest.json")}}
    paths = {"archive_dir": root / "archives/sft-final", "sft_work_dir": root / "sft", "tokenizer": tok}
    mine = H.DpoStage().make_archive(paths, dpo_plan, "rev")
    assert H.DpoStage().make_archive(paths, dpo_plan, "rev") == mine                     # a second call verifies, does not rewrite
    with reference_import_path():
        theirs = importlib.import_module("ops.dpo_handoff")
    two_ranks = theirs.validate_sft
    monkeypatch.setattr(theirs, "validate_sft", lambda checkpoint, *rest: two_ranks(
        dict(checkpoint, rng_by_rank=list(checkpoint["rng_by_rank"]) * 2), *rest))
    metadata, entries = theirs.verify_sft_archive(paths["archive_dir"], dpo_plan, sft_plan, expected_checkpoint_hash=digest(latest))
    assert metadata == mine and metadata["assistant_tokens_seen"] == done["assistant_tokens_seen"] and metadata["stage"] == "sft"
    assert tuple(entries) == A.SFT_ARCHIVE_FILES == tuple(theirs.ARCHIVE_FILES) and A.INIT_FILES == tuple(theirs.INIT_FILES)
    # and the three-file start of the next stage is what the reference's own copy routine would accept
    start = A.independent_copy(paths["archive_dir"], root / "dpo/initialization", H.DpoStage().boundary(dpo_plan), mine["snapshot_sha256"],
                               files=A.SFT_ARCHIVE_FILES, only=A.INIT_FILES)
    assert theirs.initialize_copy(paths["archive_dir"], root / "dpo/initialization", metadata) == start
    with pytest.raises(ValueError):
        theirs.verify_sft_archive(paths["archive_dir"], dict(dpo_plan, sft=dict(dpo_plan["sft"], step=done["step"] + 1)), sft_plan)
    # the reference's base -> SFT guardian accepts the run's completion records, and its trainer the resume state
    with reference_import_path():
        guardian = importlib.import_module("ops.posttrain_handoff")
        trainer = importlib.import_module("posttrain")
    completion = guardian.verify_completion(root / "sft/run", sft_plan, done["signature"]["base_sha256"])
    assert completion == H.SftStage().verify_completion(root / "sft/run", sft_plan, done["signature"]["base_sha256"])
    with pytest.raises(ValueError):
        guardian.verify_completion(root / "sft/run", sft_plan, "0" * 64)
    trainer.validate_resume(done, done["signature"], 1)
    with pytest.raises(ValueError):
        trainer.validate_resume(done, dict(done["signature"], world_size=2), 2)


def test_the_sealed_base_model_is_what_the_reference_guardian_expects(ref, tmp_path):
    """Pretraining with this trainer to its planned end, sealed by this framework's base -> SFT guardian; the reference's
    boundary check, archive verifier and initialization copy accept checkpoint and archive, and refuse them for another
    boundary."""
    from warpstate_ai_b200.data import prepare as P
    from warpstate_ai_b200.orchestration import archive as A
    from warpstate_ai_b200.orchestration import handoff as H
    from warpstate_ai_b200.train import pretrain as T
    from warpstate_ai_b200.utils.io import digest
    tok = tmp_path / "tokenizer.model"
    tok.write_bytes(TOK.read_bytes())
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(dict(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=8,
                                        gradient_checkpointing=False, parallel_memory=True)))
    base_dir = tmp_path / "base"
    P.write_synthetic_corpus(base_dir, tok, 73, 64, 32768, seed=2)
    T.STOP = False
    T.main(["--from-scratch", "--work-dir", str(base_dir), "--config", str(cfg_path), "--tokenizer", str(tok), "--stage", "train",
            "--device", "cpu", "--test-small-gpu", "--train-tokens", "73", "--val-tokens", "64", "--seq-len", "8", "--micro-batch", "2",
            "--grad-accum", "2", "--warmup-steps", "1", "--eval-batches", "1", "--no-activation-checkpointing",
            "--dataset", "synthetic/uniform", "--dataset-config", "none", "--revision", "0"])
    checkpoint = torch.load(base_dir / "run/latest.pt", weights_only=False)
    boundary = {"step": checkpoint["step"], "tokens_seen": checkpoint["tokens_seen"], "tokenizer_sha256": digest(tok)}
    with reference_import_path():
        theirs = importlib.import_module("ops.posttrain_handoff")
    theirs.validate_boundary(checkpoint, boundary, digest(tok))
    with pytest.raises(ValueError):
        theirs.validate_boundary(checkpoint, dict(boundary, step=boundary["step"] + 1), digest(tok))
    paths = {"base_work_dir": base_dir, "tokenizer": tok, "archive_dir": base_dir / "archives/final"}
    mine = H.SftStage().make_archive(paths, {"base": boundary}, "rev")
    assert theirs.verify_archive(paths["archive_dir"], boundary, mine["snapshot_sha256"]) == mine
    assert tuple(theirs.ARCHIVE_FILES) == A.ARCHIVE_FILES
    start = theirs.independent_initialization(paths["archive_dir"], tmp_path / "sft/initialization", boundary, mine["snapshot_sha256"])
    assert A.independent_copy(paths["archive_dir"], tmp_path / "sft/initialization", boundary, mine["snapshot_sha256"]) == start
    exported = torch.load(start, weights_only=False)
    assert all(torch.equal(exported["model"][k], v) for k, v in checkpoint["model"].items()) and "optimizer" not in exported
    with pytest.raises(ValueError):
        theirs.verify_archive(paths["archive_dir"], dict(boundary, tokens_seen=1))


# ------------------------------------------------------------------------------------------- the same run, both trainers
def metric_rows(path):
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    for row in rows:
        for key in [k for k in row if k == "timestamp" or "second" in k or k == "checkpoint"]:
            row.pop(key)
    return rows


def assert_same_course(mine, theirs, exact, close, rel):
    """Two metric logs tell the same story: the same events in the same order, counters and schedule exactly equal,
    measured values within the difference between FP32 and BF16-autocast arithmetic on the host."""
    assert [row["event"] for row in mine] == [row["event"] for row in theirs]
    for a, b in zip(mine, theirs):
        assert set(b) <= set(a), (set(b) - set(a), a["event"])
        for key in b:
            if key in close:
                assert a[key] == pytest.approx(b[key], rel=rel[key] if isinstance(rel, dict) else rel), (key, a, b)
            else:
                assert key in exact or isinstance(b[key], (str, bool, int)), key
                assert a[key] == b[key], (key, a, b)


@pytest.fixture
def host_settings():
    """The trainers set process-wide torch switches; a test that runs them in-process puts them back."""
    threads, deterministic = torch.get_num_threads(), torch.are_deterministic_algorithms_enabled()
    yield
    torch.set_num_threads(threads)
    torch.use_deterministic_algorithms(deterministic)


def test_the_same_sft_run_through_both_trainers(ref, tmp_path, monkeypatch, host_settings):
    """One model export, one prepared data directory, one plan (two epochs, warm-up, a last update that is not full):
    this framework's SFT trainer and the reference's, each on the host, log the same course of training, and end with the
    same weights.  (Prepared data names the hash of the renderer's source file, by design of both; the reference's copy
    of the directory differs in that one field.)"""
    import argparse
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.ckpt.formats import export_chat_snapshot
    from warpstate_ai_b200.data.prepare_posttrain import prepare
    from warpstate_ai_b200.train import sft as SFT
    from warpstate_ai_b200.utils.io import digest
    root = tmp_path / "ws"
    root.mkdir()
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(root))
    tok = root / "tokenizer.model"
    tok.write_bytes(TOK.read_bytes())
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=8,
                          gradient_checkpointing=False, parallel_memory=True)
    base = {"config": vars(cfg).copy(), "model": WarpStateLM(cfg).state_dict(), "step": 7, "tokens_seen": 700, "val_loss": 9.9}
    export_chat_snapshot(base, root / "base", tok, {"path": "test"})
    rows = [{"messages": [{"role": "user", "content": f"What is {i} plus {i + 1}?" + " please" * (i % 4)},
                          {"role": "assistant", "content": f"It is {2 * i + 1}." + " Indeed." * (i % 3)}]} for i in range(23)]
    prepare(root / "data", tok, 64, sft_rows=rows, val_modulus=5)
    plan = {"format": "warpstate-posttrain-plan-v1", "stage": "sft", "base": {"step": 7, "tokens_seen": 700, "tokenizer_sha256": digest(tok)},
            "training": {"sequence_length": 64, "micro_batch": 2, "grad_accum": 2, "lr": 1e-3, "min_lr": 1e-4, "warmup_ratio": 0.25,
                         "epochs": 2, "eval_every": 2, "save_every": 3, "eval_batches": 1, "workers": 1, "weight_decay": 0.05,
                         "compile_core": False, "loss_mode": "full", "bf16_residuals": False}}
    (root / "plan.json").write_text(json.dumps(plan))
    monkeypatch.setattr(SFT, "STOP", False)
    SFT.main(["--config", str(root / "plan.json"), "--data-dir", str(root / "data"), "--weights", str(root / "base/model.pt"),
              "--tokenizer", str(tok), "--device", "cpu", "--work-dir", str(root / "mine/run")])
    theirs = ref["posttrain"]
    data = root / "their-data"
    data.mkdir()
    for file in (root / "data").iterdir():
        (data / file.name).write_bytes(file.read_bytes())
    with reference_import_path():
        manifest = json.loads((data / "manifest.json").read_text())
        manifest["renderer_sha256"] = importlib.import_module("ops.posttrain_data").renderer_sha256()
        (data / "manifest.json").write_text(json.dumps(manifest))
        monkeypatch.setattr(theirs, "WORKSPACE", root)
        monkeypatch.setattr(theirs, "STOP", False)
        theirs.train(argparse.Namespace(config=root / "plan.json", work_dir=root / "theirs/run", data_dir=data,
                                        weights=root / "base/model.pt", tokenizer=tok, max_steps=None, stop_file=None, device="cpu"))
    a, b = metric_rows(root / "mine/run/metrics.jsonl"), metric_rows(root / "theirs/run/metrics.jsonl")
    assert sum(row["event"] == "train" for row in b) >= 8 and {row.get("update_samples") for row in b} >= {4, 1}
    assert_same_course(a, b, exact={"lr"}, close={"loss", "val_loss", "val_perplexity", "grad_norm"},
                       rel={"loss": 1e-4, "val_loss": 1e-4, "val_perplexity": 2e-3, "grad_norm": 2e-2})
    mine_end, their_end = (torch.load(root / side / "run/latest.pt", weights_only=False) for side in ("mine", "theirs"))
    for key in ("step", "sample_cursor", "tokens_seen", "assistant_tokens_seen", "completed", "total_steps", "val_step", "format"):
        assert mine_end[key] == their_end[key], key
    assert mine_end["val_loss"] == pytest.approx(their_end["val_loss"], rel=1e-4)
    # Adam divides by the gradient's own magnitude, so where a gradient is rounding noise (vocabulary rows that no
    # example touches) the two arithmetics may step in different directions; judged against how far training moved them
    for name, tensor in their_end["model"].items():
        moved = (tensor - base["model"][name]).abs().mean()
        apart = (mine_end["model"][name] - tensor).abs().mean()
        assert moved > 1e-3 and apart < 0.01 * moved, (name, float(moved), float(apart))
    for name in ("completion.json", "evaluation.json", "settings.json"):
        x, y = (json.loads((root / side / "run" / name).read_text()) for side in ("mine", "theirs"))
        assert set(y) <= set(x), (name, set(y) - set(x))
    done = [json.loads((root / side / "run/completion.json").read_text()) for side in ("mine", "theirs")]
    for key in ("format", "stage", "completed", "paused_for_evaluation", "step", "total_steps", "base_step", "tokens_seen", "assistant_tokens_seen"):
        assert done[0][key] == done[1][key], key


def test_the_same_dpo_run_through_both_trainers(ref, tmp_path, monkeypatch, host_settings):
    """One SFT export, one directory of preference pairs, one plan: both DPO trainers on the host score the frozen
    reference model alike (the cache files hold the same numbers), then log the same course of training: the same pairs
    per update (updates of three pairs included), the same schedule and counters, objective values within BF16 noise."""
    import argparse
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.ckpt.formats import export_chat_snapshot
    from warpstate_ai_b200.data.prepare_posttrain import prepare
    from warpstate_ai_b200.train import dpo as DPO
    from warpstate_ai_b200.utils.io import digest
    root = tmp_path / "ws"
    root.mkdir()
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(root))
    tok = root / "tokenizer.model"
    tok.write_bytes(TOK.read_bytes())
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=8,
                          gradient_checkpointing=False, parallel_memory=True)
    model = WarpStateLM(cfg)
    with torch.no_grad():
        model.embed.weight.normal_(0, 0.3)
    sft = {"config": vars(cfg).copy(), "model": model.state_dict(), "step": 4, "tokens_seen": 400, "assistant_tokens_seen": 90,
           "val_loss": 9.0, "origin": {"step": 7, "tokens_seen": 700}}
    export_chat_snapshot(sft, root / "sft-export", tok, {"path": "test"}, stage="sft")
    pairs = [{"prompt": [{"role": "user", "content": f"What follows {i}?" + " now" * (i % 3)}],
              "chosen": [{"role": "assistant", "content": str(i + 1)}],
              "rejected": [{"role": "assistant", "content": f"maybe {i + 3} or so" + " hm" * (i % 4)}]} for i in range(23)]
    prepare(root / "data", tok, 64, dpo_rows=pairs, val_modulus=5)
    plan = {"format": "warpstate-dpo-plan-v1", "stage": "dpo",
            "sft": {"step": 4, "tokens_seen": 400, "base_step": 7, "base_tokens_seen": 700, "tokenizer_sha256": digest(tok)},
            "training": {"sequence_length": 64, "micro_batch": 2, "grad_accum": 2, "lr": 1e-3, "min_lr": 1e-4, "warmup_ratio": 0.25,
                         "epochs": 2, "eval_every": 2, "save_every": 3, "eval_batches": 1, "workers": 1, "beta": 0.5,
                         "head_chunk_size": 16, "compile_core": False, "bf16_residuals": False}}
    (root / "plan.json").write_text(json.dumps(plan))
    monkeypatch.setattr(DPO, "STOP", False)
    DPO.main(["--config", str(root / "plan.json"), "--data-dir", str(root / "data"), "--weights", str(root / "sft-export/model.pt"),
              "--tokenizer", str(tok), "--device", "cpu", "--reference-cache-dir", str(root / "mine/reference-cache"),
              "--work-dir", str(root / "mine/run")])
    theirs = ref["dpo"]
    data = root / "their-data"
    data.mkdir()
    for file in (root / "data").iterdir():
        (data / file.name).write_bytes(file.read_bytes())
    (root / "theirs/reference-cache").mkdir(parents=True)
    with reference_import_path():
        manifest = json.loads((data / "manifest.json").read_text())
        manifest["renderer_sha256"] = importlib.import_module("ops.posttrain_data").renderer_sha256()
        (data / "manifest.json").write_text(json.dumps(manifest))
        for module in (theirs, ref["posttrain"]):
            monkeypatch.setattr(module, "WORKSPACE", root)
            monkeypatch.setattr(module, "STOP", False)
        theirs.train(argparse.Namespace(config=root / "plan.json", work_dir=root / "theirs/run", data_dir=data,
                                        weights=root / "sft-export/model.pt", tokenizer=tok, max_steps=None, stop_file=root / "theirs/stop",
                                        device="cpu", reference_cache_dir=root / "theirs/reference-cache", reference_only=False))
    for name in ("train.npy", "val.npy"):
        x, y = (np.load(root / side / "reference-cache" / name) for side in ("mine", "theirs"))
        assert x.shape == y.shape and x.dtype == y.dtype and np.allclose(x, y, rtol=1e-3, atol=5e-2), name
    a, b = metric_rows(root / "mine/run/metrics.jsonl"), metric_rows(root / "theirs/run/metrics.jsonl")
    assert sum(row["event"] == "train" for row in b) == 8 and {row.get("update_samples") for row in b} >= {4, 3}
    measured = {"loss": 3e-3, "val_loss": 3e-3, "chosen_nll": 1e-3, "grad_norm": 2e-2}
    for row in a + b:                                           # margins start at zero: an absolute bound for them, below
        row["margin"] = row.pop("reward_margin", None)
    assert_same_course([{k: v for k, v in row.items() if k != "margin"} for row in a],
                       [{k: v for k, v in row.items() if k != "margin"} for row in b], exact={"lr", "reward_accuracy"},
                       close=set(measured), rel=measured)
    for x, y in zip(a, b):
        assert (x["margin"] is None) == (y["margin"] is None)
        assert x["margin"] is None or abs(x["margin"] - y["margin"]) < 3e-3
    assert b[-2]["margin"] > 0.05 and b[-2]["val_loss"] < 0.66          # the run did learn the preference
    mine_end, their_end = (torch.load(root / side / "run/latest.pt", weights_only=False) for side in ("mine", "theirs"))
    for key in ("step", "sample_cursor", "tokens_seen", "response_tokens_seen", "completed", "total_steps", "format"):
        assert mine_end[key] == their_end[key], key
    for name, tensor in their_end["model"].items():
        moved = (tensor - sft["model"][name]).abs().mean()
        apart = (mine_end["model"][name] - tensor).abs().mean()
        assert moved > 1e-3 and apart < 0.05 * moved, (name, float(moved), float(apart))
    for name in ("completion.json", "evaluation.json", "settings.json"):
        x, y = (json.loads((root / side / "run" / name).read_text()) for side in ("mine", "theirs"))
        assert set(y) <= set(x), (name, set(y) - set(x))


# ------------------------------------------------------------------------------------------- locks
def test_locks_of_either_implementation_exclude_the_other(ref, tmp_path, monkeypatch):
    """A mixed installation stays safe: the pretraining lock and the shared pipeline lock are the same advisory locks on
    the same files, so a job of one implementation keeps out a job of the other."""
    from warpstate_ai_b200.train import stage as S
    from warpstate_ai_b200.utils.io import LockHeld, process_lock
    with reference_import_path():
        their_lock = importlib.import_module("run_40b").process_lock
    theirs = ref["posttrain"]
    monkeypatch.setattr(theirs, "WORKSPACE", tmp_path.resolve())
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(tmp_path))
    base = tmp_path / "base"
    base.mkdir()
    lock = base / "pipeline.lock"
    plan = {"handoff": {"base_work_dir": "base"}}
    with process_lock(lock):                                     # pretraining of this framework runs
        with pytest.raises(BlockingIOError):
            with their_lock(lock):
                pass
        with pytest.raises(RuntimeError):
            with theirs.base_pipeline_lock(plan):
                pass
    with their_lock(lock):                                       # the reference's pretraining runs
        with pytest.raises(LockHeld):
            with process_lock(lock):
                pass
        with pytest.raises(RuntimeError):
            with S.base_pipeline_lock(plan):
                pass
    with theirs.base_pipeline_lock(plan), S.base_pipeline_lock(plan):      # post-training ranks of both share it
        with pytest.raises(LockHeld):
            with process_lock(lock):
                pass
        with pytest.raises(BlockingIOError):
            with their_lock(lock):
                pass
    with process_lock(lock), pytest.raises(LockHeld):
        with process_lock(lock):
            pass
    for bad in ({"handoff": {"base_work_dir": "missing"}}, {"handoff": {"base_work_dir": "../outside"}}, {"handoff": {"base_work_dir": "."}}):
        for implementation in (theirs.base_pipeline_lock, S.base_pipeline_lock):
            with pytest.raises(ValueError):
                with implementation(bad):
                    pass
    for implementation in (theirs.base_pipeline_lock, S.base_pipeline_lock):
        with implementation({}):                                 # no base job named: nothing to hold
            pass


# ------------------------------------------------------------------------------------------- guardians: is the data ready?
def test_both_guardians_judge_prepared_data_alike(ref, tmp_path):
    """Data prepared here, shown to the readiness checks of the reference's two guardians and of this framework's: ready,
    verified, and -- after each kind of damage -- the same answer (not yet ready) or the same refusal."""
    from warpstate_ai_b200.data.prepare_posttrain import prepare
    from warpstate_ai_b200.orchestration import handoff as H
    from warpstate_ai_b200.utils.io import digest
    with reference_import_path():
        their = {"sft": importlib.import_module("ops.posttrain_handoff").data_readiness,
                 "dpo": importlib.import_module("ops.dpo_handoff").data_readiness}
    sft_rows = [{"messages": [{"role": "user", "content": f"Q{i}"}, {"role": "assistant", "content": f"A{i}"}]} for i in range(9)]
    dpo_rows = [{"prompt": [{"role": "user", "content": f"Q{i}"}], "chosen": [{"role": "assistant", "content": "yes"}],
                 "rejected": [{"role": "assistant", "content": "no, not at all"}]} for i in range(9)]

    def fresh(name):
        folder = tmp_path / name
        prepare(folder, TOK, 64, sft_rows=sft_rows, dpo_rows=dpo_rows, val_modulus=4)
        return folder

    def plans(folder, **training):
        settings = dict({"sequence_length": 64}, **training)
        tokenizer = digest(TOK)
        return {"sft": {"base": {"tokenizer_sha256": tokenizer}, "training": settings, "handoff": {}},
                "dpo": {"sft": {"tokenizer_sha256": tokenizer}, "training": settings,
                        "handoff": {"data_manifest_sha256": digest(folder / "manifest.json") if (folder / "manifest.json").is_file() else "-"}}}

    def verdicts(folder, plan_of, verify):
        out = {}
        for stage in ("sft", "dpo"):
            for side, check in (("theirs", lambda: their[stage](folder, plan_of[stage], verify=verify)),
                                ("mine", lambda: H.data_readiness(folder, plan_of[stage], H.STAGES[stage], verify=verify))):
                try:
                    answer = check()
                    out[stage, side] = bool(answer[0] if isinstance(answer, tuple) else answer)
                except ValueError:
                    out[stage, side] = "refused"
        return out

    good = fresh("good")
    for verify in (False, True):
        assert set(verdicts(good, plans(good), verify).values()) == {True}
    assert set(verdicts(good, plans(good, sequence_length=128), False).values()) == {"refused"}      # another context length
    other_tokenizer = plans(good)
    other_tokenizer["sft"]["base"]["tokenizer_sha256"] = other_tokenizer["dpo"]["sft"]["tokenizer_sha256"] = "0" * 64
    assert set(verdicts(good, other_tokenizer, False).values()) == {"refused"}
    missing = tmp_path / "nothing-yet"
    missing.mkdir()
    assert set(verdicts(missing, plans(missing), False).values()) == {False}
    partial = fresh("partial")
    manifest = json.loads((partial / "manifest.json").read_text())
    (partial / "manifest.json").write_text(json.dumps(dict(manifest, complete=False)))
    assert set(verdicts(partial, plans(partial), False).values()) == {False}
    for name in ("sft_val.jsonl", "dpo_train.jsonl"):
        stage = name[:3]
        gone = fresh(f"gone-{stage}")
        plan_of = plans(gone)
        (gone / name).unlink()
        found = verdicts(gone, plan_of, False)
        assert found[stage, "theirs"] == found[stage, "mine"] == "refused"
        edited = fresh(f"edited-{stage}")
        plan_of = plans(edited)
        with (edited / name).open("a") as stream:
            stream.write("\n")
        assert verdicts(edited, plan_of, False)[stage, "mine"] is True and verdicts(edited, plan_of, False)[stage, "theirs"] is True
        found = verdicts(edited, plan_of, True)                                                     # only hashing sees it
        assert found[stage, "theirs"] == found[stage, "mine"] == "refused"
    repinned = fresh("repinned")
    plan_of = plans(repinned)
    (repinned / "manifest.json").write_text((repinned / "manifest.json").read_text() + "\n")         # the DPO plan pins the manifest
    found = verdicts(repinned, plan_of, False)
    assert found["dpo", "theirs"] == found["dpo", "mine"] == "refused" and found["sft", "theirs"] is found["sft", "mine"] is True


# ------------------------------------------------------------------------------------------- guardians: directory layout rules
def test_guardian_plans_are_accepted_and_refused_alike(tmp_path, monkeypatch):
    """Directory layouts of a hand-off plan through both guardians' plan loaders.  Both keep the stage's outputs apart from the
    base run, the archives, the parent run and the data, and check the SFT parent named by a DPO plan.  Two conventions of the
    reference are not imposed here and are listed as such: DPO output below ``<base>/posttrain`` with its archive below
    ``<base>/archives``, and a polling interval of at least a second."""
    import sys
    from warpstate_ai_b200.orchestration import handoff as H
    if not (REF / "ops" / "dpo_handoff.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    root = tmp_path.resolve()
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(root))
    with reference_import_path():
        loaders = {"sft": importlib.import_module("ops.posttrain_handoff"), "dpo": importlib.import_module("ops.dpo_handoff")}
        modules = [*loaders.values(), importlib.import_module("ops.launch_training"), sys.modules["launch_training"]]
    for module in modules:
        monkeypatch.setattr(module, "WORKSPACE", root)
    parent = {"step": 7, "tokens_seen": 700, "tokenizer_sha256": "t"}
    documents = {"sft": {"format": "warpstate-posttrain-plan-v1", "stage": "sft", "after_completion": "pause_for_evaluation", "base": parent},
                 "dpo": {"format": "warpstate-dpo-plan-v1", "stage": "dpo", "after_completion": "pause_for_evaluation",
                         "sft": {"base_step": 7, "base_tokens_seen": 700, "tokenizer_sha256": "t", "step": 4, "tokens_seen": 400}}}
    (root / "sft-plan.json").write_text(json.dumps(documents["sft"]))
    common = {"base_work_dir": "work", "supervisor_socket": "run/s.sock", "data_dir": "work/posttrain/data", "tokenizer": "tokenizer.model",
              "processes": 2, "poll_seconds": 5}
    layouts = {"sft": dict(common, archive_dir="work/archives/a", work_dir="work/posttrain/sft"),
               "dpo": dict(common, sft_work_dir="work/posttrain/sft", sft_plan="sft-plan.json", archive_dir="work/archives/sft-final",
                           work_dir="work/posttrain/dpo")}
    cases = {"sft": [{}, {"work_dir": "work"}, {"work_dir": "work/run/x"}, {"work_dir": "work/archives/x"}, {"work_dir": "work/archives/a/x"},
                     {"archive_dir": "work/posttrain/sft/arch"}, {"data_dir": "work/posttrain/sft/data"}, {"work_dir": "work/posttrain/data/run"},
                     {"work_dir": "elsewhere/sft"}, {"work_dir": "../outside"}, {"poll_seconds": 61}, {"poll_seconds": 0}],
             "dpo": [{}, {"work_dir": "work"}, {"work_dir": "work/posttrain"}, {"work_dir": "work/posttrain/sft/dpo"}, {"work_dir": "work/posttrain/data/dpo"},
                     {"work_dir": "work/run/dpo"}, {"work_dir": "work/archives/dpo"}, {"archive_dir": "work/posttrain/dpo/archive"},
                     {"sft_work_dir": "work/posttrain/dpo/sft"}, {"data_dir": "work/posttrain/dpo/data"}, {"poll_seconds": 0},
                     {"work_dir": "work/posttrain/dpo/../sft"}, {"sft": {"base_step": 8}}, {"sft": {"base_tokens_seen": 1}}, {"sft": {"tokenizer_sha256": "u"}}]}
    conventions = {"sft": [{"poll_seconds": 0.5}], "dpo": [{"work_dir": "elsewhere/dpo"}, {"archive_dir": "work/archives"}, {"archive_dir": "elsewhere/archive"}]}

    def verdicts(stage, change):
        document = dict(documents[stage], handoff=dict(layouts[stage], **{k: v for k, v in change.items() if k != "sft"}))
        if "sft" in change:
            document["sft"] = dict(document["sft"], **change["sft"])
        path = root / "plan.json"
        path.write_text(json.dumps(document))
        found = []
        for load in (lambda: H.load_plan(path, H.STAGES[stage]), lambda: loaders[stage].load_plan(path)):
            try:
                found.append({key: str(value) for key, value in load()[1].items() if key != "sft_plan"})
            except ValueError:
                found.append("refused")
        return found

    for stage in ("sft", "dpo"):
        for change in cases[stage]:
            mine, theirs = verdicts(stage, change)
            assert mine == theirs, (stage, change)
        assert verdicts(stage, {})[0] != "refused"
        for change in conventions[stage]:
            mine, theirs = verdicts(stage, change)
            assert mine != "refused" and theirs == "refused", (stage, change)
