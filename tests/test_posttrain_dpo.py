"""SFT and DPO end to end on CPU with a tiny model and the real tokenizer, plus unit checks of
the objective pieces (reference test_posttrain.py:77-111, test_dpo.py:52-113).
"""
import json
import math
import os
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
from warpstate_ai_b200.ckpt.formats import export_chat_snapshot
from warpstate_ai_b200.data import dpo as DD
from warpstate_ai_b200.data import sft as SD
from warpstate_ai_b200.data.prepare_posttrain import prepare
from warpstate_ai_b200.train import dpo as DPO
from warpstate_ai_b200.train import sft as SFT

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def sp():
    import sentencepiece as spm
    return spm.SentencePieceProcessor(model_file=str(ROOT / "tokenizer.model"))


def conversations(n):
    rows = []
    for i in range(n):
        rows.append({"messages": [{"role": "system", "content": "You are terse."},
                                  {"role": "user", "content": f"What is {i} plus {i + 1}?"},
                                  {"role": "assistant", "content": f"It is {2 * i + 1}."}]})
    return rows


def pairs(n):
    return [{"prompt": [{"role": "user", "content": f"Say the number {i}."}],
             "chosen": [{"role": "assistant", "content": f"{i}"}],
             "rejected": [{"role": "assistant", "content": f"I will not say {i + 7} today."}]} for i in range(n)]


def test_renderer_masks_everything_but_assistant(sp):
    enc = SD.encode_messages(conversations(1)[0]["messages"], sp)
    ids, labels = enc["input_ids"], enc["labels"]
    assert ids[0] == sp.bos_id() and labels[0] == -100
    supervised = [t for t, l in zip(ids, labels) if l != -100]
    assert supervised[-1] == sp.eos_id()
    assert sp.decode(supervised[:-1]) == "It is 1."
    with pytest.raises(ValueError):
        SD.encode_messages([{"role": "user", "content": "only a question"}], sp)
    with pytest.raises(ValueError):
        SD.encode_messages(conversations(1)[0]["messages"], sp, max_length=5)


def test_collate_and_update_indices():
    rec = {"input_ids": [1, 5, 6, 7], "labels": [-100, -100, 6, 7]}
    x, y = SD.collate([rec, None], 6, 0)
    assert x.tolist() == [[1, 5, 6, 0, 0, 0], [0] * 6]
    assert y.tolist() == [[-100, 6, 7, -100, -100, -100], [-100] * 6]
    seen, cursor = [], 0
    while True:
        idx, cursor = SD.update_indices(10, 3, cursor, 2, 4)
        if not idx:
            break
        seen.append(idx)
    assert [len(b) for b in seen] == [4, 4, 2, 4, 4, 2]  # never crosses an epoch
    assert sorted(sum(seen[:3], [])) == list(range(10)) and sorted(sum(seen[3:], [])) == list(range(10))
    assert seen[:3] != seen[3:]


def test_token_weighting_with_an_empty_rank():
    # two "ranks": one with 3 targets, one with none; the weighted sum equals the global token mean
    losses = [torch.tensor(2.0), torch.tensor(0.0)]
    targets = [3, 0]
    total = sum(SFT.token_weighted_loss(l, t, 3, 2) for l, t in zip(losses, targets)) / 2
    assert float(total) == pytest.approx(2.0)
    with pytest.raises(ValueError):
        SFT.token_weighted_loss(torch.tensor(1.0), 0, 0, 1)


def test_preference_metrics_match_the_formula():
    policy = torch.tensor([[-10.0, -14.0], [-9.0, -3.0]], requires_grad=True)
    ref = torch.tensor([[-11.0, -12.0], [-8.0, -4.0]])
    counts = torch.tensor([[5, 7], [3, 2]])
    loss, margin, acc = DPO.preference_metrics(policy, ref, counts, 0.5, "length-normalized-dpo")
    want = 0.5 * ((policy.detach() - ref) / counts)
    assert torch.allclose(margin, want[:, 0] - want[:, 1])
    assert torch.allclose(loss, -F.logsigmoid(margin))
    assert acc.tolist() == [float(m > 0) for m in margin.tolist()]
    loss2, margin2, _ = DPO.preference_metrics(policy, ref, counts, 0.5, "summed-dpo")
    assert torch.allclose(margin2, 0.5 * ((policy.detach() - ref)[:, 0] - (policy.detach() - ref)[:, 1]))
    zero, _, _ = DPO.preference_metrics(ref.clone(), ref, counts, 5.0, "length-normalized-dpo")
    assert torch.allclose(zero, torch.full((2,), math.log(2.0)))


def test_sequence_logps_equal_full_logits():
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=61, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24, chunk_size=4,
                          gradient_checkpointing=False, parallel_memory=True)
    model = WarpStateLM(cfg)
    x = torch.randint(0, 61, (3, 12))
    y = torch.randint(0, 61, (3, 12))
    y[:, :5] = -100
    got = model.sequence_logps(x, y, head_chunk_size=4)
    got.sum().backward()
    grads = [p.grad.clone() for p in model.parameters()]
    model.zero_grad()
    logits = model(x)
    want = -F.cross_entropy(logits.reshape(-1, 61), y.reshape(-1), reduction="none", ignore_index=-100).view(3, 12).sum(1)
    want.sum().backward()
    assert torch.allclose(got, want, rtol=1e-6, atol=1e-5)
    for a, p in zip(grads, model.parameters()):
        assert torch.allclose(a, p.grad, rtol=1e-5, atol=2e-6)


@pytest.fixture()
def workspace(tmp_path, monkeypatch):
    root = tmp_path / "ws"
    root.mkdir()
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(root))
    tok = root / "tokenizer.model"
    tok.write_bytes((ROOT / "tokenizer.model").read_bytes())
    return root, tok


def make_base_export(root, tok, stage=None, state=None, name="base"):
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24,
                          chunk_size=8, gradient_checkpointing=False, parallel_memory=True)
    model = WarpStateLM(cfg)
    ckpt = {"config": vars(cfg).copy(), "model": state or model.state_dict(), "step": 7, "tokens_seen": 700,
            "val_loss": 9.9, "origin": {"step": 7, "tokens_seen": 700}}
    export_chat_snapshot(ckpt, root / name, tok, {"path": "test"}, stage=stage)
    return root / name / "model.pt"


def test_sft_then_dpo_pipeline(workspace, monkeypatch):
    root, tok = workspace
    monkeypatch.setattr(SFT, "STOP", False)
    monkeypatch.setattr(DPO, "STOP", False)
    base = make_base_export(root, tok)
    data = root / "data"
    prepare(data, tok, 64, sft_rows=conversations(24), dpo_rows=pairs(24), val_modulus=5)
    plan = root / "plans" / "sft.json"
    plan.parent.mkdir()
    plan.write_text(json.dumps({"format": "warpstate-posttrain-plan-v1", "stage": "sft", "base": {"step": 7},
                                "training": {"sequence_length": 64, "micro_batch": 2, "grad_accum": 2, "lr": 1e-3,
                                             "eval_every": 2, "save_every": 2, "eval_batches": 2, "workers": 1,
                                             "max_steps": 4}}))
    common = ["--config", str(plan), "--data-dir", str(data), "--weights", str(base), "--tokenizer", str(tok),
              "--device", "cpu"]
    SFT.main(common + ["--work-dir", str(root / "sft-a")])
    done = torch.load(root / "sft-a/latest.pt", weights_only=False)
    assert done["format"] == "warpstate-posttrain-v1" and done["step"] == 4 and done["completed"] is True
    assert json.loads((root / "sft-a/completion.json").read_text())["completed"] is True
    events = [json.loads(l) for l in (root / "sft-a/metrics.jsonl").read_text().splitlines()]
    assert events[0]["event"] == "validation" and events[0]["full_holdout"] is True
    train_events = [e for e in events if e["event"] == "train"]
    assert len(train_events) == 4 and train_events[-1]["loss"] < train_events[0]["loss"]
    # split + resume is bitwise identical
    SFT.main(common + ["--work-dir", str(root / "sft-b"), "--max-steps", "1"])
    assert torch.load(root / "sft-b/latest.pt", weights_only=False)["step"] == 1
    SFT.main(common + ["--work-dir", str(root / "sft-b")])
    again = torch.load(root / "sft-b/latest.pt", weights_only=False)
    for k in done["model"]:
        assert torch.equal(done["model"][k], again["model"][k]), k
    assert again["sample_cursor"] == done["sample_cursor"] and again["assistant_tokens_seen"] == done["assistant_tokens_seen"]
    # ---- DPO from the SFT result
    sft_export = make_base_export(root, tok, stage="sft", state=done["model"], name="sft-export")
    dplan = root / "plans" / "dpo.json"
    dplan.write_text(json.dumps({"format": "warpstate-dpo-plan-v1", "stage": "dpo",
                                 "training": {"sequence_length": 64, "micro_batch": 2, "grad_accum": 2, "lr": 1e-3,
                                              "eval_every": 2, "save_every": 2, "eval_batches": 2, "workers": 1,
                                              "max_steps": 3, "beta": 0.5, "head_chunk_size": 16}}))
    dcommon = ["--config", str(dplan), "--data-dir", str(data), "--weights", str(sft_export), "--tokenizer", str(tok),
               "--device", "cpu", "--reference-cache-dir", str(root / "ref-cache")]
    DPO.main(dcommon + ["--work-dir", str(root / "dpo-a")])
    devents = [json.loads(l) for l in (root / "dpo-a/metrics.jsonl").read_text().splitlines()]
    assert devents[0]["event"] == "validation" and devents[0]["val_loss"] == pytest.approx(math.log(2), abs=1e-6)
    dtrain = [e for e in devents if e["event"] == "train"]
    assert len(dtrain) == 3 and {"loss", "reward_margin", "reward_accuracy", "chosen_nll"} <= set(dtrain[0])
    assert dtrain[0]["loss"] == pytest.approx(math.log(2), abs=1e-5)
    final = torch.load(root / "dpo-a/latest.pt", weights_only=False)
    assert final["format"] == "warpstate-dpo-v1" and final["step"] == 3
    assert (root / "ref-cache/train.npy").exists() and (root / "ref-cache/manifest.json").exists()
    # resident reference gives the same first-step numbers as the cached reference
    rplan = root / "plans" / "dpo-resident.json"
    cfgd = json.loads(dplan.read_text())
    cfgd["training"]["reference_mode"] = "resident"
    cfgd["training"]["max_steps"] = 1
    rplan.write_text(json.dumps(cfgd))
    rcommon = list(dcommon)
    rcommon[1] = str(rplan)
    rcommon[rcommon.index("--reference-cache-dir") + 1] = str(root / "ref-cache-2")
    DPO.main(rcommon + ["--work-dir", str(root / "dpo-r")])
    revents = [json.loads(l) for l in (root / "dpo-r/metrics.jsonl").read_text().splitlines() if '"train"' in l]
    assert revents[0]["loss"] == pytest.approx(dtrain[0]["loss"], rel=1e-5)
    assert revents[0]["grad_norm"] == pytest.approx(dtrain[0]["grad_norm"], rel=1e-4)


def test_path_rules(workspace):
    root, tok = workspace
    base = make_base_export(root, tok)
    (root / "data").mkdir()
    plan = root / "plan.json"
    plan.write_text("{}")
    with pytest.raises(ValueError, match="must not be inside data"):
        SFT.validate_paths(root / "data" / "out", root / "data", base, tok, plan)
    with pytest.raises(ValueError, match="inside"):
        SFT.validate_paths("/tmp/elsewhere", root / "data", base, tok, plan)
    SFT.validate_paths(root / "out", root / "data", base, tok, plan)


def test_evaluate_snapshot_on_full_holdout(workspace):
    from warpstate_ai_b200.train import evaluate_snapshot as ES
    root, tok = workspace
    export = make_base_export(root, tok, stage="sft", name="sealed")
    (root / "sealed/tokenizer.model").write_bytes(tok.read_bytes())
    data = root / "evaldata"
    prepare(data, tok, 64, sft_rows=conversations(17), val_modulus=3)
    out = root / "reports/eval.json"
    assert ES.main(["--snapshot", str(export), "--data-dir", str(data), "--device", "cpu", "--output", str(out)]) == 0
    report = json.loads(out.read_text())
    manifest = json.loads((data / "manifest.json").read_text())
    assert report["full_holdout"] is True and report["evaluated_samples"] == manifest["outputs"]["sft_val.jsonl"]["rows"]
    assert report["assistant_target_tokens"] == manifest["outputs"]["sft_val.jsonl"]["supervised_tokens"]
    assert report["val_perplexity"] == pytest.approx(math.exp(report["val_loss"])) and 5 < report["val_loss"] < 12
    with pytest.raises(ValueError, match="new report"):
        ES.run(export, data, out, torch.device("cpu"))
    with pytest.raises(ValueError, match="new report"):
        ES.run(export, data, data / "inside.json", torch.device("cpu"))


@pytest.mark.gpu
def test_bf16_reference_copy_scores_through_the_fused_path():
    """A frozen BF16 copy of the policy (the resident DPO reference) runs the same fused forward
    and gives the policy's sequence log-probabilities up to BF16 rounding of the parameters."""
    import copy
    torch.manual_seed(0)
    cfg = WarpStateConfig(vocab_size=1024, d_model=256, n_heads=4, n_cores=2, logical_depth=2, ffn_hidden=512,
                          chunk_size=128, gradient_checkpointing=False, parallel_memory=True)
    policy = WarpStateLM(cfg).cuda().eval()
    frozen = copy.deepcopy(policy).to(torch.bfloat16).requires_grad_(False)
    x = torch.randint(0, 1024, (4, 256), device="cuda")
    y = torch.randint(0, 1024, (4, 256), device="cuda")
    y[:, :100] = -100
    with torch.no_grad():
        a = DPO.score_pairs(policy, x, y, torch.device("cuda"), 64)
        b = DPO.score_pairs(frozen, x, y, torch.device("cuda"), 64)
    assert torch.isfinite(b).all()
    assert torch.allclose(a, b, rtol=0.02, atol=0.5), (a, b)
