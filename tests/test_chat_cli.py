"""Snapshot capture / verification and generation through the chat entry points (CPU)."""
import json
from pathlib import Path

import pytest
import torch

from warpstate_ai_b200.data import prepare as P
from warpstate_ai_b200.serve import chat as C
from warpstate_ai_b200.serve import posttrain_chat as PC
from warpstate_ai_b200.serve.engine import DecodeEngine
from warpstate_ai_b200.train import pretrain as T

ROOT = Path(__file__).resolve().parents[1]
TOK = ROOT / "tokenizer.model"


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("chat")
    cfg = tmp / "cfg.json"
    cfg.write_text(json.dumps(dict(vocab_size=32768, d_model=16, n_heads=2, n_cores=1, logical_depth=2, ffn_hidden=24,
                                   chunk_size=4, gradient_checkpointing=False, parallel_memory=True)))
    work = tmp / "work"
    P.write_synthetic_corpus(work, TOK, 73, 64, 32768, seed=1)
    T.STOP = False
    T.main(["--from-scratch", "--work-dir", str(work), "--config", str(cfg), "--tokenizer", str(TOK), "--stage", "train",
            "--device", "cpu", "--test-small-gpu", "--train-tokens", "73", "--val-tokens", "64", "--seq-len", "8",
            "--micro-batch", "2", "--grad-accum", "2", "--warmup-steps", "1", "--max-steps", "1", "--eval-batches", "1",
            "--no-activation-checkpointing", "--dataset", "synthetic/uniform", "--dataset-config", "none",
            "--revision", "0"])
    return tmp, work


def test_capture_verify_generate(trained, capsys):
    tmp, work = trained
    snapshot = C.capture_latest(work / "run/latest.pt", TOK, tmp / "snaps")
    meta = json.loads(snapshot.with_name("snapshot.json").read_text())
    assert meta["format"] == "warpstate-chat-v1" and meta["step"] == 1 and "snapshot_sha256" in meta
    assert oct(snapshot.stat().st_mode & 0o777) == "0o444"
    assert C.resolve_snapshot(snapshot, TOK, tmp / "snaps") == snapshot
    model, sp, metadata = C.load_model(snapshot, TOK)
    assert metadata["inference_only"] is True and "model" not in metadata
    a = list(C.generate(model, sp, "Hello there", max_new_tokens=6, temperature=0.0, max_context=64))
    b = list(C.generate(model, sp, "Hello there", max_new_tokens=6, temperature=0.0, max_context=64))
    assert a == b and 1 <= len(a) <= 6
    # token-by-token reference path gives the same greedy continuation
    ids = sp.encode("Hello there", out_type=int)
    caches = model.init_generation_cache(1, torch.device("cpu"), torch.float32)
    with torch.no_grad():
        for t in ids:
            logits = model.step(torch.tensor([[t]]), caches)[0, -1]
    assert int(logits.argmax()) == a[0]
    C.main(["--snapshot", str(snapshot), "--tokenizer", str(TOK), "--prompt", "Hi", "--max-new-tokens", "4",
            "--max-context", "64", "--temperature", "0"])
    assert "tokens" in capsys.readouterr().out
    # tampering is detected
    bad = tmp / "bad"
    bad.mkdir()
    (bad / "model.pt").write_bytes(snapshot.read_bytes() + b"x")
    (bad / "snapshot.json").write_text(snapshot.with_name("snapshot.json").read_text())
    with pytest.raises(ValueError, match="SHA256"):
        C.load_model(bad / "model.pt", TOK)
    with pytest.raises(ValueError):
        C.capture_latest(snapshot, TOK, tmp / "snaps")  # a chat snapshot is not a training checkpoint


def test_posttrain_chat_prompt_and_suite(trained, tmp_path):
    tmp, work = trained
    snapshot = C.capture_latest(work / "run/latest.pt", TOK, tmp / "snaps2")
    model, sp, _ = C.load_model(snapshot, TOK)
    ids = PC.encode_prompt([{"role": "user", "content": "Hi"}], sp)
    assert sp.decode(ids[-len(sp.encode("<|assistant|>\n", out_type=int)):]).strip() == "<|assistant|>"
    with pytest.raises(ValueError):
        PC.encode_prompt([{"role": "assistant", "content": "Hi"}], sp)
    engine = DecodeEngine(model, dtype=torch.float32, use_cuda_graph=False)
    result = PC.generate(engine, sp, [{"role": "user", "content": "Hi"}], max_new_tokens=5, max_context=128)
    assert result["prompt_tokens"] == len(ids) and result["stop_reason"] in {"length", "eos"}
    assert len(result["token_ids"]) == result["generated_tokens"] <= 5
    suite = tmp_path / "suite.json"
    suite.write_text(json.dumps({"prompts": [{"id": "a", "prompt": "One"}, {"id": "b", "prompt": "Two"}]}))
    out = tmp_path / "report.json"
    assert PC.main(["--snapshot", str(snapshot), "--tokenizer", str(TOK), "--device", "cpu", "--prompts-json",
                    str(suite), "--output-json", str(out), "--max-new-tokens", "3", "--max-context", "64"]) == 0
    report = json.loads(out.read_text())
    assert report["complete"] is True and [r["id"] for r in report["results"]] == ["a", "b"]
    batch = PC.generate_batch(engine, torch.randint(0, 32768, (3, 8)), 5)
    assert batch["tokens"].shape == (3, 5) and batch["tokens_per_second"] > 0
