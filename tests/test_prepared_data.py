"""Prepared post-training data: what `prepare_posttrain_data` writes is what the loaders verify, and any disagreement
between manifest, files and rows refuses the directory (reference posttrain.py:117-156, ops/dpo_data.py:37-78)."""
import json
from pathlib import Path

import pytest

from warpstate_ai_b200.data import dpo as DD
from warpstate_ai_b200.data import prepare_posttrain as PP
from warpstate_ai_b200.data import sft as SD
from warpstate_ai_b200.data.prepared import DATA_FORMAT, PreparedDirectory
from warpstate_ai_b200.utils.io import digest

TOK = Path(__file__).resolve().parents[1] / "tokenizer.model"
LENGTH = 48


def conversations(n):
    return [{"messages": [{"role": "user", "content": f"Count to {i}."}, {"role": "assistant", "content": f"{i} it is."}]}
            for i in range(n)]


def pairs(n):
    return [{"prompt": [{"role": "user", "content": f"Pick {i}."}], "chosen": [{"role": "assistant", "content": f"{i}"}],
             "rejected": [{"role": "assistant", "content": f"No, {i + 1}."}]} for i in range(n)]


@pytest.fixture(scope="module")
def tokenizer():
    import sentencepiece as spm
    return spm.SentencePieceProcessor(model_file=str(TOK))


@pytest.fixture()
def prepared(tmp_path):
    too_long = {"messages": [{"role": "user", "content": "word " * 200}, {"role": "assistant", "content": "ok"}]}
    no_target = {"messages": [{"role": "user", "content": "only a question"}]}
    bad_pair = {"prompt": [{"role": "assistant", "content": "x"}], "chosen": [], "rejected": []}
    manifest = PP.prepare(tmp_path / "data", TOK, LENGTH, sft_rows=conversations(30) + [too_long, no_target],
                          dpo_rows=pairs(30) + [bad_pair], val_modulus=5)
    return tmp_path / "data", manifest


def test_preparation_counts_every_row_and_never_truncates(prepared, tokenizer):
    directory, manifest = prepared
    assert manifest["format"] == DATA_FORMAT and manifest["complete"] is True and manifest["max_length"] == LENGTH
    assert manifest["tokenizer_sha256"] == digest(TOK) and manifest["renderer_sha256"] == SD.renderer_sha256()
    assert manifest["renderer_format"] == "warpstate-segmented-roles-v1"
    assert manifest["mask_format"] == "warpstate-final-assistant-response-v1"
    assert manifest["dropped"] == {"sft": 2, "dpo": 1}
    outputs = manifest["outputs"]
    assert set(outputs) == {"sft_train.jsonl", "sft_val.jsonl", "dpo_train.jsonl", "dpo_val.jsonl"}
    assert outputs["sft_train.jsonl"]["rows"] + outputs["sft_val.jsonl"]["rows"] == 30
    assert outputs["sft_val.jsonl"]["rows"] >= 1 and outputs["dpo_val.jsonl"]["rows"] >= 1
    for name, entry in outputs.items():
        rows = [json.loads(line) for line in (directory / name).read_text().splitlines()]
        assert entry["sha256"] == digest(directory / name) and entry["rows"] == len(rows)
        if name.startswith("sft"):
            assert entry["tokens"] == sum(r["tokens"] for r in rows) and all(r["tokens"] <= LENGTH for r in rows)
            record = SD.encode_messages(rows[0]["messages"], tokenizer)
            assert (rows[0]["tokens"], rows[0]["supervised_tokens"]) == (len(record["input_ids"]), SD.supervised_count(record))
        else:
            assert entry["tokens"] == sum(sum(r["tokens"].values()) for r in rows)
            assert entry["supervised_tokens"] == sum(sum(r["supervised_tokens"].values()) for r in rows)
    assert json.loads((directory / "manifest.json").read_text()) == manifest


def test_hold_out_assignment_depends_on_the_row_alone(tmp_path):
    first = PP.prepare(tmp_path / "a", TOK, LENGTH, sft_rows=conversations(40), val_modulus=4)
    second = PP.prepare(tmp_path / "b", TOK, LENGTH, sft_rows=list(reversed(conversations(40))), val_modulus=4)
    held = lambda d: sorted(line for line in (tmp_path / d / "sft_val.jsonl").read_text().splitlines())
    assert held("a") == held("b") and 1 <= len(held("a")) < 40
    assert first["outputs"]["sft_val.jsonl"]["rows"] == second["outputs"]["sft_val.jsonl"]["rows"]
    lone = PP.prepare(tmp_path / "c", TOK, LENGTH, sft_rows=conversations(2), val_modulus=10 ** 9)
    assert lone["outputs"]["sft_val.jsonl"]["rows"] == 1 and lone["outputs"]["sft_train.jsonl"]["rows"] == 1


def test_loaders_return_what_was_prepared(prepared, tokenizer):
    directory, manifest = prepared
    train, val, loaded_manifest, manifest_hash = SD.load_data(directory, tokenizer, digest(TOK), LENGTH)
    assert loaded_manifest == manifest and manifest_hash == digest(directory / "manifest.json")
    assert len(train) == manifest["outputs"]["sft_train.jsonl"]["rows"] and len(val) == manifest["outputs"]["sft_val.jsonl"]["rows"]
    assert sum(len(r["input_ids"]) for r in train) == manifest["outputs"]["sft_train.jsonl"]["tokens"]
    ptrain, pval, _, _ = DD.load_data(directory, tokenizer, digest(TOK), LENGTH)
    assert len(ptrain) + len(pval) == 30 and set(ptrain[0]) == {"chosen", "rejected"}
    assert sum(DD.pair_targets(p) for p in ptrain) == manifest["outputs"]["dpo_train.jsonl"]["supervised_tokens"]


@pytest.mark.parametrize("key, value, complaint", [
    ("format", "warpstate-posttrain-data-v0", "is not prepared post-training data"),
    ("complete", False, "was not finished"),
    ("tokenizer_sha256", "0" * 64, "another tokenizer"),
    ("renderer_sha256", "1" * 64, "another version of the renderer"),
    ("max_length", LENGTH * 2, "another sequence length"),
])
def test_a_manifest_for_other_circumstances_is_refused(prepared, tokenizer, key, value, complaint):
    directory, manifest = prepared
    (directory / "manifest.json").write_text(json.dumps(dict(manifest, **{key: value})))
    with pytest.raises(ValueError, match=complaint):
        SD.load_data(directory, tokenizer, digest(TOK), LENGTH)
    with pytest.raises(ValueError, match=complaint):
        DD.load_data(directory, tokenizer, digest(TOK), LENGTH)


def rewrite(directory, manifest, name, rows, **entry_changes):
    """Replace a split and make its manifest entry consistent with the new file except for ``entry_changes``."""
    path = directory / name
    path.write_text("".join(json.dumps(r) + "\n" for r in rows))
    entry = dict(manifest["outputs"][name], sha256=digest(path))
    entry.update(entry_changes)
    manifest = dict(manifest, outputs=dict(manifest["outputs"], **{name: entry}))
    (directory / "manifest.json").write_text(json.dumps(manifest))


def test_files_rows_and_totals_must_agree_with_the_manifest(prepared, tokenizer):
    directory, manifest = prepared
    load = lambda: SD.load_data(directory, tokenizer, digest(TOK), LENGTH)
    name = "sft_train.jsonl"
    rows = [json.loads(line) for line in (directory / name).read_text().splitlines()]
    original = (directory / name).read_text()
    (directory / name).write_text(original + "\n")                                    # an edited file: hash differs
    with pytest.raises(ValueError, match="differs from its manifest entry"):
        load()
    edited = [dict(rows[0], tokens=rows[0]["tokens"] + 1)] + rows[1:]                  # a row lying about itself
    rewrite(directory, manifest, name, edited)
    with pytest.raises(ValueError, match=f"{name}:1: the row's token counts do not match"):
        load()
    rewrite(directory, manifest, name, rows[:-1])                                     # a row dropped, hash updated
    with pytest.raises(ValueError, match="not the .* rows its manifest promises"):
        load()
    rewrite(directory, manifest, name, rows, tokens=manifest["outputs"][name]["tokens"] + 1)
    with pytest.raises(ValueError, match="token totals differ"):
        load()
    rewrite(directory, manifest, name, rows)                                          # consistent again
    assert len(load()[0]) == len(rows)
    (directory / name).unlink()
    with pytest.raises(ValueError, match="is missing from"):
        load()


def test_pair_rows_are_checked_branch_by_branch(prepared, tokenizer):
    directory, manifest = prepared
    name = "dpo_train.jsonl"
    rows = [json.loads(line) for line in (directory / name).read_text().splitlines()]
    lying = dict(rows[2], supervised_tokens=dict(rows[2]["supervised_tokens"], rejected=rows[2]["supervised_tokens"]["rejected"] + 1))
    rewrite(directory, manifest, name, rows[:2] + [lying] + rows[3:])
    with pytest.raises(ValueError, match=f"{name}:3: the row's token counts do not match"):
        DD.load_data(directory, tokenizer, digest(TOK), LENGTH)
    SD.load_data(directory, tokenizer, digest(TOK), LENGTH)                            # the SFT splits are still fine


def test_command_line_prepares_from_jsonl_files(tmp_path, capsys):
    source = tmp_path / "sft.jsonl"
    source.write_text("".join(json.dumps(r) + "\n" for r in conversations(6)) + "\n")
    PP.main(["--out-dir", str(tmp_path / "out"), "--tokenizer", str(TOK), "--max-length", str(LENGTH), "--sft", str(source),
             "--val-modulus", "3"])
    manifest = json.loads((tmp_path / "out/manifest.json").read_text())
    assert set(manifest["outputs"]) == {"sft_train.jsonl", "sft_val.jsonl"} and manifest["dropped"] == {"sft": 0, "dpo": 0}
    directory = PreparedDirectory(tmp_path / "out", digest(TOK), SD.renderer_sha256(), LENGTH)
    assert directory.manifest_digest() == digest(tmp_path / "out/manifest.json")
