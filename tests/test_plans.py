"""Post-training plan schemas (`train/plans.py`): defaults, kinds, relations and the templates shipped in ``configs/``.

Keys and defaults are the reference's (posttrain.py:34-97, dpo.py:38-80).
"""
import json
from pathlib import Path

import pytest

from warpstate_ai_b200.train.plans import DPO_PLAN, SFT_PLAN, PlanSchema, Relation, Setting

ROOT = Path(__file__).resolve().parents[1]


def sft(**training):
    return {"format": "warpstate-posttrain-plan-v1", "stage": "sft", "training": training}


def dpo(**training):
    return {"format": "warpstate-dpo-plan-v1", "stage": "dpo", "training": training}


def test_defaults_are_the_documented_ones():
    s = SFT_PLAN.resolve(sft())
    assert (s["micro_batch"], s["grad_accum"], s["lr"], s["min_lr"], s["warmup_ratio"]) == (4, 4, 5e-6, 0.0, 0.03)
    assert (s["sequence_length"], s["epochs"], s["max_steps"], s["seed"], s["clip_grad_norm"]) == (2048, 1, None, 42, 1.0)
    assert s["bf16_residuals"] is True and s["gradient_checkpointing"] is False and s["loss_mode"] == "compiled-full"
    d = DPO_PLAN.resolve(dpo())
    assert (d["micro_batch"], d["grad_accum"], d["lr"], d["warmup_ratio"], d["beta"]) == (2, 8, 5e-7, 0.1, 5.0)
    assert (d["objective"], d["head_chunk_size"], d["reference_mode"]) == ("length-normalized-dpo", 256, "cached")
    assert set(d) - set(s) == {"beta", "objective", "head_chunk_size", "reference_mode"} and set(s) - set(d) == {"loss_mode"}
    assert SFT_PLAN.resolve({"format": "warpstate-posttrain-plan-v1", "stage": "sft"}) == s       # no training section at all


def test_overrides_replace_defaults_and_nothing_else():
    s = SFT_PLAN.resolve(sft(lr=2e-5, min_lr=2e-6, max_steps=12, loss_mode="checkpointed", bf16_residuals=False))
    assert (s["lr"], s["min_lr"], s["max_steps"], s["loss_mode"], s["bf16_residuals"]) == (2e-5, 2e-6, 12, "checkpointed", False)
    assert s["grad_accum"] == 4
    assert DPO_PLAN.resolve(dpo(reference_mode="resident", beta=0.1))["beta"] == 0.1


@pytest.mark.parametrize("schema, plan", [
    (SFT_PLAN, dpo()), (DPO_PLAN, sft()), (SFT_PLAN, {"format": "warpstate-posttrain-plan-v1", "stage": "dpo"}),
    (SFT_PLAN, {"stage": "sft"}), (DPO_PLAN, {}),
])
def test_a_plan_of_another_stage_or_format_is_refused(schema, plan):
    with pytest.raises(ValueError, match="expected a warpstate-.*-plan-v1 plan for stage"):
        schema.resolve(plan)


def test_unknown_keys_are_named():
    with pytest.raises(ValueError, match=r"unknown training settings in the plan: \['learning_rate', 'zeta'\]"):
        SFT_PLAN.resolve(sft(zeta=1, learning_rate=1e-5))
    with pytest.raises(ValueError, match=r"\['beta'\]"):
        SFT_PLAN.resolve(sft(beta=0.1))                                       # a DPO key in an SFT plan


@pytest.mark.parametrize("key, value, wording", [
    ("micro_batch", 0, "a positive integer"), ("micro_batch", 2.0, "a positive integer"), ("micro_batch", True, "a positive integer"),
    ("max_steps", 0, "null or a positive integer"), ("max_steps", "10", "null or a positive integer"),
    ("weight_decay", -0.1, "a finite number >= 0"), ("weight_decay", float("inf"), "a finite number >= 0"),
    ("lr", 0, "a finite number > 0"), ("lr", float("nan"), "a finite number > 0"), ("lr", "1e-5", "a finite number > 0"),
    ("warmup_ratio", 1.0, r"a number in \[0, 1\)"), ("warmup_ratio", -0.01, r"a number in \[0, 1\)"),
    ("compile_core", 1, "true or false"), ("deterministic", "yes", "true or false"),
    ("seed", -1, "an integer >= 0"), ("seed", 1.5, "an integer >= 0"),
    ("loss_mode", "fused", r"one of the listed choices \['full', 'compiled-full', 'checkpointed'\]"),
])
def test_each_kind_states_what_it_accepts(key, value, wording):
    with pytest.raises(ValueError, match=f"training.{key} must be {wording}; got"):
        SFT_PLAN.resolve(sft(**{key: value}))


def test_values_at_the_edges_of_their_kinds_pass():
    s = SFT_PLAN.resolve(sft(warmup_ratio=0, weight_decay=0, seed=0, max_steps=1, min_lr=5e-6, lr=5e-6, eval_every=1))
    assert s["warmup_ratio"] == 0 and s["min_lr"] == s["lr"]
    d = DPO_PLAN.resolve(dpo(objective="summed-dpo", head_chunk_size=1))
    assert d["objective"] == "summed-dpo"
    with pytest.raises(ValueError, match="objective must be one of the listed choices"):
        DPO_PLAN.resolve(dpo(objective="ipo"))
    with pytest.raises(ValueError, match="reference_mode"):
        DPO_PLAN.resolve(dpo(reference_mode="offloaded"))


def test_relations_between_keys_are_checked_after_the_keys_themselves():
    with pytest.raises(ValueError, match="training.min_lr must not exceed training.lr"):
        SFT_PLAN.resolve(sft(lr=1e-6, min_lr=1e-5))
    with pytest.raises(ValueError, match="training.min_lr must not exceed training.lr"):
        DPO_PLAN.resolve(dpo(min_lr=1e-6))                                    # above the DPO default rate of 5e-7
    with pytest.raises(ValueError, match="training.lr must be"):              # the kind error comes first
        SFT_PLAN.resolve(sft(lr=-1.0, min_lr=1e-5))
    schema = PlanSchema("f", "s", (Setting("a", 1, "count"), Setting("b", 2, "count")),
                        (Relation(lambda v: v["a"] < v["b"], "a must stay below b"),))
    assert schema.defaults == {"a": 1, "b": 2}
    assert schema.resolve({"format": "f", "stage": "s", "training": {"b": 5}}) == {"a": 1, "b": 5}
    with pytest.raises(ValueError, match="a must stay below b"):
        schema.resolve({"format": "f", "stage": "s", "training": {"a": 2}})


@pytest.mark.parametrize("name, schema", [("posttrain_plan.json", SFT_PLAN), ("dpo_plan.json", DPO_PLAN)])
def test_the_shipped_templates_are_valid_plans(name, schema):
    plan, settings = schema.read(ROOT / "configs" / name)
    assert plan["after_completion"] == "pause_for_evaluation"
    assert settings["sequence_length"] == 2048 and settings["min_lr"] <= settings["lr"]
    for key, value in plan["training"].items():
        assert settings[key] == value
    handoff = plan["handoff"]
    assert handoff["processes"] == 8 and handoff["preflight"] is True and not Path(handoff["work_dir"]).is_absolute()


def test_read_returns_the_document_and_its_effective_settings(tmp_path):
    path = tmp_path / "plan.json"
    document = dict(dpo(beta=0.1, max_steps=3), sft={"step": 9}, note="x")
    path.write_text(json.dumps(document))
    plan, settings = DPO_PLAN.read(path)
    assert plan == document and settings["beta"] == 0.1 and settings["max_steps"] == 3 and settings["grad_accum"] == 8
    path.write_text("{")
    with pytest.raises(json.JSONDecodeError):
        DPO_PLAN.read(path)
