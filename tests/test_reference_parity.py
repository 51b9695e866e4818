"""Differential tests: pure functions of this package against the reference's own, with the reference imported as a
library from ``baseline/_ref`` (skipped where it is not installed).  Random or enumerated inputs, same outputs.

Covered: token windows and update slices, resume-signature decisions, SFT batching and schedules, the SFT and DPO
renderers and collators, the chat prompt, sampling and n-gram bans, the DPO objective and its schedule.
"""
import contextlib
import importlib
import itertools
import json
import random
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REF = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
TOK = Path(__file__).resolve().parents[1] / "tokenizer.model"
SHADOWED = ("warpstate", "ops", "run_40b", "posttrain", "dpo", "chat")


@contextlib.contextmanager
def reference_import_path():
    """Inside the block, ``import run_40b`` / ``ops.*`` / ``warpstate`` resolve to the reference's files; afterwards the
    repository's own modules of the same names are back."""
    def ours(name):
        return name in SHADOWED or name.split(".")[0] in SHADOWED
    saved = {name: module for name, module in sys.modules.items() if ours(name)}
    for name in saved:
        del sys.modules[name]
    saved_path = list(sys.path)
    root = str(REF.parents[1])
    sys.path[:] = [str(REF)] + [p for p in sys.path if p not in ("", root) and Path(p or ".").resolve() != REF.parents[1]]
    try:
        yield
    finally:
        sys.path[:] = saved_path
        for name in [name for name in sys.modules if ours(name)]:
            del sys.modules[name]
        sys.modules.update(saved)


@pytest.fixture(scope="module")
def ref():
    if not (REF / "run_40b.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    with reference_import_path():
        modules = {name: importlib.import_module(name) for name in
                   ("run_40b", "posttrain", "dpo", "chat", "ops.posttrain_data", "ops.dpo_data", "ops.posttrain_chat")}
    for module in modules.values():
        assert str(REF) in str(module.__file__)
    return modules


@pytest.fixture(scope="module")
def tokenizer():
    import sentencepiece as spm
    return spm.SentencePieceProcessor(model_file=str(TOK))


# ------------------------------------------------------------------------------------------- pretraining data path
def test_token_windows_and_update_slices(ref):
    from warpstate_ai_b200.data import tokens as T
    data = np.random.default_rng(0).integers(0, 32768, size=997, dtype=np.uint16)
    for cursor, batch, length, valid in [(0, 2, 8, 16), (990, 2, 8, 5), (5000, 3, 16, 0), (996, 1, 4, 4), (123, 4, 32, 100)]:
        ours = T.batches(data, cursor, batch, length, valid, torch.device("cpu"))
        theirs = ref["run_40b"].batches(data, cursor, batch, length, valid, torch.device("cpu"))
        assert all(torch.equal(a, b) and a.dtype == b.dtype for a, b in zip(ours, theirs))
    for target, micro, world in itertools.product((1, 9, 32, 73, 1000), (8, 16, 24), (1, 2, 3)):
        for rank in range(world):
            assert list(T.update_slices(target, micro, world, rank)) == list(ref["run_40b"].update_slices(target, micro, world, rank))


def test_resume_signature_decisions(ref):
    from warpstate_ai_b200.train.signature import check_resume_signature
    base = {"settings": {"seq_len": 2048, "micro_batch": 8, "grad_accum": 4, "train_tokens": 10 ** 10, "lr": 1.5e-4, "min_lr": 1.5e-5,
                         "warmup_steps": 1000, "weight_decay": 0.1, "seed": 1, "activation_checkpointing": True,
                         "loss_chunk_size": 128, "compile": False, "world_size": 2},
            "data": {"tokens": 123, "sha": "abc"}}
    changes = [{}, {"micro_batch": 4, "grad_accum": 8}, {"micro_batch": 4}, {"world_size": 4, "grad_accum": 2}, {"lr": 1e-4},
               {"seed": 2}, {"loss_mode": "full"}, {"bf16_residuals": True, "compile_core": True}, {"train_tokens": 5},
               {"ddp_bucket_cap_mb": 64}, {"gradient_mode": "compiled-autograd"}, {"seq_len": 1024, "micro_batch": 16},
               {"activation_checkpointing": False, "loss_chunk_size": 256}, {"warmup_steps": 10}, {"matmul_execution": {"plan": 1}}]

    def outcome(check, old, new, reconfigure):
        try:
            return check(old, new, reconfigure)
        except ValueError as problem:
            return str(problem)

    for change, reconfigure, other_data in itertools.product(changes, (False, True), (False, True)):
        new = {"settings": dict(base["settings"], **change), "data": dict(base["data"], sha="xyz") if other_data else dict(base["data"])}
        legacy = {"settings": {k: v for k, v in base["settings"].items() if k != "world_size"}, "data": dict(base["data"])}
        for old in (base, legacy):
            assert outcome(check_resume_signature, old, new, reconfigure) == \
                outcome(ref["run_40b"].check_resume_signature, old, new, reconfigure), (change, reconfigure, other_data)


# ------------------------------------------------------------------------------------------- SFT batching, schedules
def test_sft_batching_and_schedules(ref):
    from warpstate_ai_b200.data import sft as SD
    from warpstate_ai_b200.train import sft as ST
    theirs = ref["posttrain"]
    for size, seed, epochs, batch in [(10, 3, 2, 4), (7, 0, 3, 7), (33, 9, 1, 8), (5, 1, 2, 16)]:
        assert list(SD.epoch_order(size, seed, 1)) == list(theirs.epoch_order(size, seed, 1))
        cursor_a = cursor_b = 0
        while True:
            a = SD.update_indices(size, seed, cursor_a, epochs, batch)
            b = theirs.update_indices(size, seed, cursor_b, epochs, batch)
            assert (list(a[0]), a[1]) == (list(b[0]), b[1])
            if not a[0]:
                break
            cursor_a, cursor_b = a[1], b[1]
    records = [{"input_ids": [1, 5, 6, 7], "labels": [-100, -100, 6, 7]}, None, {"input_ids": [1, 9], "labels": [-100, 9]}]
    for a, b in zip(SD.collate(records, 6, 0), theirs.collate(records, 6, 0)):
        assert torch.equal(a, b)
    settings = {"lr": 1e-5, "min_lr": 1e-6, "warmup_ratio": 0.03}
    for total in (1, 2, 7, 100, 1234):
        for step in range(0, total, max(1, total // 50)):
            assert ST.learning_rate(step, total, settings) == pytest.approx(theirs.learning_rate(step, total, settings), rel=1e-12)
    loss = torch.tensor(2.5)
    for local, total, world in [(3, 3, 2), (0, 7, 2), (5, 12, 4)]:
        assert torch.equal(ST.token_weighted_loss(loss, local, total, world), theirs.token_weighted_loss(loss, local, total, world))


def test_dpo_schedule_objective_and_identity(ref):
    from warpstate_ai_b200.train import dpo as DT
    from warpstate_ai_b200.train.reference_cache import identity_digest
    theirs = ref["dpo"]
    settings = {"lr": 5e-7, "min_lr": 0.0, "warmup_ratio": 0.1}
    for total in (1, 3, 10, 777):
        for step in range(total):
            assert DT.learning_rate(step, total, settings) == pytest.approx(theirs.learning_rate(step, total, settings), rel=1e-12, abs=1e-20)
    torch.manual_seed(0)
    policy = (torch.randn(6, 2) * 20).requires_grad_(True)
    reference = torch.randn(6, 2, dtype=torch.float64) * 20
    counts = torch.randint(1, 50, (6, 2))
    for objective, beta in (("length-normalized-dpo", 5.0), ("summed-dpo", 0.1)):
        mine = DT.preference_metrics(policy, reference, counts, beta, objective)
        other = theirs.preference_metrics(policy, reference, counts, beta, objective)
        for a, b in zip(mine, other):
            assert torch.allclose(a, b, rtol=1e-6, atol=1e-7)
        grad_a, = torch.autograd.grad(mine[0].sum(), policy, retain_graph=True)
        grad_b, = torch.autograd.grad(other[0].sum(), policy)
        assert torch.allclose(grad_a, grad_b, rtol=1e-6, atol=1e-8)
    identity = {"weights": "aa", "nested": {"b": 1, "a": [1, 2.5, None]}, "world": 8}
    assert identity_digest(identity) == theirs.identity_digest(identity)


# ------------------------------------------------------------------------------------------- renderers
CONVERSATIONS = [
    [{"role": "user", "content": "Name a colour."}, {"role": "assistant", "content": "Blue."}],
    [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "4"},
     {"role": "user", "content": "And 3+3?"}, {"role": "assistant", "content": "Six, of course."}],
    [{"role": "user", "content": "Use the tool."}, {"role": "assistant", "content": "calling"}, {"role": "tool", "content": "{\"x\": 1}"},
     {"role": "assistant", "content": "It says x is 1.  Ünïcödé too."}],
]


def test_sft_renderer_and_chat_prompt(ref, tokenizer):
    from warpstate_ai_b200.data import sft as SD
    from warpstate_ai_b200.serve import posttrain_chat as PC
    for messages in CONVERSATIONS:
        assert SD.encode_messages(messages, tokenizer) == ref["ops.posttrain_data"].encode_messages(messages, tokenizer)
        assert SD.encode_messages(messages, tokenizer, max_length=512) == ref["ops.posttrain_data"].encode_messages(messages, tokenizer, 512)
        prompt = messages[:-1]
        assert PC.encode_prompt(prompt, tokenizer) == ref["ops.posttrain_chat"].encode_prompt(prompt, tokenizer)
    bad = [[], [{"role": "user", "content": "no answer"}], [{"role": "user", "content": ""}, {"role": "assistant", "content": "x"}],
           [{"role": "wizard", "content": "x"}, {"role": "assistant", "content": "y"}]]
    for messages in bad:
        for function in (SD.encode_messages, ref["ops.posttrain_data"].encode_messages):
            with pytest.raises(ValueError):
                function(messages, tokenizer)
    for function in (SD.encode_messages, ref["ops.posttrain_data"].encode_messages):
        with pytest.raises(ValueError):
            function(CONVERSATIONS[1], tokenizer, max_length=8)


def test_preference_pairs_and_their_collation(ref, tokenizer):
    from warpstate_ai_b200.data import dpo as DD
    rows = [{"prompt": conversation[:-1], "chosen": [conversation[-1]], "rejected": [{"role": "assistant", "content": "I would rather not."}]}
            for conversation in CONVERSATIONS]
    pairs = []
    for row in rows:
        mine = DD.encode_pair(row, tokenizer, 256)
        assert mine == ref["ops.dpo_data"].encode_pair(row, tokenizer, 256)
        pairs.append(mine)
    for a, b in zip(DD.collate_pairs([pairs[0], None, pairs[2]], 96, 0), ref["ops.dpo_data"].collate_pairs([pairs[0], None, pairs[2]], 96, 0)):
        assert torch.equal(a, b)
    bad = dict(rows[0], rejected=rows[0]["chosen"])
    for function in (DD.encode_pair, ref["ops.dpo_data"].encode_pair):
        with pytest.raises(ValueError):
            function(bad, tokenizer, 256)
        with pytest.raises(ValueError):
            function(dict(rows[1], prompt=CONVERSATIONS[1][:3]), tokenizer, 256)     # prompt ends with an assistant turn


# ------------------------------------------------------------------------------------------- sampling
def test_sampling_and_ngram_bans(ref):
    from warpstate_ai_b200.serve import sampling as S
    rng = random.Random(0)
    for _ in range(200):
        tokens = [rng.randrange(4) for _ in range(rng.randrange(0, 12))]
        size = rng.randrange(0, 5)
        assert set(S.banned_ngram_tokens(tokens, size)) == set(ref["chat"].banned_ngram_tokens(tokens, size)), (tokens, size)
    torch.manual_seed(1)
    for case in range(60):
        logits = torch.randn(24) * 3
        previous = [rng.randrange(24) for _ in range(rng.randrange(0, 6))]
        banned = {rng.randrange(24) for _ in range(rng.randrange(0, 4))}
        settings = dict(temperature=rng.choice([0.0, 0.5, 1.0, 1.7]), top_k=rng.choice([0, 1, 5, 40]), top_p=rng.choice([0.3, 0.9, 1.0]))
        penalty = rng.choice([1.0, 1.2, 2.0])
        draws = []
        for function in (S.sample_token, ref["chat"].sample_token):
            generator = torch.Generator().manual_seed(case)
            draws.append([function(logits, settings["temperature"], settings["top_k"], settings["top_p"], generator,
                                   previous_tokens=previous, repetition_penalty=penalty, banned_tokens=banned) for _ in range(5)])
        assert draws[0] == draws[1], (case, settings, penalty)
    everything = set(range(24))
    assert S.sample_token(torch.zeros(24), 0.0, 0, 1.0, torch.Generator(), banned_tokens=everything) is None
    assert ref["chat"].sample_token(torch.zeros(24), 0.0, 0, 1.0, torch.Generator(), banned_tokens=everything) is None


# ------------------------------------------------------------------------------------------- cached decode
@pytest.mark.parametrize("parallel", [False, True])
def test_chat_generation_follows_the_reference_decoder(ref, tokenizer, parallel):
    """The same frozen model behind the reference's cached decoder and behind this framework's decode engine (FP32 on the
    CPU): same prompt tokens, same reply, same stop reason, same record; logits along the way agree to rounding."""
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.serve import posttrain_chat as PC
    from warpstate_ai_b200.serve.engine import DecodeEngine
    with reference_import_path():
        their_model_module = importlib.import_module("warpstate")
    theirs = ref["ops.posttrain_chat"]
    torch.manual_seed(7)
    settings = dict(vocab_size=32768, d_model=32, n_heads=4, n_cores=2, logical_depth=4, ffn_hidden=48, chunk_size=8,
                    gradient_checkpointing=False, parallel_memory=parallel)
    model = WarpStateLM(WarpStateConfig(**settings))
    with torch.no_grad():                                  # decisive logits: a reply must not hinge on the seventh digit
        model.embed.weight.normal_(0, 1.0)
        model.depth_scale.normal_(0, 0.1)
        for core in model.cores:
            core.memory_mix_logit.normal_()
    model.eval().requires_grad_(False)
    twin = their_model_module.WarpStateLM(their_model_module.WarpStateConfig(**settings))
    twin.load_state_dict(model.state_dict())
    twin.eval().requires_grad_(False)
    engine, decoder = DecodeEngine(model, dtype=torch.float32), theirs.CachedDecoder(twin, dtype=torch.float32)
    conversation = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Name three colours, please."}]
    for kwargs in (dict(max_new_tokens=20, max_context=200, temperature=0.0), dict(max_new_tokens=30, max_context=40, temperature=0.0),
                   dict(max_new_tokens=12, max_context=200, temperature=0.7, seed=5)):
        mine = PC.generate(engine, tokenizer, conversation, **kwargs)
        other = theirs.generate(decoder, tokenizer, conversation, **kwargs)
        assert set(mine) == set(other)
        for key in ("response", "token_ids", "prompt_tokens", "generated_tokens", "sampled_tokens", "stop_reason", "temperature", "seed"):
            assert mine[key] == other[key], (key, kwargs)
    # the prompt's last logits, position by position through two chunk boundaries
    ids = PC.encode_prompt(conversation, tokenizer)
    caches = decoder.new_caches()
    for value in ids:
        reference_logits = decoder.step(torch.tensor([[value]]), caches)[0, -1]
    mine = engine.prefill(torch.tensor([ids]))[0]
    assert len(ids) > 16 and torch.allclose(mine, reference_logits, rtol=1e-4, atol=1e-4)


def test_probe_generation_follows_the_reference_probe(ref, tokenizer):
    """The base-model probe (`chat.py`): same model, same prompt, same settings -> the same tokens, for the arg-max, for
    seeded sampling with the repetition protections on, and when the prompt has to be cut to fit the context."""
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    from warpstate_ai_b200.serve import chat as C
    with reference_import_path():
        their_model_module = importlib.import_module("warpstate")
    torch.manual_seed(9)
    settings = dict(vocab_size=32768, d_model=32, n_heads=4, n_cores=1, logical_depth=3, ffn_hidden=48, chunk_size=8,
                    gradient_checkpointing=False, parallel_memory=True)
    model = WarpStateLM(WarpStateConfig(**settings))
    with torch.no_grad():
        model.embed.weight.normal_(0, 1.0)
        model.depth_bias.normal_(0, 0.1)
    model.eval().requires_grad_(False)
    twin = their_model_module.WarpStateLM(their_model_module.WarpStateConfig(**settings))
    twin.load_state_dict(model.state_dict())
    twin.eval().requires_grad_(False)
    prompt = "Question: which way does the river run after the bridge?\nAnswer:"
    cases = [dict(max_new_tokens=24, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0, no_repeat_ngram_size=0, max_context=256),
             dict(max_new_tokens=24, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.3, no_repeat_ngram_size=3, max_context=256),
             dict(max_new_tokens=24, temperature=0.9, top_k=50, top_p=0.92, seed=21, repetition_penalty=1.2, no_repeat_ngram_size=4, max_context=256),
             dict(max_new_tokens=10, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.2, no_repeat_ngram_size=2, max_context=18)]
    for case in cases:
        mine = list(C.generate(model, tokenizer, prompt, **case))
        other = list(ref["chat"].generate(twin, tokenizer, prompt, **case))
        assert mine == other and 1 <= len(mine) <= case["max_new_tokens"], case
    plain, protected = (list(C.generate(model, tokenizer, prompt, **case)) for case in cases[:2])
    assert plain != protected                                    # the protections did change the reply


@pytest.mark.parametrize("parallel", [False, True])
def test_sequence_scores_and_masked_loss_follow_the_reference_heads(ref, parallel):
    """DPO's scoring head and the memory-saving loss head, with gradients, FP32 on the CPU."""
    from warpstate_ai_b200 import WarpStateConfig, WarpStateLM
    with reference_import_path():
        their_model_module = importlib.import_module("warpstate")
    torch.manual_seed(11)
    settings = dict(vocab_size=211, d_model=32, n_heads=4, n_cores=2, logical_depth=3, ffn_hidden=48, chunk_size=8,
                    gradient_checkpointing=False, parallel_memory=parallel, loss_chunk_size=5)
    model = WarpStateLM(WarpStateConfig(**settings))
    with torch.no_grad():
        model.embed.weight.normal_(0, 0.3)
        model.depth_scale.normal_(0, 0.1)
    scorer = their_model_module.WarpStateLM(their_model_module.WarpStateConfig(**settings))
    scorer.load_state_dict(model.state_dict())
    ref["dpo"].apply_sequence_logps(scorer, 6)
    x = torch.randint(0, 211, (4, 24))
    y = torch.randint(0, 211, (4, 24))
    y[:, :9] = -100
    y[3] = -100                                                    # a branch with nothing to score
    mine = model.sequence_logps(x, y, head_chunk_size=6)
    _, theirs = scorer(x, y, return_logits=False)
    assert torch.allclose(mine, theirs, rtol=1e-5, atol=1e-5) and float(mine[3].detach()) == 0.0
    weights = torch.tensor([1.0, -2.0, 0.5, 3.0])
    (mine * weights).sum().backward()
    (theirs * weights).sum().backward()
    for (name, a), (_, b) in zip(model.named_parameters(), scorer.named_parameters()):
        assert torch.allclose(a.grad, b.grad, rtol=1e-4, atol=1e-6), name
    # the loss head that never builds [tokens, vocabulary]
    plain = their_model_module.WarpStateLM(their_model_module.WarpStateConfig(**settings))
    plain.load_state_dict(model.state_dict())
    model.zero_grad()
    _, loss_a = model(x, y, return_logits=False)
    _, loss_b = plain(x, y, return_logits=False)
    assert torch.allclose(loss_a, loss_b, rtol=1e-6, atol=1e-6)
    loss_a.backward()
    loss_b.backward()
    for (name, a), (_, b) in zip(model.named_parameters(), plain.named_parameters()):
        assert torch.allclose(a.grad, b.grad, rtol=1e-4, atol=1e-6), name
    nothing = torch.full_like(y, -100)
    assert float(model(x, nothing, return_logits=False)[1]) == float(plain(x, nothing, return_logits=False)[1]) == 0.0


# ------------------------------------------------------------------------------------------- pretraining command line
def test_pretraining_command_line_reads_like_the_reference(ref, monkeypatch):
    """Every flag of the reference's ``run_40b.py`` exists here with the same default and the same value checks; this
    framework adds its own (device, kernels, gradient path, sharding, bootstrap)."""
    import contextlib
    import io
    from warpstate_ai_b200.train import pretrain as T
    for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(name, raising=False)

    def theirs(argv):
        monkeypatch.setattr(sys, "argv", ["run_40b.py", *argv])
        try:
            with contextlib.redirect_stderr(io.StringIO()):
                return vars(ref["run_40b"].arguments())
        except SystemExit:
            return "refused"

    def mine(argv):
        try:
            with contextlib.redirect_stderr(io.StringIO()):
                return vars(T.arguments(list(argv)))
        except SystemExit:
            return "refused"

    a, b = mine([]), theirs([])
    assert set(b) <= set(a) and set(a) - set(b) == {"bootstrap", "device", "grad_sync", "kernels", "shard_optimizer", "shard_params"}
    different = {k for k in b if a[k] != b[k]}
    assert different == {"config", "tokenizer", "work_dir", "ddp_bucket_cap_mb"}            # three path roots; buckets follow the model here
    assert (a["config"].name, a["tokenizer"].name, a["work_dir"].name) == (b["config"].name, b["tokenizer"].name, b["work_dir"].name)
    accepted = [["--micro-batch", "4", "--grad-accum", "16", "--seq-len", "1024"], ["--lr", "3e-4", "--min-lr", "3e-4"],
                ["--no-activation-checkpointing", "--bf16-residuals", "--loss-mode", "full"], ["--stage", "prepare", "--workers", "2"],
                ["--max-steps", "5", "--stop-at-step", "3", "--eval-every", "7", "--save-every", "9"],
                ["--vram-limit-gib", "150", "--vram-headroom-gib", "0"], ["--from-scratch", "--seed", "9"],
                ["--compile-core", "--compile-mode", "max-autotune-no-cudagraphs"], ["--async-checkpoint"], ["--reconfigure"],
                ["--ddp-bucket-cap-mb", "64"], ["--test-small-gpu", "--train-tokens", "73", "--val-tokens", "64", "--seq-len", "8"]]
    for argv in accepted:
        x, y = mine(argv), theirs(argv)
        assert x != "refused" and y != "refused", argv
        assert {k: x[k] for k in y if k not in different} == {k: v for k, v in y.items() if k not in different}, argv
    refused = [["--micro-batch", "0"], ["--grad-accum", "-1"], ["--seq-len", "0"], ["--lr", "1e-5", "--min-lr", "1e-4"], ["--min-lr", "0"],
               ["--weight-decay", "-0.1"], ["--max-steps", "0"], ["--stop-at-step", "0"], ["--vram-limit-gib", "0"], ["--vram-limit-gib", "inf"],
               ["--vram-headroom-gib", "-1"], ["--train-tokens", "1"], ["--val-tokens", "2048"], ["--eval-every", "0"], ["--save-every", "0"],
               ["--ddp-bucket-cap-mb", "nan"], ["--stage", "evaluate"], ["--loss-mode", "fused"], ["--weights", "w.pt", "--from-scratch"],
               ["--compile-mode", "max-autotune"], ["--warmup-steps", "0"], ["--loss-chunk-size", "0"]]
    for argv in refused:
        assert mine(argv) == theirs(argv) == "refused", argv
    # combinations of the reference's execution adapters are its own business: the flags are accepted here, reported as
    # served by the native path, and nothing is selected by them
    assert theirs(["--compile", "--compile-core"]) == "refused" and mine(["--compile", "--compile-core"]) != "refused"
    monkeypatch.setenv("WORLD_SIZE", "2")
    monkeypatch.setenv("RANK", "1")
    monkeypatch.setenv("LOCAL_RANK", "1")
    assert mine(["--stage", "all"]) == theirs(["--stage", "all"]) == "refused"              # ranks train; they do not prepare data
    x, y = mine(["--stage", "train"]), theirs(["--stage", "train"])
    assert (x["rank"], x["world_size"], x["local_rank"]) == (y["rank"], y["world_size"], y["local_rank"]) == (1, 2, 1)


# ------------------------------------------------------------------------------------------- corpus preparation
def test_corpus_preparation_writes_the_reference_bytes(ref, tmp_path, monkeypatch):
    """The same streamed documents through both ``prepare`` stages (a stand-in ``datasets`` module, the real tokenizer):
    byte-identical token files, the same manifest, and each implementation accepts the other's finished directory."""
    import types
    from warpstate_ai_b200.data import prepare as P
    rng = random.Random(4)
    words = "the of river stone and light seven quiet under machine green follows window".split()
    docs = [{"text": " ".join(rng.choice(words) for _ in range(rng.randrange(3, 40)))} for _ in range(3000)]
    docs[5] = {"text": "   "}                                                         # blank documents are skipped by both
    # holdout documents are rare (1 in 1000): make sure the stream has enough of them to fill the validation file
    from itertools import count
    held = []
    for i in count():
        text = f"validation candidate {i} " + " ".join(rng.choice(words) for _ in range(12))
        if P.is_holdout(text):
            held.append({"text": text})
        if len(held) == 12:
            break
    for position, document in zip(range(7, len(docs), 211), held):
        docs.insert(position, document)
    assert all(P.is_holdout(d["text"]) == ref["run_40b"].is_holdout(d["text"]) for d in docs[:400])

    class Stream:
        def __init__(self):
            self.position = 0

        def __iter__(self):
            while self.position < len(docs):
                self.position += 1
                yield docs[self.position - 1]

        def state_dict(self):
            return {"position": self.position}

        def load_state_dict(self, state):
            self.position = state["position"]

    monkeypatch.setitem(sys.modules, "datasets", types.SimpleNamespace(__version__="fake-1", load_dataset=lambda *a, **k: Stream()))
    monkeypatch.setitem(sys.modules, "huggingface_hub", types.SimpleNamespace(HfApi=lambda: types.SimpleNamespace(
        dataset_info=lambda name, revision: types.SimpleNamespace(sha="0123abcd"))))

    def arguments(work):
        return types.SimpleNamespace(work_dir=work, tokenizer=TOK, dataset="corpus/name", dataset_config="cfg", revision="main",
                                     train_tokens=20000, val_tokens=150, workers=1, documents_per_batch=64, test_small_gpu=True,
                                     verify_data=True)

    mine, theirs = arguments(tmp_path / "mine"), arguments(tmp_path / "theirs")
    assert P.prepare(mine) is True
    assert ref["run_40b"].prepare(theirs) is True
    for name in ("train.bin", "val.bin"):
        a, b = (mine.work_dir / "data" / name).read_bytes(), (theirs.work_dir / "data" / name).read_bytes()
        assert a == b and len(a) == 2 * (20000 if name == "train.bin" else 150), name
    m, t = (json.loads((w.work_dir / "data/manifest.json").read_text()) for w in (mine, theirs))
    assert m["signature"] == t["signature"] and m["sha256"] == t["sha256"] and m["source_revision"] == t["source_revision"] == "0123abcd"
    assert m["documents_read"] == t["documents_read"] and m["complete"] is t["complete"] is True and set(t) <= set(m)
    # a finished directory of either is "already complete" to the other
    assert ref["run_40b"].prepare(mine) is True and P.prepare(theirs) is True
    assert ref["run_40b"].check_manifest(mine)["sha256"] == m["sha256"]
    other_budget = arguments(tmp_path / "mine")
    other_budget.train_tokens = 20001
    for prepare in (P.prepare, ref["run_40b"].prepare):
        with pytest.raises(ValueError):
            prepare(other_budget)


# ------------------------------------------------------------------------------------------- prompt suites, interactive loop
SUITES = [
    [{"prompt": "one"}, {"prompt": "two", "id": "b", "system": "Be brief."}], {"prompts": [{"prompt": "x", "id": 4}, {"prompt": "y", "id": "4"}]},
    {"prompts": [{"prompt": "x", "note": "kept"}]}, [{"prompt": "a", "id": "1"}, {"prompt": "b"}],
    # refused by both
    [], {}, {"prompts": []}, {"prompts": "x"}, "text", 5, [{"prompt": ""}], [{"prompt": "  \n"}], [{"prompt": 3}], ["bare"], [{"question": "x"}],
    [{"prompt": "a", "id": "k"}, {"prompt": "b", "id": "k"}], [{"prompt": "a", "id": 1.5}], [{"prompt": "a", "id": None}], [{"prompt": "a", "id": ["l"]}],
    [{"prompt": "a"}, {"prompt": "b", "id": "0"}],
]


@pytest.mark.parametrize("document", SUITES, ids=[str(i) for i in range(len(SUITES))])
def test_prompt_suites_are_read_alike(tmp_path, document):
    import json
    from warpstate_ai_b200.serve import posttrain_chat as PC
    if not (REF / "ops" / "posttrain_chat.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    with reference_import_path():
        theirs = importlib.import_module("ops.posttrain_chat")
    path = tmp_path / "suite.json"
    path.write_text(json.dumps(document))
    verdicts = []
    for read in (lambda p: PC.PromptSuite.read(p).rows, theirs.read_prompts):
        try:
            verdicts.append(read(path))
        except ValueError:
            verdicts.append("refused")
    assert verdicts[0] == verdicts[1]


def test_interactive_conversations_ask_the_model_the_same_things(monkeypatch, capsys):
    """The same typed lines (cancellations, blank lines, a prompt that is too long, a blank reply, /reset, /quit and the
    end of input among them) lead both interactive loops to the same sequence of model calls."""
    import builtins
    from warpstate_ai_b200.serve import posttrain_chat as PC
    if not (REF / "ops" / "posttrain_chat.py").exists():
        pytest.skip("reference not installed under baseline/_ref")
    with reference_import_path():
        theirs = importlib.import_module("ops.posttrain_chat")
    typed = ["hello", KeyboardInterrupt, "", "interrupt me", "too long", "say nothing", "  again  ", "/reset", "fresh", "more",
             "/exit", "unreachable"]
    transcripts = []
    for side in ("mine", "theirs", "mine-eof", "theirs-eof"):
        asked = []

        def answer(messages, seed):
            asked.append(([dict(m) for m in messages], seed))
            text = messages[-1]["content"]
            if text == "interrupt me":
                raise KeyboardInterrupt
            if text == "too long":
                raise ValueError("the context limit is 2048")
            return {"response": "   " if text == "say nothing" else f"reply to {text}"}

        script = iter(typed[:3] if side.endswith("eof") else typed)

        def fake_input(prompt="", script=script):
            item = next(script, EOFError)
            if isinstance(item, type) and issubclass(item, BaseException):
                raise item
            return item
        monkeypatch.setattr(builtins, "input", fake_input)
        if side.startswith("mine"):
            assert PC.Conversation(answer, "Be kind.", seed=3).loop() == 0
        else:
            assert theirs.interactive_chat(lambda conversation, seed: answer(conversation, seed),
                                           lambda prompt: PC.conversation(prompt, "Be kind."), seed=3) == 0
        transcripts.append(asked)
        shown = capsys.readouterr().out
        assert shown.count("Cancelled.") == (1 if side.endswith("eof") else 2)
    assert transcripts[0] == transcripts[1] and len(transcripts[0]) == 7
    assert transcripts[2] == transcripts[3] and len(transcripts[2]) == 1


def test_a_reference_run_resumes_here_as_an_execution_change(ref, monkeypatch):
    """The signature the reference stores for a command line, against the one this framework computes for the same
    command line: same objective, same schedule, same data; what differs is execution (kernels, gradient path, bucket
    size), so its checkpoint resumes here with ``--reconfigure`` and is refused without -- and a changed objective is
    refused either way."""
    import contextlib
    import io
    from warpstate_ai_b200.train import pretrain as T
    from warpstate_ai_b200.train import signature as S
    for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(name, raising=False)
    manifest = {"signature": {"recipe": 1, "train_tokens": 10 ** 9}, "sha256": {"train.bin": "a" * 64}, "complete": True}
    for argv in ([], ["--micro-batch", "4", "--grad-accum", "8"], ["--bf16-residuals", "--no-activation-checkpointing", "--lr", "2e-4", "--min-lr", "2e-5"],
                 ["--compile-core", "--loss-mode", "full", "--gradient-mode", "compiled-autograd", "--ddp-bucket-cap-mb", "64"]):
        monkeypatch.setattr(sys, "argv", ["run_40b.py", *argv])
        with contextlib.redirect_stderr(io.StringIO()):
            theirs, mine = ref["run_40b"].arguments(), T.arguments(list(argv))
        stored, fresh = ref["run_40b"].train_signature(theirs, manifest), S.train_signature(mine, manifest)
        assert set(stored["settings"]) <= set(fresh["settings"])
        differing = {k for k in stored["settings"] if stored["settings"][k] != fresh["settings"][k]}
        assert differing <= {"ddp_bucket_cap_mb"} and differing <= S.EXECUTION_KEYS
        assert {k: fresh["settings"][k] for k in S.OBJECTIVE_KEYS} == {k: stored["settings"][k] for k in S.OBJECTIVE_KEYS}
        assert S.check_resume_signature(stored, fresh, reconfigure=True) is True
        with pytest.raises(ValueError, match="--reconfigure"):
            S.check_resume_signature(stored, fresh, reconfigure=False)
        for key, value in (("lr", 9e-4), ("seed", 3), ("train_tokens", 5), ("seq_len", 4096)):
            changed = {"settings": dict(fresh["settings"], **{key: value}), "data": fresh["data"]}
            with pytest.raises(ValueError, match="objective and global tokens per update must stay fixed"):
                S.check_resume_signature(stored, changed, reconfigure=True)
        other_corpus = {"settings": fresh["settings"], "data": dict(manifest, sha256={"train.bin": "b" * 64})}
        with pytest.raises(ValueError):
            S.check_resume_signature(stored, other_corpus, reconfigure=True)
