"""Chat with SFT / DPO exports (`serve/posttrain_chat.py`; behaviour of the reference's ops/posttrain_chat.py:35-238):
prompt rendering, one reply, batched greedy decode, prompt suites and the interactive conversation, against a scripted
engine and a character tokenizer."""
import builtins
import json

import pytest
import torch

from warpstate_ai_b200.data import sft as SD
from warpstate_ai_b200.serve import posttrain_chat as PC

EOS = 2


class CharTokenizer:
    def __init__(self, bos=1, eos=EOS, vocab=400):
        self._bos, self._eos, self._vocab = bos, eos, vocab

    def vocab_size(self):
        return self._vocab

    def bos_id(self):
        return self._bos

    def eos_id(self):
        return self._eos

    def encode(self, text, out_type=int):
        return [ord(c) + 3 for c in text]

    def decode(self, ids):
        return "".join(chr(t - 3) for t in ids)


def text_of(tokens):
    return "".join("<s>" if t == 1 else "</s>" if t == 2 else chr(t - 3) for t in tokens)


class ScriptedEngine:
    """Favours the characters of ``reply`` one after another, then end-of-sequence."""
    device = torch.device("cpu")
    dtype = torch.float32

    def __init__(self, reply, vocab=400):
        self.targets = [ord(c) + 3 for c in reply] + [EOS]
        self.vocab, self.position, self.prefilled, self.stepped = vocab, 0, None, []

    def _logits(self, rows=1):
        logits = torch.zeros(rows, self.vocab)
        logits[:, self.targets[min(self.position, len(self.targets) - 1)]] = 9.0
        return logits

    def prefill(self, ids):
        self.prefilled, self.position = ids.clone(), 0
        return self._logits(ids.shape[0])

    def step(self, token):
        self.stepped.append(token.tolist())
        self.position += 1
        return self._logits(token.shape[0])


HISTORY = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "2+2?"},
           {"role": "assistant", "content": "4"}, {"role": "user", "content": "3+3?"}]


# ------------------------------------------------------------------------------------------- prompt
def test_prompt_is_the_training_rendering_with_the_assistant_header_left_open():
    tok = CharTokenizer()
    ids = PC.encode_prompt(HISTORY, tok)
    assert text_of(ids) == "<s><|system|>\nBe brief.\n<|user|>\n2+2?\n<|assistant|>\n4</s>\n<|user|>\n3+3?\n<|assistant|>\n"
    # token for token the prefix of what training saw for the same conversation plus an answer
    trained = SD.encode_messages(HISTORY + [{"role": "assistant", "content": "6"}], tok)["input_ids"]
    assert trained[:len(ids)] == ids and text_of(trained[len(ids):]) == "6</s>\n"
    assert text_of(PC.encode_prompt(HISTORY[1:2], CharTokenizer(bos=-1))) == "<|user|>\n2+2?\n<|assistant|>\n"


@pytest.mark.parametrize("messages, complaint", [
    ([], "at least one message"), ("hello", "at least one message"),
    (HISTORY[:3], "must end with a user or tool message"),
    ([{"role": "user", "content": " "}], "nonempty text content"),
    ([{"role": "critic", "content": "x"}, {"role": "user", "content": "y"}], "Unsupported conversation role"),
    ([{"role": "user", "content": "y", "tool_calls": [1]}], "tool calls"),
])
def test_conversations_that_cannot_be_continued_are_refused(messages, complaint):
    with pytest.raises(ValueError, match=complaint):
        PC.encode_prompt(messages, CharTokenizer())
    with pytest.raises(ValueError, match="no end-of-sequence token"):
        PC.PromptEncoder(CharTokenizer(eos=-1))


# ------------------------------------------------------------------------------------------- one reply
def test_reply_stops_at_end_of_sequence_and_leaves_it_out():
    engine = ScriptedEngine("six")
    seen = []
    record = PC.generate(engine, CharTokenizer(), HISTORY, max_new_tokens=10, max_context=200, on_token=seen.append)
    assert record["response"] == "six" and record["token_ids"] == [ord(c) + 3 for c in "six"]
    assert record["stop_reason"] == "eos" and record["generated_tokens"] == 3 and record["sampled_tokens"] == 4
    assert record["prompt_tokens"] == engine.prefilled.shape[1] == len(PC.encode_prompt(HISTORY, CharTokenizer()))
    assert seen == [tuple(record["token_ids"][:n]) for n in (1, 2, 3)]
    assert engine.stepped == [[t] for t in record["token_ids"]]
    assert record["first_token_seconds"] <= record["elapsed_seconds"] and record["tokens_per_second"] > 0
    assert set(record) == {"response", "token_ids", "prompt_tokens", "generated_tokens", "sampled_tokens", "elapsed_seconds",
                           "first_token_seconds", "tokens_per_second", "stop_reason", "temperature", "seed"}


def test_length_and_context_limits_are_told_apart():
    tok = CharTokenizer()
    prompt_tokens = len(PC.encode_prompt(HISTORY, tok))
    by_length = PC.generate(ScriptedEngine("abcdefgh"), tok, HISTORY, max_new_tokens=3, max_context=prompt_tokens + 50)
    assert (by_length["response"], by_length["stop_reason"]) == ("abc", "length")
    engine = ScriptedEngine("abcdefgh")
    by_context = PC.generate(engine, tok, HISTORY, max_new_tokens=6, max_context=prompt_tokens + 2)
    assert (by_context["response"], by_context["stop_reason"]) == ("ab", "context_limit")
    assert len(engine.stepped) == 1                                                    # no step after the last token
    with pytest.raises(ValueError, match=f"the prompt alone is {prompt_tokens} tokens; the context limit is {prompt_tokens}"):
        PC.generate(ScriptedEngine("a"), tok, HISTORY, max_context=prompt_tokens)
    for bad in (dict(max_new_tokens=0), dict(max_context=1), dict(seed=-1), dict(max_new_tokens=2.0)):
        with pytest.raises(ValueError, match="must be an integer >="):
            PC.generate(ScriptedEngine("a"), tok, HISTORY, **bad)
    with pytest.raises(ValueError, match="Invalid sampling settings"):
        PC.generate(ScriptedEngine("a"), tok, HISTORY, temperature=-1.0)


def test_sampled_replies_depend_on_the_seed_alone():
    class FlatEngine(ScriptedEngine):
        def _logits(self, rows=1):
            logits = torch.full((rows, self.vocab), -30.0)
            logits[:, [ord(c) + 3 for c in "abcd"]] = 0.0
            return logits

    tok = CharTokenizer()
    state = torch.get_rng_state()
    one = PC.generate(FlatEngine(""), tok, HISTORY, max_new_tokens=12, temperature=1.0, seed=5)["response"]
    two = PC.generate(FlatEngine(""), tok, HISTORY, max_new_tokens=12, temperature=1.0, seed=5)["response"]
    others = {PC.generate(FlatEngine(""), tok, HISTORY, max_new_tokens=12, temperature=1.0, seed=s)["response"] for s in range(6, 12)}
    assert one == two and set(one) <= set("abcd") and len(others | {one}) > 1
    assert torch.equal(torch.get_rng_state(), state)


# ------------------------------------------------------------------------------------------- batched greedy decode
def test_batched_greedy_decode_on_the_host_path():
    engine = ScriptedEngine("wxyz")
    prompts = torch.randint(3, 100, (3, 5))
    out = PC.generate_batch(engine, prompts, max_new_tokens=4)
    assert out["tokens"].shape == (3, 4) and out["tokens"][1].tolist() == [ord(c) + 3 for c in "wxyz"]
    assert len(out["latencies"]) == 4 and out["timing"] == "host clock, one synchronisation per token"
    assert out["p50_latency_seconds"] == sorted(out["latencies"])[2]
    assert out["tokens_per_second"] == pytest.approx(3 * 4 / out["decode_seconds"])
    assert torch.equal(engine.prefilled, prompts) and len(engine.stepped) == 4


# ------------------------------------------------------------------------------------------- suites
def test_suite_files_keep_their_ids_and_ignore_other_fields(tmp_path):
    path = tmp_path / "suite.json"
    path.write_text(json.dumps({"prompts": [{"id": "math-1", "prompt": "2+2?", "rubric": "says 4", "system": "Terse."},
                                            {"prompt": "Name a colour."}, {"id": 7, "prompt": "Why?"}]}))
    suite = PC.PromptSuite.read(path)
    calls = []

    def answer(messages, seed):
        calls.append((messages, seed))
        return {"response": f"r{seed}", "generated_tokens": 1}

    out = tmp_path / "reports" / "run.json"
    report = suite.run(answer, {"format": PC.REPORT_FORMAT, "snapshot": "x"}, "Default system.", 40, out)
    assert [r["id"] for r in report["results"]] == ["math-1", "1", 7] and report["complete"] is True
    assert [r["system"] for r in report["results"]] == ["Terse.", "Default system.", "Default system."]
    assert all("rubric" not in r for r in report["results"]) and [r["response"] for r in report["results"]] == ["r40", "r41", "r42"]
    assert calls[0] == ([{"role": "system", "content": "Terse."}, {"role": "user", "content": "2+2?"}], 40)
    assert json.loads(out.read_text()) == json.loads(json.dumps(report))
    bare = tmp_path / "bare.json"
    bare.write_text(json.dumps([{"prompt": "only a list"}]))
    assert PC.PromptSuite.read(bare).rows == [{"prompt": "only a list"}]
    assert PC.PromptSuite.single("hi").rows == [{"id": "prompt", "prompt": "hi"}]
    assert PC.conversation("hi", "  ") == [{"role": "user", "content": "hi"}]          # a blank system prompt is left out


@pytest.mark.parametrize("document, complaint", [
    ({}, "non-empty list"), ([], "non-empty list"), ({"prompts": "x"}, "non-empty list"),
    ([{"prompt": " "}], "row 0 has no prompt text"), (["text"], "row 0 has no prompt text"),
    ([{"id": "a", "prompt": "x"}, {"id": "a", "prompt": "y"}], "ids must be distinct"),
    ([{"prompt": "x"}, {"id": "0", "prompt": "y"}], "ids must be distinct"),          # collides with the position default
    ([{"id": 1.5, "prompt": "x"}], "ids must be distinct strings or integers"),
])
def test_malformed_suites_are_refused(tmp_path, document, complaint):
    path = tmp_path / "suite.json"
    path.write_text(json.dumps(document))
    with pytest.raises(ValueError, match=complaint):
        PC.PromptSuite.read(path)
    with pytest.raises(ValueError, match="the prompt is empty"):
        PC.PromptSuite.single("  ")


def test_an_interrupted_suite_leaves_a_valid_incomplete_report(tmp_path):
    suite = PC.PromptSuite([{"prompt": "a"}, {"prompt": "b"}, {"prompt": "c"}])

    def answer(messages, seed):
        if messages[-1]["content"] == "c":
            raise KeyboardInterrupt
        return {"response": "ok"}

    out = tmp_path / "run.json"
    with pytest.raises(KeyboardInterrupt):
        suite.run(answer, {"format": PC.REPORT_FORMAT}, "", 0, out)
    report = json.loads(out.read_text())
    assert report["complete"] is False and [r["prompt"] for r in report["results"]] == ["a", "b"]


# ------------------------------------------------------------------------------------------- conversation
def feed_input(monkeypatch, script):
    script = iter(script)

    def fake_input(prompt=""):
        item = next(script, EOFError)
        if isinstance(item, type) and issubclass(item, BaseException):
            raise item
        return item
    monkeypatch.setattr(builtins, "input", fake_input)


def test_conversation_keeps_finished_turns_through_cancellations_and_errors(monkeypatch, capsys):
    asked = []

    def answer(messages, seed):
        asked.append([dict(m) for m in messages])
        text = messages[-1]["content"]
        if text == "interrupt me":
            raise KeyboardInterrupt
        if text == "too long":
            raise ValueError("the prompt alone is 9999 tokens; the context limit is 2048")
        return {"response": "   " if text == "say nothing" else f"reply to {text}"}

    talk = PC.Conversation(answer, "Be kind.", seed=3)
    feed_input(monkeypatch, ["hello", KeyboardInterrupt, "", "interrupt me", "too long", "say nothing", "again", "/reset",
                             "fresh", "/quit", "unreachable"])
    assert talk.loop() == 0
    out = capsys.readouterr().out
    assert out.count("Cancelled.") == 2 and "the context limit is 2048; /reset starts a new conversation." in out
    first = [{"role": "system", "content": "Be kind."}, {"role": "user", "content": "hello"}]
    kept = first + [{"role": "assistant", "content": "reply to hello"}]
    assert asked[0] == first
    assert asked[1] == kept + [{"role": "user", "content": "interrupt me"}]
    assert asked[2] == kept + [{"role": "user", "content": "too long"}]               # the cancelled turn left no trace
    assert asked[3] == kept + [{"role": "user", "content": "say nothing"}]
    assert asked[4] == kept + [{"role": "user", "content": "again"}]                  # a blank reply is not recorded either
    assert asked[5] == [{"role": "system", "content": "Be kind."}, {"role": "user", "content": "fresh"}]
    assert len(asked) == 6
    feed_input(monkeypatch, [])                                                       # end of input ends the loop too
    assert PC.Conversation(answer, "", 0).loop() == 0


def test_command_line_refuses_bad_combinations_before_loading_anything(tmp_path, capsys):
    snapshot = tmp_path / "export" / "model.pt"
    snapshot.parent.mkdir()
    snapshot.write_bytes(b"")
    existing = tmp_path / "out.json"
    existing.write_text("{}")
    cases = [
        (["--output-json", str(tmp_path / "new.json")], "--output-json needs a prompt or a suite"),
        (["--prompt", "hi", "--output-json", str(existing)], "--output-json needs a prompt or a suite and a new file"),
        (["--prompt", "hi", "--output-json", str(snapshot.parent / "inside.json")], "outside the snapshot directory"),
        (["--prompt", "hi", "--max-new-tokens", "10", "--max-context", "10"], "0 < max-new-tokens < max-context"),
        (["--prompt", "hi", "--temperature", "-2"], "Invalid sampling settings"),
        (["--prompt", "  "], "the prompt is empty"),
        (["--prompt", "hi"], "snapshot.json is missing"),                              # an export without its seal
    ]
    for extra, complaint in cases:
        with pytest.raises(SystemExit) as stop:
            PC.main(["--snapshot", str(snapshot), "--device", "cpu", *extra])
        assert stop.value.code == 2 and complaint in capsys.readouterr().err, extra
