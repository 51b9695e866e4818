"""The base-model probe's generation loop and interactive session (`serve/chat.py`; behaviour of the reference's
chat.py:154-260) against a scripted decode engine: no model is run, so every expected token is stated in the test."""
import builtins
from argparse import Namespace
from types import SimpleNamespace

import pytest
import torch

from warpstate_ai_b200.serve import chat as C

VOCAB = 12
EOS = 2


class WordTokenizer:
    """Tokens 3.. are the words of a tiny vocabulary; 2 ends the sequence."""
    words = ["<unk>", "<s>", "</s>", "a", "b", "c", "d", "e", "f", "g", "h", "i"]

    def eos_id(self):
        return EOS

    def encode(self, text, out_type=int):
        return [self.words.index(w) if w in self.words else 0 for w in text.split()]

    def decode(self, ids):
        return " ".join(self.words[i] for i in ids)


class ScriptedEngine:
    """Returns logits that favour ``script[k]`` at the k-th position after the prompt (then EOS for ever)."""

    def __init__(self, script, runner_up=None):
        self.script, self.runner_up = list(script), runner_up
        self.position = 0
        self.prefilled = None
        self.stepped = []

    def _logits(self):
        want = self.script[self.position] if self.position < len(self.script) else EOS
        logits = torch.full((1, VOCAB), -4.0)
        logits[0, want] = 5.0
        if self.runner_up is not None:
            logits[0, self.runner_up] = 4.0
        return logits

    def prefill(self, ids):
        self.prefilled = ids.clone()
        self.position = 0
        return self._logits()

    def step(self, token):
        self.stepped.append(int(token[0]))
        self.position += 1
        return self._logits()


MODEL = SimpleNamespace(embed=SimpleNamespace(weight=torch.zeros(1)), num_parameters=lambda: 2_005_111_424)


def run(script, prompt="a b", **kw):
    engine = ScriptedEngine(script, kw.pop("runner_up", None))
    settings = dict(max_new_tokens=8, temperature=0.0, max_context=32, repetition_penalty=1.0, no_repeat_ngram_size=0)
    settings.update(kw)
    return list(C.generate(MODEL, WordTokenizer(), prompt, engine=engine, **settings)), engine


def test_reply_ends_at_end_of_sequence_without_yielding_it():
    tokens, engine = run([3, 4, 5, EOS, 6])
    assert tokens == [3, 4, 5]
    assert engine.prefilled.tolist() == [[3, 4]] and engine.stepped == [3, 4, 5]      # every yielded token is fed back once


def test_reply_ends_at_the_length_limit_without_a_wasted_step():
    tokens, engine = run([3, 4, 5, 6, 7, 8], max_new_tokens=4)
    assert tokens == [3, 4, 5, 6] and engine.stepped == [3, 4, 5]                      # no step after the last token


def test_only_the_end_of_a_long_prompt_is_kept():
    prompt = " ".join(["a", "b", "c", "d", "e", "f", "g", "h"])
    _, engine = run([EOS], prompt=prompt, max_new_tokens=3, max_context=8)
    assert engine.prefilled.tolist() == [[6, 7, 8, 9, 10]]                             # 8 - 3 = 5 most recent tokens
    with pytest.raises(ValueError, match="max-new-tokens < max-context"):
        run([EOS], max_new_tokens=8, max_context=8)
    with pytest.raises(ValueError, match="encodes to no tokens"):
        run([EOS], prompt="   ")


def test_the_no_repeat_rule_breaks_a_phrase_loop_with_the_runner_up():
    # the engine insists on "a b a b a b"; with trigrams forbidden, "a b" may not be followed by "a" a second time
    tokens, _ = run([3, 4, 3, 4, 3, 4], runner_up=7, no_repeat_ngram_size=3, max_new_tokens=6)
    assert tokens == [3, 4, 3, 4, 7, 4]
    unprotected, _ = run([3, 4, 3, 4, 3, 4], runner_up=7, max_new_tokens=6)
    assert unprotected == [3, 4, 3, 4, 3, 4]


def test_the_repetition_penalty_counts_the_reply_not_the_prompt():
    # "a" is in the prompt but not yet in the reply: its first use is not penalised; the second one is (5 / 2 < 4)
    tokens, _ = run([3, 3, 3], prompt="a a a", runner_up=7, repetition_penalty=2.0, max_new_tokens=3)
    assert tokens == [3, 7, 3]                                                         # then 7 is penalised too: 4 / 2 < 5 / 2


def test_a_unigram_ban_never_repeats_a_token_and_an_exhausted_vocabulary_ends_the_reply():
    tokens, _ = run([3, 3, 3], no_repeat_ngram_size=1, max_new_tokens=3, runner_up=7)
    assert tokens[:2] == [3, 7] and len(set(tokens)) == len(tokens)
    # twelve tokens in the vocabulary, end-of-sequence among them: a reply can never be longer than eleven
    tokens, _ = run([3] * 20, no_repeat_ngram_size=1, max_new_tokens=20)
    assert len(tokens) <= VOCAB - 1 and len(set(tokens)) == len(tokens)


def test_seeded_sampling_is_reproducible_and_leaves_the_global_generator_alone():
    state = torch.get_rng_state()
    first, _ = run([3, 4, 5, 6, 7], runner_up=8, temperature=1.5, top_k=0, top_p=1.0, seed=11)
    again, _ = run([3, 4, 5, 6, 7], runner_up=8, temperature=1.5, top_k=0, top_p=1.0, seed=11)
    other = [run([3, 4, 5, 6, 7], runner_up=8, temperature=1.5, top_k=0, top_p=1.0, seed=s)[0] for s in range(12, 20)]
    assert first == again and any(o != first for o in other)
    assert torch.equal(torch.get_rng_state(), state)


@pytest.mark.parametrize("settings", [dict(repetition_penalty=0.5), dict(no_repeat_ngram_size=-1), dict(top_p=0.0),
                                      dict(temperature=-1.0)])
def test_invalid_settings_are_refused_before_the_model_is_used(settings):
    engine = ScriptedEngine([3])
    with pytest.raises(ValueError, match="Invalid sampling settings"):
        list(C.generate(MODEL, WordTokenizer(), "a", engine=engine, max_new_tokens=2, max_context=8, **settings))
    assert engine.prefilled is None


# ------------------------------------------------------------------------------------------- printing
def test_printer_holds_back_incomplete_characters(capsys):
    class ByteTokenizer:
        pieces = {1: b"caf", 2: b"\xc3", 3: b"\xa9", 4: b"!"}

        def decode(self, ids):
            return b"".join(self.pieces[i] for i in ids).decode("utf-8", errors="replace")

    printer = C.ReplyPrinter(ByteTokenizer())
    printer.feed(1)
    assert capsys.readouterr().out == "caf"
    printer.feed(2)                                                                   # first byte of a two-byte character
    assert capsys.readouterr().out == ""
    printer.feed(3)
    assert capsys.readouterr().out == "é"
    printer.feed(4)
    assert printer.finish() == "café!"
    tail = capsys.readouterr().out
    assert tail.startswith("!\n[4 tokens;") and "TTFT" in tail and "tok/s]" in tail
    empty = C.ReplyPrinter(ByteTokenizer())
    assert empty.finish() == "" and "[0 tokens;" in capsys.readouterr().out and empty.first_token_at is None


# ------------------------------------------------------------------------------------------- session
def session_args(**changes):
    values = dict(raw=False, device="cpu", max_new_tokens=4, temperature=0.0, top_k=0, top_p=1.0, seed=1, max_context=64,
                  repetition_penalty=1.0, no_repeat_ngram_size=0)
    values.update(changes)
    return Namespace(**values)


@pytest.fixture()
def scripted_reply(monkeypatch):
    prompts = []

    def fake_reply(model, sp, prompt, args, engine=None):
        prompts.append(prompt)
        if prompt.endswith("Question: boom\nAnswer:"):             # the user presses Ctrl-C during this reply
            raise KeyboardInterrupt
        return f"answer{len(prompts)}"

    monkeypatch.setattr(C, "reply", fake_reply)
    return prompts


def feed_input(monkeypatch, lines):
    lines = iter(lines)

    def fake_input(prompt=""):
        try:
            return next(lines)
        except StopIteration:
            raise EOFError
    monkeypatch.setattr(builtins, "input", fake_input)


def test_question_answer_framing_accumulates_and_commands_reset_it(monkeypatch, capsys, scripted_reply):
    session = C.ChatSession(MODEL, WordTokenizer(), {"step": 7, "tokens_seen": 112}, session_args())
    feed_input(monkeypatch, ["first", "", "second", "/new", "third", "/raw", "plain text", "/chat", "/info", "/help",
                             "/unknown command", "/exit", "never reached"])
    session.banner()
    session.loop()
    assert scripted_reply == [
        "Question: first\nAnswer:",
        "Question: first\nAnswer: answer1\n\nQuestion: second\nAnswer:",
        "Question: third\nAnswer:",                                                   # /new forgot the conversation
        "plain text",                                                                 # raw mode: no framing
        "Question: /unknown command\nAnswer:",                                        # not a command: asked like any text
    ]
    out = capsys.readouterr().out
    assert "WarpState 2.005B | cpu | step 7 | 112 training tokens" in out and "without instruction tuning" in out
    assert out.count("Context cleared.") == 3 and "Mode: raw completion" in out and "Mode: Q/A probe" in out
    assert '"tokens_seen": 112' in out and "/info snapshot metadata" in out
    assert session.raw is False


def test_ctrl_c_cancels_the_reply_and_keeps_the_finished_turns(monkeypatch, capsys, scripted_reply):
    session = C.ChatSession(MODEL, WordTokenizer(), {"step": 1, "tokens_seen": 1}, session_args())
    feed_input(monkeypatch, ["first", "boom", "after"])
    session.loop()                                                                    # ends at end of input, not by the interrupt
    assert "Reply cancelled" in capsys.readouterr().out
    assert scripted_reply[-1] == "Question: first\nAnswer: answer1\n\nQuestion: after\nAnswer:"   # the cancelled turn left no trace
    assert session.transcript.endswith("answer3\n\n")


def test_command_line_checks_come_before_any_file_is_opened(capsys):
    for argv, message in ((["--threads", "0"], "--threads must be at least 1"),
                          (["--max-new-tokens", "64", "--max-context", "64"], "--max-new-tokens < --max-context"),
                          (["--repetition-penalty", "0.8"], "repetition penalty must be finite and >= 1"),
                          (["--prompt", "  "], "--prompt is empty")):
        with pytest.raises(SystemExit) as stop:
            C.main(argv + ["--checkpoint", "/nonexistent/latest.pt"])
        assert stop.value.code == 2 and message in capsys.readouterr().err
