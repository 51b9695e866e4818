"""Conversation and preference-pair rendering, masks, collation and per-rank batching (`data/sft.py`, `data/dpo.py`).

Formats as in the reference (ops/posttrain_data.py:24-71, ops/dpo_data.py:13-35, posttrain.py:159-189, 468-474).  A
character-level stand-in tokenizer makes every expected token sequence readable; one case uses the real model file.
"""
from pathlib import Path

import pytest
import torch

from warpstate_ai_b200.data import dpo as DD
from warpstate_ai_b200.data import sft as SD

TOK = Path(__file__).resolve().parents[1] / "tokenizer.model"


class CharTokenizer:
    """One token per character (code point + 3); 1 = BOS, 2 = EOS."""

    def __init__(self, bos=1, eos=2, vocab=400):
        self._bos, self._eos, self._vocab = bos, eos, vocab

    def vocab_size(self):
        return self._vocab

    def bos_id(self):
        return self._bos

    def eos_id(self):
        return self._eos

    def encode(self, text, out_type=int):
        return [ord(c) + 3 for c in text]


def text_of(tokens):
    return "".join("<s>" if t == 1 else "</s>" if t == 2 else chr(t - 3) for t in tokens)


CONVERSATION = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "2+2?"},
                {"role": "assistant", "content": "4"}, {"role": "user", "content": "3+3?"},
                {"role": "assistant", "content": "6"}]


def test_sft_rendering_segments_roles_and_supervises_every_assistant_turn():
    record = SD.encode_messages(CONVERSATION, CharTokenizer())
    ids, labels = record["input_ids"], record["labels"]
    assert text_of(ids) == ("<s><|system|>\nBe brief.\n<|user|>\n2+2?\n<|assistant|>\n4</s>\n<|user|>\n3+3?\n"
                            "<|assistant|>\n6</s>\n")
    scored = [(i, t) for i, (t, l) in enumerate(zip(ids, labels)) if l != SD.IGNORE_INDEX]
    assert text_of([t for _, t in scored]) == "4</s>6</s>"
    assert all(labels[i] == ids[i] for i, _ in scored)
    assert SD.supervised_count(record) == 4
    without_bos = SD.encode_messages(CONVERSATION, CharTokenizer(bos=-1))
    assert without_bos["input_ids"] == ids[1:] and without_bos["labels"] == labels[1:]


def test_preference_branches_share_the_prompt_and_score_only_the_final_response():
    row = {"prompt": CONVERSATION[:4], "chosen": [{"role": "assistant", "content": "6"}],
           "rejected": [{"role": "assistant", "content": "seven"}]}
    pair = DD.encode_pair(row, CharTokenizer(), None)
    chosen, rejected = pair["chosen"], pair["rejected"]
    # the chosen branch is token for token the SFT rendering of the whole conversation ...
    assert chosen["input_ids"] == SD.encode_messages(CONVERSATION, CharTokenizer())["input_ids"]
    # ... but the earlier assistant turn belongs to the prompt and is not scored
    assert text_of([t for t, l in zip(chosen["input_ids"], chosen["labels"]) if l != SD.IGNORE_INDEX]) == "6</s>"
    assert text_of([t for t, l in zip(rejected["input_ids"], rejected["labels"]) if l != SD.IGNORE_INDEX]) == "seven</s>"
    prefix = len(text_of(chosen["input_ids"]).split("6</s>")[0].replace("<s>", "\x01").replace("</s>", "\x02"))
    assert chosen["input_ids"][:prefix] == rejected["input_ids"][:prefix]
    assert all(l == SD.IGNORE_INDEX for l in chosen["labels"][:prefix] + rejected["labels"][:prefix])
    assert chosen["labels"][-1] == SD.IGNORE_INDEX                                  # the closing newline is not scored
    assert DD.pair_targets(pair) == 2 + 6 and DD.pair_tokens(pair) == len(chosen["input_ids"]) + len(rejected["input_ids"]) - 2


@pytest.mark.parametrize("change, message", [
    (dict(prompt=[]), "shared prompt"),
    (dict(prompt=CONVERSATION[:3]), "shared prompt"),                               # ends with an assistant turn
    (dict(prompt="2+2?"), "shared prompt"),
    (dict(chosen=[]), "'chosen' must be exactly one assistant message"),
    (dict(chosen=[{"role": "assistant", "content": "4"}] * 2), "'chosen' must be exactly one"),
    (dict(rejected=[{"role": "user", "content": "5"}]), "'rejected' must be exactly one"),
    (dict(rejected=[{"role": "assistant", "content": "4"}]), "render to the same tokens"),
    (dict(rejected=[{"role": "assistant", "content": "   "}]), "nonempty text content"),
    (dict(prompt=[{"role": "narrator", "content": "x"}, {"role": "user", "content": "y"}]), "Unsupported conversation role"),
    (dict(prompt=[{"role": "user", "content": "y", "tool_calls": [{"name": "f"}]}]), "tool calls"),
])
def test_malformed_pairs_are_refused(change, message):
    row = {"prompt": CONVERSATION[:2], "chosen": [{"role": "assistant", "content": "4"}],
           "rejected": [{"role": "assistant", "content": "5"}]}
    row.update(change)
    with pytest.raises(ValueError, match=message):
        DD.encode_pair(row, CharTokenizer(), None)


def test_length_limits_never_truncate():
    row = {"prompt": CONVERSATION[:2], "chosen": [{"role": "assistant", "content": "4"}],
           "rejected": [{"role": "assistant", "content": "a much longer answer than the other one"}]}
    longest = len(DD.encode_pair(row, CharTokenizer(), None)["rejected"]["input_ids"])
    assert DD.encode_pair(row, CharTokenizer(), longest)["rejected"]["input_ids"][-1] == ord("\n") + 3
    with pytest.raises(ValueError, match=f"has {longest} tokens, exceeds max_length={longest - 1}"):
        DD.encode_pair(row, CharTokenizer(), longest - 1)
    with pytest.raises(ValueError, match="integer >= 2"):
        SD.encode_messages(CONVERSATION, CharTokenizer(), max_length=1)
    with pytest.raises(ValueError, match="real EOS"):
        SD.encode_messages(CONVERSATION, CharTokenizer(eos=-1))
    with pytest.raises(ValueError, match="real EOS"):
        DD.encode_pair(row, CharTokenizer(eos=500), None)
    with pytest.raises(ValueError, match="nonempty list"):
        SD.encode_messages([], CharTokenizer())
    with pytest.raises(ValueError, match="no supervised"):
        SD.encode_messages(CONVERSATION[:2], CharTokenizer())


def test_the_real_tokenizer_is_applied_segment_by_segment():
    import sentencepiece as spm
    sp = spm.SentencePieceProcessor(model_file=str(TOK))
    messages = [{"role": "user", "content": "Name a colour."}, {"role": "assistant", "content": "Blue."}]
    record = SD.encode_messages(messages, sp)
    pieces = [[sp.bos_id()]] if 0 <= sp.bos_id() < sp.vocab_size() else []
    for m in messages:
        pieces += [sp.encode(f"<|{m['role']}|>\n", out_type=int), sp.encode(m["content"], out_type=int)]
        if m["role"] == "assistant":
            pieces.append([sp.eos_id()])
        pieces.append(sp.encode("\n", out_type=int))
    assert record["input_ids"] == [t for piece in pieces for t in piece]
    scored = [t for t, l in zip(record["input_ids"], record["labels"]) if l != SD.IGNORE_INDEX]
    assert scored[-1] == sp.eos_id() and sp.decode(scored[:-1]) == "Blue."
    pair = DD.encode_pair({"prompt": messages[:1], "chosen": messages[1:], "rejected": [{"role": "assistant", "content": "No."}]},
                          sp, 64)
    assert pair["chosen"] == record                                                  # single-turn: same ids, same mask


def test_pairs_collate_interleaved_with_a_mask_of_real_pairs():
    a = {"chosen": {"input_ids": [1, 9, 8, 7], "labels": [-100, -100, 8, 7]},
         "rejected": {"input_ids": [1, 9, 5], "labels": [-100, -100, 5]}}
    b = {"chosen": {"input_ids": [1, 4, 4], "labels": [-100, -100, 4]},
         "rejected": {"input_ids": [1, 4, 3, 2, 6], "labels": [-100, -100, 3, 2, -100]}}
    x, y, real = DD.collate_pairs([a, None, b], 5, pad_id=0)
    assert x.shape == (6, 5) and real.tolist() == [True, False, True] and real.dtype == torch.bool
    assert x.tolist() == [[1, 9, 8, 0, 0], [1, 9, 0, 0, 0], [0] * 5, [0] * 5, [1, 4, 0, 0, 0], [1, 4, 3, 2, 0]]
    assert y.tolist() == [[-100, 8, 7, -100, -100], [-100, 5, -100, -100, -100], [-100] * 5, [-100] * 5,
                          [-100, 4, -100, -100, -100], [-100, 3, 2, -100, -100]]
    with pytest.raises(ValueError, match="Invalid encoded record length"):
        DD.collate_pairs([b], 4, pad_id=0)                                           # five tokens do not fit four
    with pytest.raises(ValueError, match="Invalid encoded record length"):
        SD.collate([{"input_ids": [1], "labels": [-100]}], 4, 0)
    with pytest.raises(ValueError, match="Invalid encoded record length"):
        SD.collate([{"input_ids": [1, 2], "labels": [-100]}], 4, 0)


@pytest.mark.parametrize("world", [1, 2, 3])
def test_ranks_split_an_update_without_overlap_and_pad_with_inactive_rows(world):
    records = [f"r{i}" for i in range(10)]
    mb, accum = 2, 2
    indices, cursor = SD.update_indices(10, seed=5, cursor=0, epochs=1, global_batch=mb * accum * world)
    per_rank = [SD.rank_microbatches(indices, records, mb, accum, world, rank) for rank in range(world)]
    assert all(len(steps) == accum and all(len(rows) == mb for rows in steps) for steps in per_rank)
    real = [row for steps in per_rank for rows in steps for row in rows if row is not None]
    assert sorted(real) == sorted(records[i] for i in indices) and len(set(real)) == len(real)
    assert cursor == len(indices) == min(10, mb * accum * world)
    # the last, short update of an epoch: the ranks at the end get rows of None and still take every step
    tail, _ = SD.update_indices(10, seed=5, cursor=8, epochs=1, global_batch=mb * accum * world)
    assert len(tail) == 2
    per_rank = [SD.rank_microbatches(tail, records, mb, accum, world, rank) for rank in range(world)]
    assert per_rank[0][0] == [records[tail[0]], records[tail[1]]]
    assert all(rows == [None, None] for steps in per_rank[1:] for rows in steps)
    assert per_rank[0][1] == [None, None]


def test_epoch_orders_are_seeded_permutations():
    first, second = SD.epoch_order(50, 9, 0), SD.epoch_order(50, 9, 1)
    assert sorted(first) == sorted(second) == list(range(50)) and first != second
    assert SD.epoch_order(50, 9, 0) == first and SD.epoch_order(50, 10, 0) == second       # seed + epoch picks the order
    assert SD.update_indices(50, 9, 100, 2, 8) == ([], 100)                                 # both epochs consumed
    assert SD.update_indices(50, 9, 48, 2, 8) == (list(first[48:50]), 50)
    assert SD.update_indices(50, 9, 50, 2, 8) == (list(second[:8]), 58)
