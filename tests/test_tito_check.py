"""Decode + re-encode consistency of multi-turn token streams, with a toy longest-match tokenizer."""

import math
from types import SimpleNamespace

import torch

from research_b200.training.tito_check import (check_rollout, find_retokenization_mismatches, forward_logprob_fn,
                                               segments_of_sample)


class LongestMatch:
    """Greedy longest-match over a fixed vocabulary: 'ab' always wins over 'a' + 'b' when encoding text."""

    def __init__(self, vocab):
        self.vocab = list(vocab)
        self.ids = {p: i for i, p in enumerate(self.vocab)}

    def decode(self, ids):
        return "".join(self.vocab[i] for i in ids)

    def encode(self, text, add_special_tokens=False):
        out, i = [], 0
        while i < len(text):
            piece = max((p for p in self.vocab if text.startswith(p, i)), key=len)
            out.append(self.ids[piece])
            i += len(piece)
        return out


TOK = LongestMatch(["a", "b", "c", "ab", "bc", "abc", " ", "1", "2", "12"])
A, B, C, AB, BC, ABC, SP, ONE, TWO, TWELVE = range(10)


def test_stable_stream_has_no_mismatch():
    ids = [AB, SP, C, SP, TWELVE]
    found, re_ids = find_retokenization_mismatches(ids, TOK)
    assert found == [] and re_ids == ids
    rep = check_rollout([ids[:2], ids[2:]], TOK)
    assert rep.ok and "unchanged" in rep.summary()


def test_merge_across_a_seam_is_found_and_scored():
    # turn 1 ends with "a"; the inserted tool text starts with "b": re-encoding merges them into "ab"
    turn1, tool, turn2 = [C, SP, A], [B, SP, ONE], [TWO, SP, C]
    found, re_ids = find_retokenization_mismatches(turn1 + tool + turn2, TOK)
    assert [(m.start, m.original, m.retokenized, m.text) for m in found] == [(2, (A, B), (AB,), "ab"), (5, (ONE, TWO), (TWELVE,), "12")]
    assert re_ids == [C, SP, AB, SP, TWELVE, SP, C]

    table = {AB: math.log(1e-9), TWELVE: math.log(0.2)}
    seen = []

    def lp(prefix, token):
        seen.append((tuple(prefix), token))
        return table[token]

    rep = check_rollout([turn1, tool, turn2], TOK, lp, threshold=-10.0, smoking_gun=-15.0)
    assert not rep.ok and rep.num_tokens == 9 and rep.num_retokenized == 7
    m1, m2 = rep.mismatches
    assert m1.seams == (3,) and m2.seams == (6,) and len(rep.at_seams) == 2
    assert seen[0] == ((C, SP), AB) and seen[1] == ((C, SP, A, B, SP), TWELVE)         # scored against the true prefix
    assert [m.start for m in rep.suspicious] == [2] and [m.start for m in rep.smoking_guns] == [2]
    text = rep.summary()
    assert "2 at segment seams" in text and "(seam)" in text and "'ab'" in text


def test_split_inside_a_generation_is_not_a_seam_and_three_way_merge():
    # the sampler emitted "a","b","c" one by one inside a single turn; the text re-encodes to one token
    rep = check_rollout([[SP, A, B, C, SP], [ONE]], TOK)
    (m,) = rep.mismatches
    assert m.original == (A, B, C) and m.retokenized == (ABC,) and m.start == 1 and not m.at_seam and m.logprobs == ()
    # re-encoding can also split differently: "a"+"bc" vs "ab"+"c" when no "abc" piece exists
    tok2 = LongestMatch(["a", "b", "c", "ab", "bc"])
    found, _ = find_retokenization_mismatches([0, 4], tok2)                              # a + bc
    assert found[0].original == (0, 4) and found[0].retokenized == (3, 2)                # ab + c


def test_forward_scorer_and_sample_segments():
    V = 10

    def forward(ids):                                   # a "model" that always predicts (last token + 1) mod V
        logits = torch.full((1, ids.shape[1], V), -20.0)
        logits[0, torch.arange(ids.shape[1]), (ids[0] + 1) % V] = 20.0
        return logits

    lp = forward_logprob_fn(forward)
    assert lp([1, 2], 3) > -1e-3 and lp([1, 2], 5) < -30 and lp([], 4) == 0.0
    sample = SimpleNamespace(tokens=[5, 6, 7, 8, 9, 1, 2], loss_mask=[0, 0, 1, 1, 0, 1, 1])
    assert segments_of_sample(sample) == [[5, 6], [7, 8], [9], [1, 2]]
