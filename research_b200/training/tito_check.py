"""Token-in / token-out consistency checks for multi-turn rollouts (the methodology of
rollouts/tests/test_tito_correctness.py:59-620 and :626-1057, as a library instead of a remote script).

A multi-turn rollout is a list of *segments* of token ids: what the model generated in turn 1, the tool result that
was inserted, what it generated in turn 2, ... Training on ``decode -> re-encode`` of that text instead of on the ids
themselves can change the tokens around the seams: two tokens the model emitted separately merge into one, or an
inserted text re-splits the end of a generation. The trainer would then compute log-probabilities for tokens the
sampler never produced, often with a very low probability, which wrecks the importance ratio.

``find_retokenization_mismatches`` locates those spans by aligning both tokenisations on character offsets;
``check_rollout`` adds which seams they touch and, given a ``logprob_fn``, how (un)likely the re-encoded tokens are
under the model given the true prefix; spans below ``smoking_gun`` are the ones that break training.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Sequence


@dataclass(frozen=True)
class Mismatch:
    start: int                         # index of the first differing token in the original stream
    original: tuple[int, ...]
    retokenized: tuple[int, ...]
    text: str
    seams: tuple[int, ...] = ()        # segment boundaries (token indices) inside or at the edge of the span
    logprobs: tuple[float, ...] = ()   # model log-prob of each re-encoded token given the true prefix (+ earlier re-encoded ones)

    @property
    def at_seam(self) -> bool:
        return bool(self.seams)

    @property
    def min_logprob(self) -> float | None:
        return min(self.logprobs) if self.logprobs else None


@dataclass
class TitoReport:
    num_tokens: int
    num_retokenized: int
    mismatches: list[Mismatch] = field(default_factory=list)
    threshold: float = -10.0
    smoking_gun: float = -15.0

    @property
    def ok(self) -> bool:
        return not self.mismatches

    @property
    def at_seams(self) -> list[Mismatch]:
        return [m for m in self.mismatches if m.at_seam]

    @property
    def suspicious(self) -> list[Mismatch]:
        return [m for m in self.mismatches if m.min_logprob is not None and m.min_logprob < self.threshold]

    @property
    def smoking_guns(self) -> list[Mismatch]:
        return [m for m in self.mismatches if m.min_logprob is not None and m.min_logprob < self.smoking_gun]

    def summary(self) -> str:
        if self.ok:
            return f"{self.num_tokens} tokens survive decode + re-encode unchanged"
        lines = [f"{len(self.mismatches)} span(s) change under decode + re-encode ({self.num_tokens} -> {self.num_retokenized} tokens), "
                 f"{len(self.at_seams)} at segment seams, {len(self.suspicious)} below {self.threshold}, "
                 f"{len(self.smoking_guns)} below {self.smoking_gun}"]
        for m in self.mismatches:
            lp = f" min logprob {m.min_logprob:.2f}" if m.logprobs else ""
            lines.append(f"  @{m.start}{' (seam)' if m.at_seam else ''}: {list(m.original)} -> {list(m.retokenized)} {m.text!r}{lp}")
        return "\n".join(lines)


def _offsets(ids: Sequence[int], tokenizer: Any, text: str) -> list[int]:
    """Character offset after every token. Per-token decoding is tried first; tokenizers whose pieces do not decode
    independently (byte fallbacks, leading-space rules) get the slower prefix decoding."""
    out, pos = [], 0
    for t in ids:
        pos += len(tokenizer.decode([t]))
        out.append(pos)
    if pos == len(text):
        return out
    return [len(tokenizer.decode(list(ids[:i + 1]))) for i in range(len(ids))]


def find_retokenization_mismatches(ids: Sequence[int], tokenizer: Any) -> tuple[list[Mismatch], list[int]]:
    """Spans where ``encode(decode(ids))`` differs from ``ids``; also returns the re-encoded ids."""
    ids = list(ids)
    text = tokenizer.decode(ids)
    try:
        re_ids = list(tokenizer.encode(text, add_special_tokens=False))
    except TypeError:
        re_ids = list(tokenizer.encode(text))
    if re_ids == ids:
        return [], re_ids
    oa, ob = _offsets(ids, tokenizer, text), _offsets(re_ids, tokenizer, text)
    out: list[Mismatch] = []
    i = j = 0                   # next token of each stream
    si = sj = 0                 # start of the current block (both streams sit on a common character boundary there)
    char0 = 0
    while i < len(ids) and j < len(re_ids):
        if oa[i] == ob[j]:      # common boundary: close the block
            a, b = ids[si:i + 1], re_ids[sj:j + 1]
            if a != b:
                out.append(Mismatch(si, tuple(a), tuple(b), text[char0:oa[i]]))
            char0 = oa[i]
            i, j = i + 1, j + 1
            si, sj = i, j
        elif oa[i] < ob[j]:
            i += 1
        else:
            j += 1
    if si < len(ids) or sj < len(re_ids):
        out.append(Mismatch(si, tuple(ids[si:]), tuple(re_ids[sj:]), text[char0:]))
    return out, re_ids


def check_rollout(segments: Sequence[Sequence[int]], tokenizer: Any, logprob_fn: Callable[[list[int], int], float] | None = None,
                  threshold: float = -10.0, smoking_gun: float = -15.0) -> TitoReport:
    """``segments``: the rollout's token ids cut where their source changes (generation / inserted text / next
    generation). ``logprob_fn(prefix_ids, token) -> log p(token | prefix)`` is any scorer (an engine's prompt log-probs,
    a forward pass of the trainer's model)."""
    ids = [t for seg in segments for t in seg]
    seams, n = [], 0
    for seg in segments[:-1]:
        n += len(seg)
        seams.append(n)
    found, re_ids = find_retokenization_mismatches(ids, tokenizer)
    out = []
    for m in found:
        end = m.start + len(m.original)
        touching = tuple(s for s in seams if m.start <= s <= end)
        lps: tuple[float, ...] = ()
        if logprob_fn is not None:
            prefix = ids[:m.start]
            got = []
            for t in m.retokenized:
                got.append(float(logprob_fn(list(prefix), t)))
                prefix = prefix + [t]
            lps = tuple(got)
        out.append(Mismatch(m.start, m.original, m.retokenized, m.text, touching, lps))
    return TitoReport(len(ids), len(re_ids), out, threshold, smoking_gun)


def forward_logprob_fn(forward_fn: Callable[[Any], Any]) -> Callable[[list[int], int], float]:
    """``logprob_fn`` from a full-sequence forward ``forward_fn(ids [1, T]) -> logits [1, T, V]``."""
    import torch

    def lp(prefix: list[int], token: int) -> float:
        if not prefix:
            return 0.0
        with torch.no_grad():
            logits = forward_fn(torch.tensor([prefix]))[0, -1].float()
        return float(torch.log_softmax(logits, -1)[token])
    return lp


def segments_of_sample(sample: Any) -> list[list[int]]:
    """Cut a training ``Sample`` (``tokens`` + ``loss_mask``) where the mask flips: generated vs. inserted runs."""
    toks, mask = list(sample.tokens), list(sample.loss_mask)
    segs: list[list[int]] = []
    for t, m in zip(toks, mask):
        if not segs or (m > 0) != cur:
            segs.append([])
            cur = m > 0
        segs[-1].append(t)
    return segs
