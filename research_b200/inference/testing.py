"""Correctness harness: exact match first, else "top-N containment"
(rollouts/inference/testing.py:39-378, the vLLM-style criterion the reference adopts).

Two generations agree if every token is identical, or, at the first divergence, each side's
token is among the other side's top-N candidates at that position and the log-probabilities
of the shared prefix are close."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .backends.generate import GenerationOutput, generate_hf


@dataclass(frozen=True)
class LogprobCheck:
    ok: bool
    exact: bool
    first_divergence: int | None
    max_logprob_diff: float
    detail: str = ""


def generate_with_logprobs_forward(forward_fn, prompts: list[list[int]], max_tokens: int, top_n: int = 5) -> list[GenerationOutput]:
    return generate_hf(forward_fn, prompts, max_tokens, temperature=0.0, top_logprobs_num=top_n)


def topn_at(forward_fn, ids: list[int], top_n: int) -> list[tuple[int, float]]:
    lp = torch.log_softmax(forward_fn(torch.tensor([ids]))[0, -1].float(), -1)
    v, i = lp.topk(top_n)
    return [(int(a), float(b)) for a, b in zip(i, v)]


def check_logprobs_close(ref: GenerationOutput, test_ids: tuple[int, ...], test_logprobs: tuple[float, ...], forward_fn=None,
                         top_n: int = 5, logprob_tol: float = 0.05) -> LogprobCheck:
    n = min(len(ref.output_ids), len(test_ids))
    div = next((i for i in range(n) if ref.output_ids[i] != test_ids[i]), None)
    upto = n if div is None else div
    diffs = [abs(a - b) for a, b in zip(ref.logprobs[:upto], test_logprobs[:upto])]
    mx = max(diffs) if diffs else 0.0
    if mx > logprob_tol:
        return LogprobCheck(False, False, div, mx, f"log-probs differ by {mx:.4f} on the common prefix")
    if div is None:
        return LogprobCheck(True, len(ref.output_ids) == len(test_ids), None, mx)
    if ref.top_logprobs is not None:
        cands = {t for t, _ in ref.top_logprobs[div]}
    elif forward_fn is not None:
        cands = {t for t, _ in topn_at(forward_fn, list(ref.input_ids) + list(ref.output_ids[:div]), top_n)}
    else:
        return LogprobCheck(False, False, div, mx, "diverged and no top-N candidates available")
    if test_ids[div] in cands:
        return LogprobCheck(True, False, div, mx, f"diverged at {div} inside the reference top-{top_n}")
    return LogprobCheck(False, False, div, mx, f"token {test_ids[div]} at {div} is outside the reference top-{top_n}")


def check_outputs_equal(a: list[GenerationOutput], b: list[GenerationOutput]) -> list[bool]:
    return [x.output_ids == y.output_ids for x, y in zip(a, b)]
