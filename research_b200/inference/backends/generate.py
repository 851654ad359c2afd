"""Token-in/token-out generation against four engines with one output type
(rollouts/inference/backends/generate.py:52-339): the native engine, SGLang ``/generate``,
vLLM ``/v1/completions`` and a step-by-step functional forward used as ground truth."""

from __future__ import annotations

import asyncio
from dataclasses import dataclass

import torch

from ..types import SamplingParams


@dataclass(frozen=True)
class GenerationOutput:
    input_ids: tuple[int, ...]
    output_ids: tuple[int, ...]
    logprobs: tuple[float, ...]
    finish_reason: str = "length"
    top_logprobs: tuple[tuple[tuple[int, float], ...], ...] | None = None


def generate_native(engine, input_ids: list[list[int]], max_tokens: int = 256, temperature: float = 1.0,
                    num_samples: int = 1) -> list[GenerationOutput]:
    outs = engine.generate(input_ids, SamplingParams(temperature=temperature, max_tokens=max_tokens), num_samples)
    return [GenerationOutput(o.prompt_tokens, o.completion_tokens, o.logprobs, o.finish_reason) for o in outs]


async def generate_sglang(base_url: str, input_ids: list[list[int]], max_tokens: int = 256, temperature: float = 1.0,
                          top_logprobs_num: int = 0) -> list[GenerationOutput]:
    from ...agents.providers.token_level import generate_sglang as _one

    res = await asyncio.gather(*[_one(base_url, ids, max_tokens, temperature, top_logprobs_num=top_logprobs_num) for ids in input_ids])
    return [GenerationOutput(tuple(i), tuple(o), tuple(lp), fin) for i, (o, lp, fin) in zip(input_ids, res)]


async def generate_vllm(base_url: str, input_ids: list[list[int]], max_tokens: int = 256, temperature: float = 1.0,
                        model: str = "") -> list[GenerationOutput]:
    from ...agents.providers.token_level import generate_vllm as _one

    res = await asyncio.gather(*[_one(base_url, ids, max_tokens, temperature, model) for ids in input_ids])
    return [GenerationOutput(tuple(i), tuple(o), tuple(lp), fin) for i, (o, lp, fin) in zip(input_ids, res)]


def generate_hf(forward_fn, input_ids: list[list[int]], max_tokens: int = 256, temperature: float = 1.0, top_k: int = 0,
                top_p: float = 1.0, top_logprobs_num: int = 0, eos_token_id: int | None = None,
                generator: torch.Generator | None = None) -> list[GenerationOutput]:
    """Ground truth: recompute the full forward per token. ``forward_fn(ids [1,T]) -> logits [1,T,V]``
    can wrap an HF model (``lambda x: model(x).logits``) or the functional oracle."""
    outs = []
    for prompt in input_ids:
        ids = list(prompt)
        lps, tops, fin = [], [], "length"
        for _ in range(max_tokens):
            logits = forward_fn(torch.tensor([ids]))[0, -1].float()
            logprobs = torch.log_softmax(logits, -1)
            if temperature <= 0:
                tok = int(logits.argmax())
            else:
                scaled = logits / temperature
                if top_k > 0:
                    kth = scaled.topk(top_k).values[-1]
                    scaled = scaled.masked_fill(scaled < kth, float("-inf"))
                if top_p < 1.0:
                    sp, si = scaled.softmax(-1).sort(descending=True)
                    cut = sp.cumsum(-1) - sp > top_p
                    scaled[si[cut]] = float("-inf")
                tok = int(torch.multinomial(scaled.softmax(-1), 1, generator=generator))
            lps.append(float(logprobs[tok]))
            if top_logprobs_num:
                tv, ti = logprobs.topk(top_logprobs_num)
                tops.append(tuple((int(i), float(v)) for i, v in zip(ti, tv)))
            ids.append(tok)
            if eos_token_id is not None and tok == eos_token_id:
                fin = "stop"
                break
        outs.append(GenerationOutput(tuple(prompt), tuple(ids[len(prompt):]), tuple(lps), fin, tuple(tops) if tops else None))
    return outs
