"""Token-in/token-out providers: the trajectory is rendered to token ids ONCE, the engine
returns token ids and log-probs, and those exact ids are stored on the ``Choice``
(rollouts/providers/sglang.py:386-781, rollouts/inference/backends/generate.py:66-339).

``rollout_native_token_level`` drives the in-process ``InferenceEngine``; the SGLang / vLLM
variants speak the servers' token-level HTTP endpoints.
"""

from __future__ import annotations

import uuid
from dataclasses import replace
from typing import Any

from ...inference.types import SamplingParams
from ..dtypes import Actor, ChatCompletion, Choice, Logprob, Logprobs, Message, RunConfig, Usage
from .base import NonRetryableError, async_retry, classify_http_status
from .tool_parsers import parse_tool_calls, render_tools_system_prompt


def build_input_ids_from_trajectory(actor: Actor, tokenizer: Any, suffix_ids: tuple[int, ...] | None = None) -> list[int]:
    """Prompt token ids for the next assistant turn.

    Earlier assistant turns contribute the engine's own ``Choice.token_ids`` (never re-tokenised
    text); everything between them is tokenised with the chat template. Without stored ids the
    whole conversation goes through ``apply_chat_template``.
    """
    msgs = list(actor.trajectory.messages)
    tools_prompt = render_tools_system_prompt(list(actor.tools))
    dicts = [{"role": m.role, "content": m.text()} for m in msgs]
    if tools_prompt:
        if dicts and dicts[0]["role"] == "system":
            dicts[0] = {"role": "system", "content": dicts[0]["content"] + "\n\n" + tools_prompt}
        else:
            dicts.insert(0, {"role": "system", "content": tools_prompt})
    stored = [c.choices[0] for c in actor.trajectory.completions if c.choices and c.choices[0].token_ids is not None]
    if stored and stored[-1].prompt_token_ids is not None:
        # continue from the last engine-visible prefix: prompt + completion, then the new non-assistant messages
        last = stored[-1]
        prefix = list(last.prompt_token_ids) + list(last.token_ids)
        n_assistant = sum(1 for m in msgs if m.role == "assistant")
        last_assistant_idx = [i for i, m in enumerate(msgs) if m.role == "assistant"][n_assistant - 1]
        tail = [{"role": m.role, "content": m.text()} for m in msgs[last_assistant_idx + 1:]]
        if not tail:
            return prefix
        full_tail = tokenizer.apply_chat_template(tail, tokenize=True, add_generation_prompt=True)
        return prefix + list(suffix_ids or ()) + list(full_tail)
    return list(tokenizer.apply_chat_template(dicts, tokenize=True, add_generation_prompt=True))


def _completion_from_tokens(actor: Actor, prompt_ids: list[int], out_ids: list[int], logprobs: list[float],
                            finish: str, tokenizer: Any, model: str, weight_version: int | None) -> Actor:
    text = tokenizer.decode(out_ids, skip_special_tokens=True) if tokenizer is not None else ""
    rest, calls = parse_tool_calls(text) if actor.tools else (text, [])
    msg = Message("assistant", rest, tool_calls=tuple(calls))
    choice = Choice(0, msg, finish, Logprobs(tuple(Logprob("", lp, tid) for lp, tid in zip(logprobs, out_ids))),
                    tuple(out_ids), tuple(prompt_ids))
    comp = ChatCompletion(f"cmpl_{uuid.uuid4().hex[:12]}", model, (choice,),
                          Usage(input_tokens=len(prompt_ids), output_tokens=len(out_ids)), weight_version=weight_version)
    return replace(actor, trajectory=actor.trajectory.append(msg).with_completion(comp))


async def rollout_native_token_level(actor: Actor, run_config: RunConfig) -> Actor:
    ep = actor.endpoint
    engine = ep.engine
    if engine is None:
        raise NonRetryableError("endpoint.engine is required for the native provider", provider="native")
    tok = run_config.tokenizer or engine.tokenizer
    if tok is None:
        raise NonRetryableError("token-level rollouts need a tokenizer", provider="native")
    prompt_ids = build_input_ids_from_trajectory(actor, tok, run_config.suffix_ids)
    # concurrent agent loops share the engine's batches through its asyncio front
    from ...inference.async_engine import batcher_for

    out = await batcher_for(engine).generate(prompt_ids, SamplingParams(temperature=ep.temperature, max_tokens=ep.max_tokens))
    return _completion_from_tokens(actor, prompt_ids, list(out.completion_tokens), list(out.logprobs), out.finish_reason,
                                   tok, ep.model or "native", out.weight_version)


async def _post_json(url: str, payload: dict, timeout: float, provider: str) -> dict:
    try:
        import httpx
    except ImportError as e:  # pragma: no cover
        raise NonRetryableError("HTTP providers need the httpx package", provider=provider) from e
    async with httpx.AsyncClient(timeout=timeout) as client:
        r = await client.post(url, json=payload)
    if r.status_code != 200:
        raise classify_http_status(r.status_code, r.text, provider)
    return r.json()


@async_retry(max_attempts=3)
async def generate_sglang(api_base: str, input_ids: list[int], max_tokens: int, temperature: float, timeout: float = 120.0,
                          top_logprobs_num: int = 0) -> tuple[list[int], list[float], str]:
    """SGLang ``/generate`` with ``input_ids`` in and token ids + log-probs out."""
    data = await _post_json(f"{api_base.rstrip('/')}/generate",
                            {"input_ids": input_ids, "return_logprob": True, "top_logprobs_num": top_logprobs_num,
                             "sampling_params": {"max_new_tokens": max_tokens, "temperature": temperature}}, timeout, "sglang")
    meta = data.get("meta_info", {})
    lps = meta.get("output_token_logprobs", [])
    ids = [int(t[1]) for t in lps] if lps else list(data.get("output_ids", []))
    fin = meta.get("finish_reason", {})
    return ids, [float(t[0]) for t in lps], (fin.get("type", "stop") if isinstance(fin, dict) else str(fin))


@async_retry(max_attempts=3)
async def generate_vllm(api_base: str, input_ids: list[int], max_tokens: int, temperature: float, model: str = "",
                        timeout: float = 120.0) -> tuple[list[int], list[float], str]:
    """vLLM ``/v1/completions`` with ``prompt_token_ids``."""
    data = await _post_json(f"{api_base.rstrip('/')}/v1/completions",
                            {"model": model, "prompt": input_ids, "max_tokens": max_tokens, "temperature": temperature,
                             "logprobs": 1, "return_tokens_as_token_ids": True}, timeout, "vllm")
    ch = data["choices"][0]
    lp = ch.get("logprobs") or {}
    toks = lp.get("tokens", [])
    ids = [int(t.split(":")[1]) if isinstance(t, str) and t.startswith("token_id:") else int(t) for t in toks]
    return ids, [float(x) for x in lp.get("token_logprobs", [])], ch.get("finish_reason", "stop")


async def rollout_sglang_token_level(actor: Actor, run_config: RunConfig) -> Actor:
    ep, tok = actor.endpoint, run_config.tokenizer
    if tok is None:
        raise NonRetryableError("token-level rollouts need RunConfig.tokenizer", provider="sglang")
    prompt_ids = build_input_ids_from_trajectory(actor, tok, run_config.suffix_ids)
    ids, lps, fin = await generate_sglang(ep.api_base, prompt_ids, ep.max_tokens, ep.temperature, ep.timeout)
    return _completion_from_tokens(actor, prompt_ids, ids, lps, fin, tok, ep.model, None)


async def rollout_vllm_token_level(actor: Actor, run_config: RunConfig) -> Actor:
    ep, tok = actor.endpoint, run_config.tokenizer
    if tok is None:
        raise NonRetryableError("token-level rollouts need RunConfig.tokenizer", provider="vllm")
    prompt_ids = build_input_ids_from_trajectory(actor, tok, run_config.suffix_ids)
    ids, lps, fin = await generate_vllm(ep.api_base, prompt_ids, ep.max_tokens, ep.temperature, ep.model, ep.timeout)
    return _completion_from_tokens(actor, prompt_ids, ids, lps, fin, tok, ep.model, None)
