"""Text-level providers: any OpenAI-compatible ``/v1/chat/completions`` server (SGLang, vLLM,
OpenAI and friends) and a scripted mock used by tests
(rollouts/providers/openai_completions.py:289-499, sglang.py:200-380)."""

from __future__ import annotations

import json
import logging
import uuid
from dataclasses import replace
from typing import Any

from ..dtypes import (Actor, ChatCompletion, Choice, Cost, ImageContent, Message, RunConfig, TextDelta, ToolCall, ToolCallEnd, ToolCallStart,
                      Usage)
from .base import (NonRetryableError, async_retry, classify_http_status, classify_server_error, explain_server_error,
                   prepare_messages_for_llm, sanitize_request_for_logging)
from .models import estimate_cost
from .tool_parsers import parse_tool_calls


def messages_to_openai(actor: Actor) -> list[dict[str, Any]]:
    out = []
    for m in prepare_messages_for_llm(list(actor.trajectory.messages)):
        d: dict[str, Any] = {"role": m.role, "content": m.text()}
        calls = m.get_tool_calls()
        if m.role == "assistant" and calls:
            d["tool_calls"] = [{"id": c.id, "type": "function", "function": {"name": c.name, "arguments": json.dumps(c.args)}}
                               for c in calls]
        images = [b for b in m.content if isinstance(b, ImageContent)] if isinstance(m.content, list) else []
        image_parts = [{"type": "image_url", "image_url": {"url": f"data:{b.mime_type};base64,{b.data}"}} for b in images]
        if m.role == "tool":
            d["tool_call_id"] = m.tool_call_id
            out.append(d)
            if image_parts:                                  # tool messages carry text only: the picture follows as a user message
                out.append({"role": "user", "content": [{"type": "text", "text": f"(image returned by {m.name or 'the tool'})"}] + image_parts})
            continue
        if image_parts and m.role == "user":
            d["content"] = ([{"type": "text", "text": m.text()}] if m.text() else []) + image_parts
        out.append(d)
    return out


@async_retry(max_attempts=3)
async def _chat_completion(ep, payload: dict) -> dict:
    try:
        import httpx
    except ImportError as e:  # pragma: no cover
        raise NonRetryableError("HTTP providers need the httpx package", provider=ep.provider) from e
    headers = {"Authorization": f"Bearer {ep.api_key}"} if ep.api_key else {}
    async with httpx.AsyncClient(timeout=ep.timeout) as client:
        r = await client.post(f"{ep.api_base.rstrip('/')}/v1/chat/completions", json=payload, headers=headers)
    if r.status_code != 200:
        kind = classify_server_error(r.status_code, r.text)
        if kind in ("context_length", "invalid_param"):     # retrying cannot help: say what will, once
            logging.getLogger(__name__).error("%s\nrequest: %s", explain_server_error(kind, max_tokens=payload.get("max_tokens"), param_keys=list(payload)),
                                              sanitize_request_for_logging(payload))
        raise classify_http_status(r.status_code, r.text, ep.provider)
    return r.json()


async def rollout_openai_compatible(actor: Actor, run_config: RunConfig) -> Actor:
    ep = actor.endpoint
    payload: dict[str, Any] = {"model": ep.model, "messages": messages_to_openai(actor), "max_tokens": ep.max_tokens,
                               "temperature": ep.temperature, **ep.extra_params}
    if ep.top_p is not None:
        payload["top_p"] = ep.top_p
    if actor.tools:
        payload["tools"] = [t.to_openai() for t in actor.tools]
    data = await _chat_completion(ep, payload)
    ch = data["choices"][0]
    m = ch["message"]
    text = m.get("content") or ""
    calls = [ToolCall(c["id"], c["function"]["name"], json.loads(c["function"].get("arguments") or "{}"))
             for c in (m.get("tool_calls") or [])]
    if not calls and actor.tools:
        text, calls = parse_tool_calls(text)
    u = data.get("usage", {})
    usage = Usage(u.get("prompt_tokens", 0), u.get("completion_tokens", 0))
    usage = replace(usage, cost=estimate_cost(ep.model, usage))
    msg = Message("assistant", text, tool_calls=tuple(calls))
    if run_config.on_chunk is not None and text:
        await run_config.on_chunk(TextDelta(delta=text))
    comp = ChatCompletion(data.get("id", f"cmpl_{uuid.uuid4().hex[:12]}"), ep.model,
                          (Choice(0, msg, ch.get("finish_reason", "stop")),), usage)
    return replace(actor, trajectory=actor.trajectory.append(msg).with_completion(comp))


class ScriptedLLM:
    """Deterministic stand-in for a model: replies come from a list (tests, dry runs)."""

    def __init__(self, replies: list[str | Message]):
        self.replies = list(replies)
        self.calls = 0

    async def __call__(self, actor: Actor, run_config: RunConfig) -> Actor:
        r = self.replies[min(self.calls, len(self.replies) - 1)]
        self.calls += 1
        if isinstance(r, Message):
            msg = r
        else:
            text, calls = parse_tool_calls(r)
            msg = Message("assistant", text, tool_calls=tuple(calls))
        if run_config.on_chunk is not None and msg.text():
            await run_config.on_chunk(TextDelta(delta=msg.text()))
        if run_config.on_chunk is not None:
            for c in msg.get_tool_calls():      # the same events a streaming provider emits per call
                await run_config.on_chunk(ToolCallStart(tool_call_id=c.id, name=c.name))
                await run_config.on_chunk(ToolCallEnd(tool_call_id=c.id, name=c.name, args=dict(c.args)))
        comp = ChatCompletion(f"mock_{self.calls}", "scripted", (Choice(0, msg),), Usage(1, 1, cost=Cost()))
        return replace(actor, trajectory=actor.trajectory.append(msg).with_completion(comp))
