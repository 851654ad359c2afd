"""Streaming providers: wire formats, server-sent-event parsing and stream aggregation for the
Anthropic Messages API, OpenAI chat completions, the OpenAI Responses API and Google Gemini
(rollouts/providers/anthropic.py:216-600, openai_completions.py:289-499, openai_responses.py:58-557,
google.py:40-312).

Every aggregator consumes an async iterator of already-decoded JSON events, forwards
``TextDelta`` / ``ThinkingDelta`` / ``ToolCallStart`` / ``ToolCallEnd`` to ``on_chunk`` as they arrive
and returns one ``ChatCompletion``. The network layer (``sse_events`` over an ``httpx`` stream) is
separate, so the aggregators are tested offline against recorded event sequences.
"""

from __future__ import annotations

import json
import uuid
from dataclasses import replace
from typing import Any, AsyncIterator, Awaitable, Callable

from ..dtypes import (Actor, ChatCompletion, Choice, ImageContent, Message, RunConfig, StreamEvent, StreamStart, TextContent, TextDelta,
                      TextEnd, TextStart, ThinkingContent, ThinkingDelta, ThinkingEnd, ThinkingStart, Tool, ToolCall, ToolCallContent,
                      ToolCallDelta, ToolCallEnd, ToolCallError, ToolCallStart, Usage, parse_streaming_json)
from .base import NonRetryableError, classify_http_status
from .models import estimate_cost

OnChunk = Callable[[StreamEvent], Awaitable[None]] | None


async def _emit(on_chunk: OnChunk, ev: StreamEvent) -> None:
    if on_chunk is not None:
        await on_chunk(ev)


def _loads(s: str) -> dict[str, Any]:
    try:
        v = json.loads(s) if s.strip() else {}
        return v if isinstance(v, dict) else {"value": v}
    except json.JSONDecodeError:
        return {"_raw": s}


async def _tool_call_done(on_chunk: OnChunk, call_id: str, name: str, raw: str) -> dict[str, Any]:
    """Parse a finished call's arguments; arguments that are not JSON are reported (``ToolCallError``) and still handed
    on as ``{"_raw": text}``, so that the environment can answer the model with what was wrong."""
    args = _loads(raw)
    if "_raw" in args and len(args) == 1:
        await _emit(on_chunk, ToolCallError(tool_call_id=call_id, tool_name=name, error="the arguments are not valid JSON", raw_arguments=raw))
    await _emit(on_chunk, ToolCallEnd(tool_call_id=call_id, name=name, args=args))
    return args


def _finish(model: str, blocks: list[Any], stop: str, usage: Usage, cid: str | None = None) -> ChatCompletion:
    text_only = all(isinstance(b, TextContent) for b in blocks)
    content: Any = "".join(b.text for b in blocks) if text_only else blocks
    usage = replace(usage, cost=estimate_cost(model, usage))
    return ChatCompletion(cid or f"cmpl_{uuid.uuid4().hex[:12]}", model, (Choice(0, Message("assistant", content), stop),), usage)


# ------------------------------------------------------------------------------------------ SSE
async def sse_events(lines: AsyncIterator[str]) -> AsyncIterator[dict[str, Any]]:
    """Decode ``data:`` lines of a server-sent-event stream into JSON objects (``[DONE]`` ends it)."""
    buf: list[str] = []
    async for line in lines:
        line = line.rstrip("\r\n")
        if line.startswith("data:"):
            buf.append(line[5:].lstrip())
            continue
        if line == "" and buf:
            payload = "\n".join(buf)
            buf = []
            if payload == "[DONE]":
                return
            yield _loads(payload)
    if buf and "\n".join(buf) != "[DONE]":
        yield _loads("\n".join(buf))


# ------------------------------------------------------------------------------------------ Anthropic
def messages_to_anthropic(messages: tuple[Message, ...]) -> tuple[str, list[dict[str, Any]]]:
    """Split out the system prompt; tool results become ``tool_result`` blocks in a user turn;
    consecutive turns of one role are merged (the API rejects them otherwise)."""
    system = "\n\n".join(m.text() for m in messages if m.role == "system")
    out: list[dict[str, Any]] = []
    for m in messages:
        if m.role == "system":
            continue
        if m.role == "tool":
            images = [b for b in m.content if isinstance(b, ImageContent)] if isinstance(m.content, list) else []
            body: Any = m.text()
            if images:                                       # a tool that returned a picture: text and image blocks in the result
                body = ([{"type": "text", "text": m.text()}] if m.text() else []) + [
                    {"type": "image", "source": {"type": "base64", "media_type": b.mime_type, "data": b.data}} for b in images]
            role, blocks = "user", [{"type": "tool_result", "tool_use_id": m.tool_call_id, "content": body}]
        else:
            role, blocks = m.role, []
            if isinstance(m.content, list):
                for b in m.content:
                    if isinstance(b, TextContent) and b.text:
                        blocks.append({"type": "text", "text": b.text})
                    elif isinstance(b, ThinkingContent) and b.signature:
                        blocks.append({"type": "thinking", "thinking": b.thinking, "signature": b.signature})
                    elif isinstance(b, ImageContent):
                        blocks.append({"type": "image", "source": {"type": "base64", "media_type": b.mime_type, "data": b.data}})
            elif m.text():
                blocks.append({"type": "text", "text": m.text()})
            for c in m.get_tool_calls():
                blocks.append({"type": "tool_use", "id": c.id, "name": c.name, "input": c.args})
        if not blocks:
            continue
        if out and out[-1]["role"] == role:
            out[-1]["content"].extend(blocks)
        else:
            out.append({"role": role, "content": blocks})
    return system, out


def tool_to_anthropic(t: Tool) -> dict[str, Any]:
    p = t.function.parameters
    return {"name": t.function.name, "description": t.function.description,
            "input_schema": {"type": p.type, "properties": p.properties, "required": list(p.required)}}


async def aggregate_anthropic_stream(events: AsyncIterator[dict[str, Any]], model: str, on_chunk: OnChunk = None) -> ChatCompletion:
    blocks: dict[int, dict[str, Any]] = {}
    usage, stop, cid = Usage(), "stop", None
    async for ev in events:
        t = ev.get("type")
        if t == "message_start":
            msg = ev.get("message", {})
            cid = msg.get("id")
            u = msg.get("usage", {})
            usage = Usage(u.get("input_tokens", 0), u.get("output_tokens", 0), 0, u.get("cache_read_input_tokens", 0),
                          u.get("cache_creation_input_tokens", 0))
            await _emit(on_chunk, StreamStart())
        elif t == "content_block_start":
            cb = ev.get("content_block", {})
            blocks[ev["index"]] = {"type": cb.get("type"), "text": cb.get("text", ""), "thinking": cb.get("thinking", ""),
                                   "signature": None, "id": cb.get("id"), "name": cb.get("name"), "json": ""}
            if cb.get("type") == "tool_use":
                await _emit(on_chunk, ToolCallStart(tool_call_id=cb.get("id", ""), name=cb.get("name", "")))
            elif cb.get("type") == "text":
                await _emit(on_chunk, TextStart(content_index=ev["index"]))
            elif cb.get("type") == "thinking":
                await _emit(on_chunk, ThinkingStart(content_index=ev["index"]))
        elif t == "content_block_delta":
            b, d = blocks.setdefault(ev["index"], {"type": "text", "text": "", "thinking": "", "json": "", "signature": None}), ev.get("delta", {})
            if d.get("type") == "text_delta":
                b["text"] += d.get("text", "")
                await _emit(on_chunk, TextDelta(delta=d.get("text", "")))
            elif d.get("type") == "thinking_delta":
                b["thinking"] += d.get("thinking", "")
                await _emit(on_chunk, ThinkingDelta(delta=d.get("thinking", "")))
            elif d.get("type") == "signature_delta":
                b["signature"] = (b["signature"] or "") + d.get("signature", "")
            elif d.get("type") == "input_json_delta":
                b["json"] += d.get("partial_json", "")
                await _emit(on_chunk, ToolCallDelta(tool_call_id=b.get("id") or "", delta=d.get("partial_json", ""), partial_args=parse_streaming_json(b["json"])))
        elif t == "content_block_stop":
            b = blocks.get(ev["index"], {})
            if b.get("type") == "tool_use":
                await _tool_call_done(on_chunk, b["id"], b["name"], b["json"])
            elif b.get("type") == "text":
                await _emit(on_chunk, TextEnd(content_index=ev["index"], content=b["text"]))
            elif b.get("type") == "thinking":
                await _emit(on_chunk, ThinkingEnd(content_index=ev["index"], content=b["thinking"]))
        elif t == "message_delta":
            stop = {"end_turn": "stop", "tool_use": "tool_calls", "max_tokens": "length"}.get(ev.get("delta", {}).get("stop_reason"), stop)
            if "usage" in ev:
                usage = replace(usage, output_tokens=ev["usage"].get("output_tokens", usage.output_tokens))
        elif t == "error":
            raise classify_http_status(529 if ev.get("error", {}).get("type") == "overloaded_error" else 500,
                                       json.dumps(ev.get("error", {})), "anthropic")
    content = []
    for i in sorted(blocks):
        b = blocks[i]
        if b["type"] == "text":
            content.append(TextContent(b["text"]))
        elif b["type"] == "thinking":
            content.append(ThinkingContent(b["thinking"], b["signature"]))
        elif b["type"] == "tool_use":
            content.append(ToolCallContent(b["id"], b["name"], _loads(b["json"])))
    return _finish(model, content, stop, usage, cid)


# ------------------------------------------------------------------------------------------ OpenAI chat
async def aggregate_openai_stream(events: AsyncIterator[dict[str, Any]], model: str, on_chunk: OnChunk = None) -> ChatCompletion:
    text, reasoning, calls, stop, usage, cid = "", "", {}, "stop", Usage(), None
    started = False
    async for ev in events:
        if not started:
            started = True
            await _emit(on_chunk, StreamStart())
        cid = cid or ev.get("id")
        if ev.get("usage"):
            u = ev["usage"]
            usage = Usage(u.get("prompt_tokens", 0), u.get("completion_tokens", 0),
                          (u.get("completion_tokens_details") or {}).get("reasoning_tokens", 0),
                          (u.get("prompt_tokens_details") or {}).get("cached_tokens", 0))
        for ch in ev.get("choices", []):
            d = ch.get("delta", {})
            r = d.get("reasoning_content") or d.get("reasoning")
            if r:
                if not reasoning:
                    await _emit(on_chunk, ThinkingStart(content_index=0))
                reasoning += r
                await _emit(on_chunk, ThinkingDelta(delta=r))
            if d.get("content"):
                if not text:
                    if reasoning:                       # the answer begins: the reasoning block is complete
                        await _emit(on_chunk, ThinkingEnd(content_index=0, content=reasoning))
                    await _emit(on_chunk, TextStart(content_index=1 if reasoning else 0))
                text += d["content"]
                await _emit(on_chunk, TextDelta(delta=d["content"]))
            for tc in d.get("tool_calls") or []:
                slot = calls.setdefault(tc.get("index", 0), {"id": "", "name": "", "json": ""})
                fn = tc.get("function", {})
                if tc.get("id"):
                    slot["id"] = tc["id"]
                if fn.get("name"):
                    slot["name"] = fn["name"]
                    await _emit(on_chunk, ToolCallStart(tool_call_id=slot["id"], name=slot["name"]))
                if fn.get("arguments"):
                    slot["json"] += fn["arguments"]
                    await _emit(on_chunk, ToolCallDelta(tool_call_id=slot["id"], delta=fn["arguments"], partial_args=parse_streaming_json(slot["json"])))
            if ch.get("finish_reason"):
                stop = ch["finish_reason"]
    blocks: list[Any] = []
    if reasoning:
        blocks.append(ThinkingContent(reasoning))
        if not text:
            await _emit(on_chunk, ThinkingEnd(content_index=0, content=reasoning))
    if text or not calls:
        blocks.append(TextContent(text))
    if text:
        await _emit(on_chunk, TextEnd(content_index=1 if reasoning else 0, content=text))
    for i in sorted(calls):
        c = calls[i]
        args = await _tool_call_done(on_chunk, c["id"], c["name"], c["json"])
        blocks.append(ToolCallContent(c["id"] or f"call_{uuid.uuid4().hex[:8]}", c["name"], args))
    return _finish(model, blocks, stop, usage, cid)


# ------------------------------------------------------------------------------------------ OpenAI responses
def messages_to_openai_responses(messages: tuple[Message, ...]) -> list[dict[str, Any]]:
    """Input items of the Responses API: messages, ``function_call`` and ``function_call_output`` items."""
    items: list[dict[str, Any]] = []
    for m in messages:
        if m.role == "tool":
            items.append({"type": "function_call_output", "call_id": m.tool_call_id, "output": m.text()})
            continue
        if m.text():
            kind = "output_text" if m.role == "assistant" else "input_text"
            items.append({"type": "message", "role": "developer" if m.role == "system" else m.role,
                          "content": [{"type": kind, "text": m.text()}]})
        for c in m.get_tool_calls():
            items.append({"type": "function_call", "call_id": c.id, "name": c.name, "arguments": json.dumps(c.args)})
    return items


async def aggregate_openai_responses_stream(events: AsyncIterator[dict[str, Any]], model: str, on_chunk: OnChunk = None) -> ChatCompletion:
    text, reasoning, calls, usage, stop, cid = "", "", {}, Usage(), "stop", None
    async for ev in events:
        t = ev.get("type", "")
        if t == "response.created":
            cid = ev.get("response", {}).get("id")
            await _emit(on_chunk, StreamStart())
        elif t == "response.output_text.delta":
            if not text:
                await _emit(on_chunk, TextStart(content_index=1 if reasoning else 0))
            text += ev.get("delta", "")
            await _emit(on_chunk, TextDelta(delta=ev.get("delta", "")))
        elif t == "response.output_text.done":
            await _emit(on_chunk, TextEnd(content_index=1 if reasoning else 0, content=ev.get("text", text)))
        elif t in ("response.reasoning_summary_text.delta", "response.reasoning_text.delta"):
            if not reasoning:
                await _emit(on_chunk, ThinkingStart(content_index=0))
            reasoning += ev.get("delta", "")
            await _emit(on_chunk, ThinkingDelta(delta=ev.get("delta", "")))
        elif t in ("response.reasoning_summary_text.done", "response.reasoning_text.done"):
            await _emit(on_chunk, ThinkingEnd(content_index=0, content=ev.get("text", reasoning)))
        elif t == "response.output_item.added" and ev.get("item", {}).get("type") == "function_call":
            it = ev["item"]
            calls[it.get("id") or it.get("call_id")] = {"id": it.get("call_id") or it.get("id"), "name": it.get("name", ""), "json": it.get("arguments", "")}
            await _emit(on_chunk, ToolCallStart(tool_call_id=it.get("call_id", ""), name=it.get("name", "")))
        elif t == "response.function_call_arguments.delta":
            if ev.get("item_id") in calls:
                slot = calls[ev["item_id"]]
                slot["json"] += ev.get("delta", "")
                await _emit(on_chunk, ToolCallDelta(tool_call_id=slot["id"] or "", delta=ev.get("delta", ""), partial_args=parse_streaming_json(slot["json"])))
        elif t == "response.output_item.done" and ev.get("item", {}).get("type") == "function_call":
            it = ev["item"]
            slot = calls.setdefault(it.get("id") or it.get("call_id"), {"id": it.get("call_id"), "name": it.get("name", ""), "json": ""})
            slot["json"] = it.get("arguments") or slot["json"]
            await _tool_call_done(on_chunk, slot["id"], slot["name"], slot["json"])
        elif t in ("response.completed", "response.incomplete"):
            r = ev.get("response", {})
            u = r.get("usage") or {}
            usage = Usage(u.get("input_tokens", 0), u.get("output_tokens", 0),
                          (u.get("output_tokens_details") or {}).get("reasoning_tokens", 0),
                          (u.get("input_tokens_details") or {}).get("cached_tokens", 0))
            if t == "response.incomplete":
                stop = "length"
        elif t in ("response.failed", "error"):
            raise classify_http_status(500, json.dumps(ev), "openai")
    blocks: list[Any] = []
    if reasoning:
        blocks.append(ThinkingContent(reasoning))
    if text or not calls:
        blocks.append(TextContent(text))
    blocks += [ToolCallContent(c["id"], c["name"], _loads(c["json"])) for c in calls.values()]
    if calls:
        stop = "tool_calls"
    return _finish(model, blocks, stop, usage, cid)


# ------------------------------------------------------------------------------------------ Google
def messages_to_google(messages: tuple[Message, ...]) -> tuple[str, list[dict[str, Any]]]:
    system = "\n\n".join(m.text() for m in messages if m.role == "system")
    names = {c.id: c.name for m in messages for c in m.get_tool_calls()}
    out: list[dict[str, Any]] = []
    for m in messages:
        if m.role == "system":
            continue
        if m.role == "tool":
            role = "user"
            parts = [{"functionResponse": {"name": names.get(m.tool_call_id, m.name or "tool"), "response": {"result": m.text()}}}]
        else:
            role = "model" if m.role == "assistant" else "user"
            parts = [{"text": m.text()}] if m.text() else []
            parts += [{"functionCall": {"name": c.name, "args": c.args}} for c in m.get_tool_calls()]
        if not parts:
            continue
        if out and out[-1]["role"] == role:
            out[-1]["parts"].extend(parts)
        else:
            out.append({"role": role, "parts": parts})
    return system, out


async def aggregate_google_stream(events: AsyncIterator[dict[str, Any]], model: str, on_chunk: OnChunk = None) -> ChatCompletion:
    text, thinking, calls, usage, stop = "", "", [], Usage(), "stop"
    started = False
    async for ev in events:
        if not started:
            started = True
            await _emit(on_chunk, StreamStart())
        for cand in ev.get("candidates", []):
            for part in (cand.get("content") or {}).get("parts", []):
                if "text" in part and part.get("thought"):
                    if not thinking:
                        await _emit(on_chunk, ThinkingStart(content_index=0))
                    thinking += part["text"]
                    await _emit(on_chunk, ThinkingDelta(delta=part["text"]))
                elif "text" in part:
                    if not text:
                        if thinking:
                            await _emit(on_chunk, ThinkingEnd(content_index=0, content=thinking))
                        await _emit(on_chunk, TextStart(content_index=1 if thinking else 0))
                    text += part["text"]
                    await _emit(on_chunk, TextDelta(delta=part["text"]))
                elif "functionCall" in part:
                    fc = part["functionCall"]
                    call = ToolCallContent(f"call_{uuid.uuid4().hex[:8]}", fc.get("name", ""), dict(fc.get("args") or {}))
                    calls.append(call)
                    await _emit(on_chunk, ToolCallStart(tool_call_id=call.id, name=call.name))
                    await _emit(on_chunk, ToolCallEnd(tool_call_id=call.id, name=call.name, args=call.arguments))
            fr = cand.get("finishReason")
            if fr:
                stop = {"STOP": "stop", "MAX_TOKENS": "length"}.get(fr, fr.lower())
        u = ev.get("usageMetadata")
        if u:
            usage = Usage(u.get("promptTokenCount", 0), u.get("candidatesTokenCount", 0), u.get("thoughtsTokenCount", 0),
                          u.get("cachedContentTokenCount", 0))
    blocks: list[Any] = []
    if thinking:
        blocks.append(ThinkingContent(thinking))
        if not text:
            await _emit(on_chunk, ThinkingEnd(content_index=0, content=thinking))
    if text or not calls:
        blocks.append(TextContent(text))
    if text:
        await _emit(on_chunk, TextEnd(content_index=1 if thinking else 0, content=text))
    blocks += calls
    if calls:
        stop = "tool_calls"
    return _finish(model, blocks, stop, usage)


# ------------------------------------------------------------------------------------------ rollouts over HTTP
async def _stream_post(url: str, payload: dict[str, Any], headers: dict[str, str], timeout: float, provider: str):
    try:
        import httpx
    except ImportError as e:  # pragma: no cover
        raise NonRetryableError("HTTP providers need the httpx package", provider=provider) from e
    async with httpx.AsyncClient(timeout=timeout) as client:
        async with client.stream("POST", url, json=payload, headers=headers) as r:
            if r.status_code != 200:
                raise classify_http_status(r.status_code, (await r.aread()).decode(errors="replace"), provider)
            async for ev in sse_events(r.aiter_lines()):
                yield ev


def _append(actor: Actor, comp: ChatCompletion) -> Actor:
    msg = comp.choices[0].message
    return replace(actor, trajectory=actor.trajectory.append(msg).with_completion(comp))


async def rollout_anthropic(actor: Actor, run_config: RunConfig) -> Actor:
    ep = actor.endpoint
    from .base import add_cache_control_to_last_content, prepare_messages_for_llm

    system, msgs = messages_to_anthropic(prepare_messages_for_llm(list(actor.trajectory.messages)))
    extra = dict(ep.extra_params)
    if extra.pop("prompt_caching", True):      # a cache break point at the end of the conversation so far (at most four per request)
        msgs = add_cache_control_to_last_content(msgs)
    headers = {"anthropic-version": "2023-06-01", **extra.pop("request_headers", {})}
    payload: dict[str, Any] = {"model": ep.model, "max_tokens": ep.max_tokens, "messages": msgs, "stream": True,
                               "temperature": ep.temperature, **extra}
    if isinstance(payload.get("thinking"), dict) and payload["thinking"].get("type") == "enabled":
        payload["temperature"] = 1.0           # the API accepts no other temperature together with extended thinking
        payload["max_tokens"] = max(payload["max_tokens"], int(payload["thinking"].get("budget_tokens", 0)) + 1024)
    if system:
        payload["system"] = system
    if actor.tools:
        payload["tools"] = [tool_to_anthropic(t) for t in actor.tools]
    token = ep.oauth_token
    app_name = extra.pop("oauth_app", None)
    if app_name:            # a long session outlives an access token: take a fresh one (refreshed when near expiry) per request
        from ..oauth import OAuthApp, OAuthClient, OAuthError

        try:
            token = await OAuthClient(OAuthApp.load(app_name)).get_valid_access_token() or token
        except OAuthError:
            pass
        payload.pop("oauth_app", None)
    if token:
        headers["Authorization"] = f"Bearer {token}"
    else:
        headers["x-api-key"] = ep.api_key
    base = ep.api_base.rstrip("/") or "https://api.anthropic.com"
    events = _stream_post(f"{base}/v1/messages", payload, headers, ep.timeout, "anthropic")
    return _append(actor, await aggregate_anthropic_stream(events, ep.model, run_config.on_chunk))


async def rollout_openai_streaming(actor: Actor, run_config: RunConfig) -> Actor:
    from .chat import messages_to_openai

    ep = actor.endpoint
    payload: dict[str, Any] = {"model": ep.model, "messages": messages_to_openai(actor), "max_tokens": ep.max_tokens,
                               "temperature": ep.temperature, "stream": True, "stream_options": {"include_usage": True},
                               **ep.extra_params}
    if actor.tools:
        payload["tools"] = [t.to_openai() for t in actor.tools]
    headers = {"Authorization": f"Bearer {ep.api_key}"} if ep.api_key else {}
    events = _stream_post(f"{ep.api_base.rstrip('/')}/v1/chat/completions", payload, headers, ep.timeout, ep.provider)
    return _append(actor, await aggregate_openai_stream(events, ep.model, run_config.on_chunk))


async def rollout_openai_responses(actor: Actor, run_config: RunConfig) -> Actor:
    ep = actor.endpoint
    payload: dict[str, Any] = {"model": ep.model, "input": messages_to_openai_responses(actor.trajectory.messages),
                               "max_output_tokens": ep.max_tokens, "stream": True, **ep.extra_params}
    if ep.reasoning_effort:
        payload["reasoning"] = {"effort": ep.reasoning_effort}
    if actor.tools:
        payload["tools"] = [{"type": "function", **t.to_openai()["function"]} for t in actor.tools]
    headers = {"Authorization": f"Bearer {ep.api_key}"}
    base = ep.api_base.rstrip("/") or "https://api.openai.com"
    events = _stream_post(f"{base}/v1/responses", payload, headers, ep.timeout, "openai")
    return _append(actor, await aggregate_openai_responses_stream(events, ep.model, run_config.on_chunk))


async def rollout_google(actor: Actor, run_config: RunConfig) -> Actor:
    ep = actor.endpoint
    system, contents = messages_to_google(actor.trajectory.messages)
    payload: dict[str, Any] = {"contents": contents, "generationConfig": {"maxOutputTokens": ep.max_tokens, "temperature": ep.temperature}}
    if system:
        payload["systemInstruction"] = {"parts": [{"text": system}]}
    if actor.tools:
        payload["tools"] = [{"functionDeclarations": [{"name": t.function.name, "description": t.function.description,
                                                       "parameters": t.to_openai()["function"]["parameters"]} for t in actor.tools]}]
    base = ep.api_base.rstrip("/") or "https://generativelanguage.googleapis.com"
    url = f"{base}/v1beta/models/{ep.model}:streamGenerateContent?alt=sse"
    events = _stream_post(url, payload, {"x-goog-api-key": ep.api_key}, ep.timeout, "google")
    return _append(actor, await aggregate_google_stream(events, ep.model, run_config.on_chunk))
