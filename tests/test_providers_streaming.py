"""Stream aggregators and message transforms against recorded event sequences (no network)."""

import asyncio

from research_b200.agents.dtypes import (Message, TextContent, ThinkingContent, ToolCall, ToolCallContent)
from research_b200.agents.providers import (aggregate_anthropic_stream, aggregate_google_stream,
                                            aggregate_openai_responses_stream, aggregate_openai_stream, get_provider,
                                            messages_to_anthropic, messages_to_google, messages_to_openai_responses, sse_events)
from research_b200.agents.transform_messages import transform_messages


async def _aiter(items):
    for x in items:
        yield x


def _run(coro):
    return asyncio.run(coro)


def test_sse_parser():
    async def go():
        lines = ["event: a", 'data: {"x": 1}', "", ": comment", 'data: {"y":', "data: 2}", "", "data: [DONE]", "", 'data: {"z": 3}', ""]
        return [e async for e in sse_events(_aiter(lines))]

    assert _run(go()) == [{"x": 1}, {"y": 2}]


def test_anthropic_stream():
    events = [
        {"type": "message_start", "message": {"id": "msg_1", "usage": {"input_tokens": 12, "cache_read_input_tokens": 4}}},
        {"type": "content_block_start", "index": 0, "content_block": {"type": "thinking", "thinking": ""}},
        {"type": "content_block_delta", "index": 0, "delta": {"type": "thinking_delta", "thinking": "hmm"}},
        {"type": "content_block_delta", "index": 0, "delta": {"type": "signature_delta", "signature": "sig"}},
        {"type": "content_block_stop", "index": 0},
        {"type": "content_block_start", "index": 1, "content_block": {"type": "text", "text": ""}},
        {"type": "content_block_delta", "index": 1, "delta": {"type": "text_delta", "text": "Let me "}},
        {"type": "content_block_delta", "index": 1, "delta": {"type": "text_delta", "text": "compute."}},
        {"type": "content_block_stop", "index": 1},
        {"type": "content_block_start", "index": 2, "content_block": {"type": "tool_use", "id": "tu_1", "name": "calc"}},
        {"type": "content_block_delta", "index": 2, "delta": {"type": "input_json_delta", "partial_json": '{"expr": "1'}},
        {"type": "content_block_delta", "index": 2, "delta": {"type": "input_json_delta", "partial_json": '+1"}'}},
        {"type": "content_block_stop", "index": 2},
        {"type": "message_delta", "delta": {"stop_reason": "tool_use"}, "usage": {"output_tokens": 30}},
        {"type": "message_stop"},
    ]
    seen, partial = [], []

    async def on_chunk(ev):
        seen.append(ev.type)
        if ev.type == "toolcall_delta":
            partial.append(ev.partial_args)

    comp = _run(aggregate_anthropic_stream(_aiter(events), "claude-x", on_chunk))
    msg = comp.choices[0].message
    assert comp.id == "msg_1" and comp.choices[0].finish_reason == "tool_calls"
    assert msg.text() == "Let me compute." and msg.get_tool_calls() == [ToolCall("tu_1", "calc", {"expr": "1+1"})]
    assert isinstance(msg.content[0], ThinkingContent) and msg.content[0].signature == "sig"
    assert comp.usage.input_tokens == 12 and comp.usage.output_tokens == 30 and comp.usage.cache_read_tokens == 4
    assert seen == ["start", "thinking_start", "thinking_delta", "thinking_end", "text_start", "text_delta", "text_delta", "text_end",
                    "tool_call_start", "toolcall_delta", "toolcall_delta", "tool_call_end"]
    assert partial == [{"expr": "1"}, {"expr": "1+1"}]                   # arguments readable while they stream


def test_openai_chat_stream():
    events = [
        {"id": "c1", "choices": [{"delta": {"role": "assistant", "content": "Hi"}}]},
        {"id": "c1", "choices": [{"delta": {"tool_calls": [{"index": 0, "id": "call_a", "function": {"name": "f", "arguments": '{"a"'}}]}}]},
        {"id": "c1", "choices": [{"delta": {"tool_calls": [{"index": 0, "function": {"arguments": ": 1}"}}]}}]},
        {"id": "c1", "choices": [{"delta": {}, "finish_reason": "tool_calls"}]},
        {"id": "c1", "choices": [], "usage": {"prompt_tokens": 5, "completion_tokens": 7}},
    ]
    comp = _run(aggregate_openai_stream(_aiter(events), "gpt-x"))
    assert comp.choices[0].message.text() == "Hi" and comp.choices[0].finish_reason == "tool_calls"
    assert comp.choices[0].message.get_tool_calls() == [ToolCall("call_a", "f", {"a": 1})]
    assert comp.usage.total_tokens == 12


def test_openai_responses_stream():
    events = [
        {"type": "response.created", "response": {"id": "resp_1"}},
        {"type": "response.reasoning_summary_text.delta", "delta": "thinking"},
        {"type": "response.output_text.delta", "delta": "Answer"},
        {"type": "response.output_item.added", "item": {"type": "function_call", "id": "fc_1", "call_id": "call_1", "name": "g", "arguments": ""}},
        {"type": "response.function_call_arguments.delta", "item_id": "fc_1", "delta": '{"q": "x"}'},
        {"type": "response.output_item.done", "item": {"type": "function_call", "id": "fc_1", "call_id": "call_1", "name": "g", "arguments": '{"q": "x"}'}},
        {"type": "response.completed", "response": {"usage": {"input_tokens": 3, "output_tokens": 9, "output_tokens_details": {"reasoning_tokens": 4}}}},
    ]
    comp = _run(aggregate_openai_responses_stream(_aiter(events), "o-x"))
    m = comp.choices[0].message
    assert comp.id == "resp_1" and m.text() == "Answer" and m.get_tool_calls() == [ToolCall("call_1", "g", {"q": "x"})]
    assert comp.usage.reasoning_tokens == 4 and comp.choices[0].finish_reason == "tool_calls"


def test_google_stream():
    events = [
        {"candidates": [{"content": {"parts": [{"text": "plan", "thought": True}]}}]},
        {"candidates": [{"content": {"parts": [{"text": "Hello "}, {"text": "world"}]}}]},
        {"candidates": [{"content": {"parts": [{"functionCall": {"name": "lookup", "args": {"k": 2}}}]}, "finishReason": "STOP"}],
         "usageMetadata": {"promptTokenCount": 8, "candidatesTokenCount": 6, "thoughtsTokenCount": 2}},
    ]
    comp = _run(aggregate_google_stream(_aiter(events), "gemini-x"))
    m = comp.choices[0].message
    assert m.text() == "Hello world" and m.get_tool_calls()[0].name == "lookup" and m.get_tool_calls()[0].args == {"k": 2}
    assert comp.usage.input_tokens == 8 and comp.usage.reasoning_tokens == 2


def test_wire_formats():
    msgs = (Message("system", "be brief"), Message("user", "2+2?"),
            Message("assistant", [TextContent("calling"), ToolCallContent("t1", "calc", {"e": "2+2"})]),
            Message("tool", "4", tool_call_id="t1", name="calc"), Message("user", "thanks"))
    system, a = messages_to_anthropic(msgs)
    assert system == "be brief" and [m["role"] for m in a] == ["user", "assistant", "user"]
    assert a[2]["content"][0]["type"] == "tool_result" and a[2]["content"][1] == {"type": "text", "text": "thanks"}
    system, g = messages_to_google(msgs)
    assert [m["role"] for m in g] == ["user", "model", "user"] and g[2]["parts"][0]["functionResponse"]["name"] == "calc"
    items = messages_to_openai_responses(msgs)
    assert [i["type"] for i in items] == ["message", "message", "message", "function_call", "function_call_output", "message"]
    assert items[0]["role"] == "developer"
    assert get_provider("anthropic").__name__ == "rollout_anthropic"


def test_transform_messages():
    msgs = [Message("user", "q"),
            Message("assistant", [ThinkingContent("secret", "sig"), TextContent("a"), ToolCallContent("t1", "f", {})]),
            Message("tool", "orphan", tool_call_id="zzz"),
            Message("user", "next"), Message("user", "again")]
    out = transform_messages(msgs, source=("anthropic", "m1"), target=("openai", "m2"), require_alternation=True)
    roles = [m.role for m in out]
    assert roles == ["user", "assistant", "tool", "user"]
    assert not any(isinstance(b, ThinkingContent) for b in out[1].content)
    assert out[2].tool_call_id == "t1" and "interrupted" in out[2].text()
    assert out[3].text() == "next\n\nagain"
    same = transform_messages(msgs, source=("anthropic", "m1"), target=("anthropic", "m1"))
    assert isinstance(same[1].content[0], ThinkingContent)
    inl = transform_messages(msgs, source=("a", "1"), target=("b", "2"), inline_thinking="<think>{thinking}</think>")
    assert inl[1].content[0].text == "<think>secret</think>"


def test_provider_request_hygiene_and_errors():
    """Context-overflow parsing in the three providers' wordings, error kinds and advice, log sanitising of inline images,
    prompt-cache markers capped at four, UI-only tool details stripped, cache-aware cost, retry exhaustion wrapped."""
    import asyncio

    import pytest

    from research_b200.agents.dtypes import Message, Usage
    from research_b200.agents.providers import (ContextTooLongError, NonRetryableError, ProviderError, add_cache_control_to_last_content,
                                                 async_retry, calculate_cost_from_usage, classify_http_status, classify_server_error,
                                                 explain_server_error, get_model, get_models, get_providers, parse_context_overflow,
                                                 prepare_messages_for_llm, sanitize_request_for_logging)

    openai_msg = "This model's maximum context length is 8192 tokens. However, you requested 9000 tokens (8000 in the messages, 1000 in the completion)."
    assert parse_context_overflow(openai_msg) == (9000, 8192)
    assert parse_context_overflow("prompt is too long: 210000 tokens > 200000 maximum") == (210000, 200000)
    assert parse_context_overflow("The input token count (1200000) exceeds the maximum number of tokens allowed (1048576).") == (1200000, 1048576)
    assert parse_context_overflow("context window exceeded") == (None, None) and parse_context_overflow("bad json") is None
    err = classify_http_status(400, openai_msg, "vllm")
    assert isinstance(err, ContextTooLongError) and (err.current_tokens, err.max_tokens, err.provider) == (9000, 8192, "vllm")
    assert classify_server_error(200, "") == "success" and classify_server_error(400, "logprobs is not a valid parameter") == "invalid_param"
    assert classify_server_error(429, "slow down") == "rate_limit" and classify_server_error(401, "") == "auth"
    assert classify_server_error(503, "") == "server" and classify_server_error(404, "") == "http_error"
    assert "try 2048" in explain_server_error("context_length", max_tokens=4096) and "echo" in explain_server_error("invalid_param", param_keys=["echo"])
    assert isinstance(classify_http_status(401, ""), NonRetryableError)

    req = {"model": "m", "api_key": "sk-secret", "messages": [
        {"role": "user", "content": [{"type": "image_url", "image_url": {"url": "data:image/png;base64," + "A" * 200_000}},
                                     {"type": "image", "source": {"type": "base64", "data": "B" * 50_000}},
                                     {"type": "text", "text": "x" * 2000}]}]}
    clean = sanitize_request_for_logging(req)
    blob = str(clean)
    assert len(blob) < 1500 and "<image: 200022 bytes>" in blob and "<image: 50000 bytes>" in blob and "(2000 chars total)" in blob
    assert clean["api_key"] == "***" and len(req["messages"][0]["content"][2]["text"]) == 2000      # the original is untouched

    msgs = [{"role": "user", "content": "hello"}]
    marked = add_cache_control_to_last_content(msgs)
    assert marked[0]["content"] == [{"type": "text", "text": "hello", "cache_control": {"type": "ephemeral"}}] and msgs[0]["content"] == "hello"
    four = [{"role": "user", "content": [{"type": "text", "text": str(i), "cache_control": {"type": "ephemeral"}}]} for i in range(4)]
    capped = add_cache_control_to_last_content(four + [{"role": "user", "content": [{"type": "text", "text": "new"}]}])
    assert "cache_control" not in capped[-1]["content"][0]

    tool = Message("tool", "ok", tool_call_id="c1", metadata={"details": {"diff": "x" * 1000}, "kept": 1})
    sent = prepare_messages_for_llm([Message("user", "q"), tool])
    assert len(sent) == 2 and sent[1].metadata == {"kept": 1} and tool.metadata["details"]

    sonnet = get_model("claude-sonnet-4-5")
    cost = calculate_cost_from_usage(Usage(1_000_000, 100_000, cache_read_tokens=2_000_000, cache_write_tokens=500_000), sonnet)
    assert (cost.input, cost.output, cost.cache_read, cost.cache_write) == (3.0, 1.5, pytest.approx(0.6), pytest.approx(1.875))
    assert calculate_cost_from_usage(Usage(10, 10), None).total == 0.0
    assert get_model("gpt-4o-2024-08-06").name == "gpt-4o" and get_model("gpt-4o", provider="anthropic") is None
    assert "anthropic" in get_providers() and all(m.provider == "google" for m in get_models("google"))

    calls = {"n": 0}

    async def nosleep(_):
        return None

    @async_retry(max_attempts=2, sleep=nosleep, wrap_as_provider_error="anthropic")
    async def always_down():
        calls["n"] += 1
        raise ConnectionError("reset")

    with pytest.raises(ProviderError) as ei:
        asyncio.run(always_down())
    assert ei.value.provider == "anthropic" and ei.value.attempts == 2 and isinstance(ei.value.original_error, ConnectionError) and calls["n"] == 2


def test_anthropic_request_credentials_thinking_and_headers(tmp_path, monkeypatch):
    """What leaves for the API: bearer token from a stored log-in (refreshed per request) instead of the key, the
    application's extra headers, temperature forced to 1 with extended thinking, and no private fields in the payload."""
    import time

    from research_b200.agents import oauth
    from research_b200.agents.dtypes import Actor, Endpoint, Message, RunConfig, Trajectory
    from research_b200.agents.providers import streaming

    sent = {}

    async def fake_post(url, payload, headers, timeout, provider):
        sent.update(url=url, payload=payload, headers=headers)
        for ev in ({"type": "message_start", "message": {"id": "m1", "usage": {"input_tokens": 3}}},
                   {"type": "content_block_start", "index": 0, "content_block": {"type": "text", "text": ""}},
                   {"type": "content_block_delta", "index": 0, "delta": {"type": "text_delta", "text": "hi"}},
                   {"type": "content_block_stop", "index": 0},
                   {"type": "message_delta", "delta": {"stop_reason": "end_turn"}, "usage": {"output_tokens": 1}}, {"type": "message_stop"}):
            yield ev

    monkeypatch.setattr(streaming, "_stream_post", fake_post)
    monkeypatch.setattr(oauth, "DEFAULT_DIR", tmp_path)
    for k, v in {"AUTHORIZE_URL": "https://a/x", "TOKEN_URL": "https://a/t", "CLIENT_ID": "c", "REDIRECT_URI": "https://a/cb"}.items():
        monkeypatch.setenv(f"RB_OAUTH_SUB_{k}", v)
    oauth.TokenStorage(tmp_path / "sub.json").save(oauth.OAuthTokens("fresh-token", "rt", time.time() + 3600))
    real = oauth.OAuthClient
    monkeypatch.setattr(oauth, "OAuthClient", lambda app, storage=None, **kw: real(app, storage or oauth.TokenStorage(tmp_path / f"{app.name}.json"), **kw))
    ep = Endpoint(provider="anthropic", model="claude-x", api_key="sk-key", oauth_token="stale-token", temperature=0.3, max_tokens=2000,
                  extra_params={"oauth_app": "sub", "request_headers": {"x-app": "1"}, "thinking": {"type": "enabled", "budget_tokens": 4096}})
    actor = Actor(Trajectory((Message("system", "be brief"), Message("user", "hello"))), ep)
    out = asyncio.run(streaming.rollout_anthropic(actor, RunConfig()))
    assert out.trajectory.messages[-1].text() == "hi"
    h, p = sent["headers"], sent["payload"]
    assert h["Authorization"] == "Bearer fresh-token" and "x-api-key" not in h and h["x-app"] == "1" and h["anthropic-version"]
    assert p["temperature"] == 1.0 and p["max_tokens"] == 5120 and p["thinking"]["budget_tokens"] == 4096 and p["system"] == "be brief"
    assert "oauth_app" not in p and "request_headers" not in p and "prompt_caching" not in p
    # no log-in: the API key travels in its own header
    asyncio.run(streaming.rollout_anthropic(Actor(actor.trajectory, Endpoint(provider="anthropic", model="claude-x", api_key="sk-key")), RunConfig()))
    assert sent["headers"]["x-api-key"] == "sk-key" and "Authorization" not in sent["headers"] and sent["payload"]["temperature"] == 1.0


def test_fine_grained_events_partial_arguments_and_bad_json():
    from research_b200.agents.dtypes import parse_streaming_json
    from research_b200.agents.providers.streaming import aggregate_openai_stream

    for text, want in [('{"foo": "bar"', {"foo": "bar"}), ('{"foo": "bar", "baz":', {"foo": "bar"}), ('{"nested": {"a": 1', {"nested": {"a": 1}}),
                       ('{"arr": [1, 2', {"arr": [1, 2]}), ("", {}), ("{", {}), ('{"path": "src/ma', {"path": "src/ma"}), ('{"a": 1, "b', {"a": 1}),
                       ('{"a": tru', {}), ('{"a": "x\\', {"a": "x"}), ("[1,2", {}), ('{"a": "say \\"hi\\", ok", "b": 2', {"a": 'say "hi", ok', "b": 2}),
                       ('{"a": {"b": [1, {"c": 2}], "d": "e"}, "f', {"a": {"b": [1, {"c": 2}], "d": "e"}})]:
        assert parse_streaming_json(text) == want, text
    chunks = [{"id": "c1", "choices": [{"delta": {"reasoning_content": "think"}}]},
              {"choices": [{"delta": {"content": "Answer"}}]},
              {"choices": [{"delta": {"tool_calls": [{"index": 0, "id": "t1", "function": {"name": "read", "arguments": '{"path": "a'}}]}}]},
              {"choices": [{"delta": {"tool_calls": [{"index": 0, "function": {"arguments": '.py"}'}}]}}]},
              {"choices": [{"delta": {"tool_calls": [{"index": 1, "id": "t2", "function": {"name": "bash", "arguments": "{not json"}}]}, "finish_reason": "tool_calls"}]}]
    seen = []

    async def on_chunk(ev):
        seen.append(ev)

    comp = _run(aggregate_openai_stream(_aiter(chunks), "m", on_chunk))
    kinds = [e.type for e in seen]
    assert kinds == ["start", "thinking_start", "thinking_delta", "thinking_end", "text_start", "text_delta", "tool_call_start", "toolcall_delta",
                     "toolcall_delta", "tool_call_start", "toolcall_delta", "text_end", "tool_call_end", "toolcall_error", "tool_call_end"]
    deltas = [e for e in seen if e.type == "toolcall_delta"]
    assert deltas[0].partial_args == {"path": "a"} and deltas[1].partial_args == {"path": "a.py"} and deltas[2].partial_args == {}
    err = next(e for e in seen if e.type == "toolcall_error")
    assert err.tool_name == "bash" and err.raw_arguments == "{not json" and next(e for e in seen if e.type == "text_end").content == "Answer"
    calls = comp.choices[0].message.get_tool_calls()
    assert calls[0].args == {"path": "a.py"} and calls[1].args == {"_raw": "{not json"}
