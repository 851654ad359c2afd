"""Make a stored conversation acceptable to a different provider or model
(rollouts/transform_messages.py:28-559).

Rules applied in order:
1. thinking blocks are kept only when the target is the same provider+model that produced them
   (their signatures are model-bound); otherwise they are dropped or, if asked, inlined as text;
2. assistant tool calls without a matching tool result get a synthetic error result, and tool
   results whose call is gone are dropped (APIs reject both);
3. image blocks are replaced with a placeholder for targets that cannot take images;
4. consecutive messages of the same role are merged for providers that require alternation.
"""

from __future__ import annotations

from dataclasses import replace

from .dtypes import ImageContent, Message, TextContent, ThinkingContent, ToolCallContent


def _blocks(m: Message) -> list:
    if isinstance(m.content, list):
        return list(m.content)
    return [TextContent(m.content)] if m.content else []


def transform_thinking(messages: list[Message], same_model: bool, inline_template: str | None = None) -> list[Message]:
    out = []
    for m in messages:
        if m.role != "assistant" or not isinstance(m.content, list) or same_model:
            out.append(m)
            continue
        blocks = []
        for b in m.content:
            if isinstance(b, ThinkingContent):
                if inline_template and b.thinking:
                    blocks.append(TextContent(inline_template.format(thinking=b.thinking)))
            else:
                blocks.append(b)
        out.append(replace(m, content=blocks))
    return out


def strip_non_last_thinking(messages: list[Message]) -> list[Message]:
    """Keep thinking only on the last assistant message (earlier reasoning is dead weight in the prompt)."""
    last = max((i for i, m in enumerate(messages) if m.role == "assistant"), default=-1)
    out = []
    for i, m in enumerate(messages):
        if m.role == "assistant" and i != last and isinstance(m.content, list):
            m = replace(m, content=[b for b in m.content if not isinstance(b, ThinkingContent)])
        out.append(m)
    return out


def repair_tool_pairs(messages: list[Message]) -> list[Message]:
    """Every tool call is followed by exactly one result and every result has a call."""
    out: list[Message] = []
    open_calls: dict[str, str] = {}

    def flush() -> None:
        for cid, name in open_calls.items():
            out.append(Message("tool", "Error: tool call was interrupted; no result was recorded.", tool_call_id=cid, name=name))
        open_calls.clear()

    for m in messages:
        if m.role == "tool":
            if m.tool_call_id in open_calls:
                del open_calls[m.tool_call_id]
                out.append(m)
            continue                      # orphaned result: drop
        flush()
        out.append(m)
        if m.role == "assistant":
            for c in m.get_tool_calls():
                open_calls[c.id] = c.name
    flush()
    return out


def replace_images(messages: list[Message], placeholder: str = "[image omitted]") -> list[Message]:
    out = []
    for m in messages:
        if isinstance(m.content, list) and any(isinstance(b, ImageContent) for b in m.content):
            m = replace(m, content=[TextContent(placeholder) if isinstance(b, ImageContent) else b for b in m.content])
        out.append(m)
    return out


def merge_consecutive_messages(messages: list[Message]) -> list[Message]:
    out: list[Message] = []
    for m in messages:
        if out and out[-1].role == m.role and m.role in ("user", "assistant") and not out[-1].get_tool_calls():
            prev = out[-1]
            merged = _blocks(prev) + _blocks(m)
            if all(isinstance(b, TextContent) for b in merged):
                content = "\n\n".join(b.text for b in merged)
                out[-1] = replace(prev, content=content, tool_calls=prev.tool_calls + m.tool_calls)
            else:
                out[-1] = replace(prev, content=merged, tool_calls=prev.tool_calls + m.tool_calls)
        else:
            out.append(m)
    return out


def transform_messages(messages: list[Message], *, source: tuple[str, str] | None = None, target: tuple[str, str] | None = None,
                       supports_images: bool = True, inline_thinking: str | None = None, keep_only_last_thinking: bool = False,
                       require_alternation: bool = False) -> list[Message]:
    """``source`` / ``target`` are ``(provider, model)`` pairs; equal pairs keep thinking blocks intact."""
    msgs = transform_thinking(list(messages), same_model=source is not None and source == target, inline_template=inline_thinking)
    if keep_only_last_thinking:
        msgs = strip_non_last_thinking(msgs)
    msgs = repair_tool_pairs(msgs)
    if not supports_images:
        msgs = replace_images(msgs)
    if require_alternation:
        msgs = merge_consecutive_messages(msgs)
    return [m for m in msgs if m.role == "tool" or m.content or m.get_tool_calls()]


__all__ = ["transform_messages", "transform_thinking", "strip_non_last_thinking", "repair_tool_pairs", "replace_images",
           "merge_consecutive_messages", "ToolCallContent"]
