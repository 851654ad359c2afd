"""Session slicing: select, summarise, compact and inject messages with a small spec language
(rollouts/slice.py:38-560).

    "0:4, compact:4:60%, summarize:60%:-2:'focus on the failing test', -2:, inject:'now run the tests'"

``range`` segments copy messages, ``compact`` keeps the structure but shrinks tool results,
``summarize`` replaces a span by one message produced by an injectable async summariser, ``inject``
appends a user message. Indices are Python-style (negative allowed) or percentages of the session.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, replace
from typing import Awaitable, Callable

from .dtypes import Message

Summarizer = Callable[[list[Message], str | None], Awaitable[str]]


@dataclass
class SliceSegment:
    type: str                              # range | summarize | compact | inject
    start: int | str | None = None
    end: int | str | None = None
    content: str | None = None
    goal: str | None = None

    @staticmethod
    def resolve(value: int | str | None, total: int, default: int) -> int:
        if value is None:
            return default
        if isinstance(value, str) and value.endswith("%"):
            return total * int(value[:-1]) // 100
        v = int(value)
        return max(0, total + v) if v < 0 else min(v, total)


def _split(spec: str) -> list[str]:
    parts, cur, quote = [], "", ""
    for ch in spec:
        if quote:
            cur += ch
            if ch == quote:
                quote = ""
        elif ch in "'\"":
            quote = ch
            cur += ch
        elif ch == ",":
            parts.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        parts.append(cur.strip())
    return parts


def _idx(s: str | None) -> int | str | None:
    if s is None or s == "":
        return None
    return s if s.endswith("%") else int(s)


_IDX = r"(-?\d*%?)"


def parse_slice_spec(spec: str) -> list[SliceSegment]:
    out = []
    for part in _split(spec):
        m = re.fullmatch(r"inject:\s*(['\"])(.+)\1", part, re.DOTALL)
        if m:
            out.append(SliceSegment("inject", content=m.group(2)))
            continue
        m = re.fullmatch(rf"summarize:\s*{_IDX}:{_IDX}(?::\s*(['\"])(.+)\3)?", part, re.DOTALL)
        if m:
            out.append(SliceSegment("summarize", _idx(m.group(1)), _idx(m.group(2)), goal=m.group(4)))
            continue
        m = re.fullmatch(rf"compact:\s*{_IDX}:{_IDX}", part)
        if m:
            out.append(SliceSegment("compact", _idx(m.group(1)), _idx(m.group(2))))
            continue
        m = re.fullmatch(rf"{_IDX}:{_IDX}", part)
        if m:
            out.append(SliceSegment("range", _idx(m.group(1)), _idx(m.group(2))))
            continue
        raise ValueError(f"invalid slice segment: {part!r}")
    return out


# ------------------------------------------------------------------------------ compaction of tool results
def _tool_name(messages: list[Message], idx: int) -> str | None:
    cid = messages[idx].tool_call_id
    for m in reversed(messages[:idx]):
        for c in m.get_tool_calls():
            if c.id == cid:
                return c.name
    return messages[idx].name


def compact_tool_result(content: str, tool: str | None, max_chars: int = 200) -> str:
    n_lines = content.count("\n") + 1
    if tool == "read":
        return f"[read {n_lines} lines, {len(content)} chars]"
    if tool in ("write", "edit"):
        return content.splitlines()[0][:max_chars] if content else f"[{tool} done]"
    if tool == "bash":
        tail = "\n".join(content.splitlines()[-3:])
        return f"[bash output, {n_lines} lines; last lines]\n{tail[:max_chars]}"
    if tool == "list":
        return f"[{n_lines} entries]"
    return content if len(content) <= max_chars else content[:max_chars] + f"... [{len(content) - max_chars} more chars]"


def compact_messages(messages: list[Message], start: int = 0, end: int | None = None) -> list[Message]:
    """Compact ``messages[start:end]``; the tool that produced a result is looked up in the whole list."""
    end = len(messages) if end is None else end
    out = []
    for i in range(start, end):
        m = messages[i]
        if m.role == "tool" and isinstance(m.content, str):
            m = replace(m, content=compact_tool_result(m.content, _tool_name(messages, i)))
        out.append(m)
    return out


async def plain_summarizer(messages: list[Message], goal: str | None) -> str:
    """Model-free fallback: the first line of every message."""
    lines = [f"- {m.role}: {(m.text() or '[tool calls]').strip().splitlines()[0][:160]}" for m in messages if m.text() or m.get_tool_calls()]
    return (f"(focus: {goal})\n" if goal else "") + "\n".join(lines)


async def apply_slice(messages: list[Message], spec: str | list[SliceSegment], summarizer: Summarizer = plain_summarizer) -> list[Message]:
    segs = parse_slice_spec(spec) if isinstance(spec, str) else spec
    n, out = len(messages), []
    for s in segs:
        if s.type == "inject":
            out.append(Message("user", s.content or ""))
            continue
        a, b = SliceSegment.resolve(s.start, n, 0), SliceSegment.resolve(s.end, n, n)
        span = messages[a:b]
        if s.type == "range":
            out.extend(span)
        elif s.type == "compact":
            out.extend(compact_messages(messages, a, b))
        elif s.type == "summarize" and span:
            text = await summarizer(span, s.goal)
            out.append(Message("user", f"[Summary of messages {a}-{b - 1}]\n{text}"))
    return out


async def slice_session(store, session_id: str, spec: str, summarizer: Summarizer = plain_summarizer) -> str:
    """Create a child session holding the sliced conversation; returns its id."""
    session, messages = await store.get(session_id)
    new = await apply_slice(messages, spec, summarizer)
    child = await store.create(session.endpoint, session.environment, parent_id=session_id, branch_point=len(messages),
                               tags={**session.tags, "slice": spec})
    for m in new:
        await store.append_message(child, m)
    return child
