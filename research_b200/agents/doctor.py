"""Session health checks and repairs (rollouts/cli.py:724-909: ``--doctor``, ``--fix``, ``--trim``).

A stored conversation can end up in a shape a provider rejects: the same tool result recorded twice (a retry after a
crash), a tool result whose call is gone (a slice that cut between them), an assistant turn whose tool calls never got
an answer (the process died mid-tool), or one message so large that it fills the context window. ``diagnose`` finds
these; ``fix_session`` and ``trim_session`` never edit a session in place: they write a child session (``parent_id``,
``branch_point``, a ``doctor`` tag) that can be resumed instead.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any

from .dtypes import Message

OVERSIZED_CHARS = 100_000


@dataclass(frozen=True)
class SessionIssue:
    kind: str                      # duplicate_tool_result | orphaned_tool_result | unanswered_tool_call | oversized_message | empty_message
    description: str
    indices: tuple[int, ...] = ()  # messages a fix would drop
    fixable: bool = True


@dataclass
class SessionStats:
    session_id: str
    status: str
    messages: int
    chars: int
    est_tokens: int
    by_role: dict[str, int] = field(default_factory=dict)
    parent_id: str | None = None


def _chars(m: Message) -> int:
    n = len(m.text())
    for c in m.get_tool_calls():
        n += len(str(c.args)) + len(c.name)
    return n


def session_stats(session, messages: list[Message]) -> SessionStats:
    chars = sum(_chars(m) for m in messages)
    roles: dict[str, int] = {}
    for m in messages:
        roles[m.role] = roles.get(m.role, 0) + 1
    return SessionStats(session.session_id, str(session.status), len(messages), chars, chars // 4, roles, session.parent_id)


def diagnose(messages: list[Message], oversized_chars: int = OVERSIZED_CHARS) -> list[SessionIssue]:
    issues: list[SessionIssue] = []
    results: dict[str, list[int]] = {}
    calls: dict[str, int] = {}
    for i, m in enumerate(messages):
        if m.role == "tool" and m.tool_call_id:
            results.setdefault(m.tool_call_id, []).append(i)
        if m.role == "assistant":
            for c in m.get_tool_calls():
                calls[c.id] = i
    for cid, idx in results.items():
        if len(idx) > 1:
            issues.append(SessionIssue("duplicate_tool_result", f"result of call {cid[:24]!r} recorded {len(idx)} times (messages {idx})",
                                       tuple(idx[1:])))
        if cid not in calls:
            issues.append(SessionIssue("orphaned_tool_result", f"result at message {idx[0]} answers call {cid[:24]!r}, which is not in the session",
                                       tuple(idx)))
    for cid, i in calls.items():
        if cid not in results and any(m.role in ("user", "assistant") for m in messages[i + 1:]):
            # the conversation went on without an answer to this call: providers reject that; dropping the assistant
            # turn would lose its text, so this one is reported and left to --trim
            issues.append(SessionIssue("unanswered_tool_call", f"call {cid[:24]!r} at message {i} never got a result", (i,), fixable=False))
    for i, m in enumerate(messages):
        n = _chars(m)
        if n > oversized_chars:
            issues.append(SessionIssue("oversized_message", f"message {i} ({m.role}) has {n:,} characters (about {n // 4:,} tokens)", (i,), fixable=False))
        if m.role == "assistant" and n == 0:
            issues.append(SessionIssue("empty_message", f"assistant message {i} is empty", (i,)))
    return issues


async def _child(store, session, messages: list[Message], tags: dict[str, Any]) -> str:
    sid = await store.create(session.endpoint, session.environment, parent_id=session.session_id, branch_point=len(messages), tags=tags)
    for m in messages:
        await store.append_message(sid, m)
    return sid


async def fix_session(store, session_id: str) -> tuple[str | None, list[int]]:
    """Child session without the messages that the fixable issues name; ``(None, [])`` when there is nothing to fix."""
    session, messages = await store.get(session_id)
    drop = sorted({i for issue in diagnose(messages) if issue.fixable for i in issue.indices})
    if not drop:
        return None, []
    kept = [m for i, m in enumerate(messages) if i not in set(drop)]
    return await _child(store, session, kept, {"doctor": "fixed", "removed_indices": str(drop)}), drop


async def trim_session(store, session_id: str, count: int) -> str:
    """Child session without the last ``count`` messages."""
    session, messages = await store.get(session_id)
    if count <= 0 or count >= len(messages):
        raise ValueError(f"cannot trim {count} of {len(messages)} messages")
    return await _child(store, session, messages[:-count], {"doctor": "trimmed", "trimmed_count": str(count)})


def format_time_ago(ts: float, now: float | None = None) -> str:
    """``just now`` / ``12m ago`` / ``3h ago`` / ``5d ago`` for a POSIX time stamp."""
    s = (time.time() if now is None else now) - float(ts)
    if s < 60:
        return "just now"
    if s < 3600:
        return f"{int(s // 60)}m ago"
    if s < 86400:
        return f"{int(s // 3600)}h ago"
    return f"{int(s // 86400)}d ago"


async def latest_session_id(store) -> str | None:
    sessions = await store.list()
    return max(sessions, key=lambda s: s.updated_at).session_id if sessions else None


def report(stats: SessionStats, issues: list[SessionIssue], messages: list[Message], tail: int = 5) -> str:
    lines = [f"Session: {stats.session_id}", f"  Messages: {stats.messages} ({', '.join(f'{r} {n}' for r, n in sorted(stats.by_role.items()))})",
             f"  Characters: {stats.chars:,}  (about {stats.est_tokens:,} tokens)", f"  Status: {stats.status}"]
    if stats.parent_id:
        lines.append(f"  Parent: {stats.parent_id}")
    if issues:
        lines += ["", f"{len(issues)} issue(s):"] + [f"  [{i.kind}] {i.description}{'' if i.fixable else '  (not auto-fixable: use --trim)'}" for i in issues]
    else:
        lines += ["", "no issues found"]
    if messages and tail:
        lines += ["", f"Last {min(tail, len(messages))} messages:"]
        for m in messages[-tail:]:
            text = m.text().replace("\n", " ")
            lines.append(f"  [{m.role}] {text[:80]}{'...' if len(text) > 80 else ''} ({_chars(m):,} chars)")
    return "\n".join(lines)
