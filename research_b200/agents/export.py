"""Render a stored session as Markdown or self-contained HTML (rollouts/export.py:24-360)."""

from __future__ import annotations

import html
import json
import time
from typing import Any

from .dtypes import AgentSession, ImageContent, Message, TextContent, ThinkingContent, ToolCallContent

_ROLE_TITLE = {"system": "System", "user": "User", "assistant": "Assistant", "tool": "Tool result"}


def _blocks(m: Message) -> list[Any]:
    blocks = list(m.content) if isinstance(m.content, list) else ([TextContent(m.content)] if m.content else [])
    return blocks + [ToolCallContent(c.id, c.name, c.args) for c in m.tool_calls]


def format_content_block(b: Any) -> str:
    if isinstance(b, TextContent):
        return b.text
    if isinstance(b, ThinkingContent):
        return "> *thinking*\n" + "\n".join("> " + line for line in b.thinking.splitlines())
    if isinstance(b, ToolCallContent):
        return f"**tool call** `{b.name}` (`{b.id}`)\n```json\n{json.dumps(b.arguments, indent=2)}\n```"
    if isinstance(b, ImageContent):
        return f"*[image, {b.mime_type}, {len(b.data)} base64 chars]*"
    return str(b)


def session_to_markdown(session: AgentSession, messages: list[Message], include_metadata: bool = True) -> str:
    out = [f"# Session {session.session_id}", ""]
    if include_metadata:
        out += [f"- created: {time.strftime('%Y-%m-%d %H:%M:%S', time.localtime(session.created_at))}",
                f"- model: {session.endpoint.get('provider', '?')}/{session.endpoint.get('model', '?')}",
                f"- status: {session.status}", f"- messages: {len(messages)}"]
        if session.parent_id:
            out.append(f"- parent: {session.parent_id} (branched at message {session.branch_point})")
        out.append("")
    for i, m in enumerate(messages):
        title = _ROLE_TITLE.get(m.role, m.role)
        if m.role == "tool" and m.name:
            title += f" ({m.name})"
        out += [f"## {i}. {title}", ""]
        body = "\n\n".join(format_content_block(b) for b in _blocks(m))
        out += [f"```\n{body}\n```" if m.role == "tool" else body, ""]
    return "\n".join(out)


_CSS = """body{font-family:system-ui,sans-serif;max-width:60rem;margin:2rem auto;padding:0 1rem;background:#fafafa}
.msg{border-radius:8px;padding:.8rem 1rem;margin:.8rem 0;border:1px solid #ddd;background:#fff}
.user{border-left:4px solid #3b82f6}.assistant{border-left:4px solid #10b981}.tool{border-left:4px solid #f59e0b;background:#fffbeb}
.system{border-left:4px solid #6b7280;color:#374151}.role{font-weight:600;font-size:.85rem;text-transform:uppercase;color:#555}
pre{background:#f3f4f6;padding:.6rem;border-radius:6px;overflow-x:auto;white-space:pre-wrap}
.thinking{color:#6b7280;font-style:italic;border-left:2px solid #d1d5db;padding-left:.6rem}"""


def format_content_html(m: Message) -> str:
    parts = []
    for b in _blocks(m):
        if isinstance(b, TextContent):
            tag = "pre" if m.role == "tool" else "div"
            parts.append(f"<{tag}>{html.escape(b.text)}</{tag}>" if tag == "pre" else
                         "<div>" + html.escape(b.text).replace("\n", "<br>") + "</div>")
        elif isinstance(b, ThinkingContent):
            parts.append(f'<div class="thinking">{html.escape(b.thinking)}</div>')
        elif isinstance(b, ToolCallContent):
            parts.append(f"<div><b>tool call</b> <code>{html.escape(b.name)}</code></div>"
                         f"<pre>{html.escape(json.dumps(b.arguments, indent=2))}</pre>")
        elif isinstance(b, ImageContent):
            parts.append(f'<img alt="image" style="max-width:100%" src="data:{b.mime_type};base64,{b.data}">')
    return "\n".join(parts)


def session_to_html(session: AgentSession, messages: list[Message]) -> str:
    rows = [f'<div class="msg {html.escape(m.role)}"><div class="role">{i}. {html.escape(_ROLE_TITLE.get(m.role, m.role))}'
            f'{" · " + html.escape(m.name) if m.role == "tool" and m.name else ""}</div>{format_content_html(m)}</div>'
            for i, m in enumerate(messages)]
    title = f"Session {html.escape(session.session_id)}"
    meta = html.escape(f"{session.endpoint.get('provider', '?')}/{session.endpoint.get('model', '?')} · {session.status} · {len(messages)} messages")
    return (f"<!doctype html><html><head><meta charset='utf-8'><title>{title}</title><style>{_CSS}</style></head>"
            f"<body><h1>{title}</h1><p>{meta}</p>{''.join(rows)}</body></html>")


async def export_session(store, session_id: str, fmt: str = "md", path: str | None = None) -> str:
    session, messages = await store.get(session_id)
    text = session_to_html(session, messages) if fmt == "html" else session_to_markdown(session, messages)
    if fmt == "ansi":                          # the Markdown export rendered for a terminal
        import shutil

        from ..frontend.widgets import render_markdown

        text = "\n".join(render_markdown(text, min(shutil.get_terminal_size((100, 24)).columns, 120)))
    if path:
        with open(path, "w") as f:
            f.write(text)
    return text


async def handoff_summary(store, session_id: str, goal: str | None = None) -> str:
    """A compact brief for continuing the work in a fresh session: goal, files touched, last exchange."""
    session, messages = await store.get(session_id)
    files = sorted({str(c.args.get("path")) for m in messages for c in m.get_tool_calls() if c.args.get("path")})
    first_user = next((m.text() for m in messages if m.role == "user"), "")
    last = [m for m in messages if m.role in ("user", "assistant") and m.text()][-2:]
    lines = [f"# Handoff from session {session.session_id}", "", f"**Original request:** {first_user[:500]}"]
    if goal:
        lines.append(f"**Goal for the next session:** {goal}")
    if files:
        lines += ["", "**Files touched:**"] + [f"- {f}" for f in files]
    lines += ["", "**Last exchange:**"] + [f"- {m.role}: {m.text()[:400]}" for m in last]
    return "\n".join(lines)
