"""Import coding-assistant transcripts stored as JSONL under ``~/.claude/projects/<encoded path>/``
into the session store (rollouts/import_cc.py:39-366).

A project directory name is the absolute project path with ``/`` replaced by ``-``. Each line of a
session file is one event; ``user`` and ``assistant`` events carry an API-style message whose
content is a string or a list of ``text`` / ``thinking`` / ``tool_use`` / ``tool_result`` blocks.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .dtypes import Message, TextContent, ThinkingContent, ToolCallContent


def encode_project_path(path: Path) -> str:
    return str(path.resolve()).replace("/", "-")


def decode_project_path(encoded: str) -> Path:
    return Path("/" + encoded.lstrip("-").replace("-", "/"))


@dataclass
class TranscriptSession:
    session_id: str
    path: Path
    num_events: int
    first_user_message: str
    modified: float


def transcripts_root() -> Path:
    return Path.home() / ".claude" / "projects"


def list_projects(root: Path | None = None) -> list[tuple[str, Path]]:
    root = root or transcripts_root()
    if not root.is_dir():
        return []
    return sorted((d.name, decode_project_path(d.name)) for d in root.iterdir() if d.is_dir())


def list_sessions(project: Path, root: Path | None = None) -> list[TranscriptSession]:
    d = (root or transcripts_root()) / encode_project_path(project)
    out = []
    for f in sorted(d.glob("*.jsonl")) if d.is_dir() else []:
        first, n = "", 0
        for line in f.read_text().splitlines():
            if not line.strip():
                continue
            n += 1
            if not first:
                try:
                    ev = json.loads(line)
                except json.JSONDecodeError:
                    continue
                if ev.get("type") == "user":
                    c = ev.get("message", {}).get("content")
                    first = c if isinstance(c, str) else next((b.get("text", "") for b in c or [] if b.get("type") == "text"), "")
        out.append(TranscriptSession(f.stem, f, n, first[:200], f.stat().st_mtime))
    return out


def _tool_result_text(block: dict[str, Any]) -> str:
    c = block.get("content")
    if isinstance(c, list):
        c = "\n".join(x.get("text", "") for x in c if isinstance(x, dict))
    return ("Error: " if block.get("is_error") else "") + (c or "")


def parse_transcript(path: Path) -> tuple[list[Message], dict[str, Any]]:
    """Returns messages plus metadata (model, cwd, counts). Tool results become ``tool`` messages."""
    messages: list[Message] = []
    meta: dict[str, Any] = {"source": str(path), "skipped": 0}
    names: dict[str, str] = {}
    for line in path.read_text().splitlines():
        if not line.strip():
            continue
        try:
            ev = json.loads(line)
        except json.JSONDecodeError:
            meta["skipped"] += 1
            continue
        if ev.get("type") not in ("user", "assistant") or ev.get("isMeta"):
            continue
        msg = ev.get("message", {})
        meta.setdefault("cwd", ev.get("cwd"))
        if msg.get("model"):
            meta["model"] = msg["model"]
        content = msg.get("content")
        if isinstance(content, str):
            messages.append(Message(ev["type"], content))
            continue
        blocks: list[Any] = []
        for b in content or []:
            t = b.get("type")
            if t == "text":
                blocks.append(TextContent(b.get("text", "")))
            elif t == "thinking":
                blocks.append(ThinkingContent(b.get("thinking", ""), b.get("signature")))
            elif t == "tool_use":
                names[b["id"]] = b.get("name", "")
                blocks.append(ToolCallContent(b["id"], b.get("name", ""), b.get("input", {})))
            elif t == "tool_result":
                messages.append(Message("tool", _tool_result_text(b), tool_call_id=b.get("tool_use_id"),
                                        name=names.get(b.get("tool_use_id", ""))))
        if blocks:
            only_text = all(isinstance(b, TextContent) for b in blocks)
            messages.append(Message(ev["type"], "".join(b.text for b in blocks) if only_text else blocks))
    meta["num_messages"] = len(messages)
    return messages, meta


async def import_transcript(store, path: Path, provider: str = "anthropic") -> str:
    """Create a session in ``store`` from a transcript file; returns the new session id."""
    messages, meta = parse_transcript(path)
    sid = await store.create({"provider": provider, "model": meta.get("model", "")}, None, tags={"imported_from": str(path)})
    for m in messages:
        await store.append_message(sid, m)
    return sid
