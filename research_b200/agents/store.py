"""Session persistence: ``session.json`` + append-only ``messages.jsonl`` per session, atomic
metadata writes (tmp + rename), branching, crash logs (rollouts/store.py:39-446)."""

from __future__ import annotations

import json
import os
import time
import traceback
import uuid
from dataclasses import asdict
from pathlib import Path
from typing import Any, Protocol, runtime_checkable

from .dtypes import AgentSession, Message


@runtime_checkable
class SessionStore(Protocol):
    async def create(self, endpoint: dict[str, Any], environment: dict[str, Any] | None = None, parent_id: str | None = None,
                     branch_point: int | None = None, tags: dict[str, Any] | None = None) -> str: ...
    async def get(self, session_id: str) -> tuple[AgentSession, list[Message]]: ...
    async def append_message(self, session_id: str, message: Message) -> None: ...
    async def update(self, session_id: str, **fields: Any) -> None: ...
    async def list(self) -> list[AgentSession]: ...


class FileSessionStore:
    def __init__(self, root: str | Path):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)

    def _dir(self, sid: str) -> Path:
        return self.root / sid

    def _write_meta(self, s: AgentSession) -> None:
        d = self._dir(s.session_id)
        d.mkdir(parents=True, exist_ok=True)
        tmp = d / f".session.json.{os.getpid()}.tmp"
        tmp.write_text(json.dumps(asdict(s), indent=2, default=str))
        os.replace(tmp, d / "session.json")

    def _read_meta(self, sid: str) -> AgentSession:
        return AgentSession(**json.loads((self._dir(sid) / "session.json").read_text()))

    async def create(self, endpoint, environment=None, parent_id=None, branch_point=None, tags=None) -> str:
        sid = f"{time.strftime('%Y%m%d-%H%M%S')}-{uuid.uuid4().hex[:8]}"
        self._write_meta(AgentSession(sid, endpoint=endpoint, environment=environment, parent_id=parent_id,
                                      branch_point=branch_point, tags=tags or {}))
        (self._dir(sid) / "messages.jsonl").touch()
        return sid

    async def get(self, session_id: str) -> tuple[AgentSession, list[Message]]:
        msgs = []
        p = self._dir(session_id) / "messages.jsonl"
        if p.exists():
            for line in p.read_text().splitlines():
                if line.strip():
                    try:
                        msgs.append(Message.from_dict(json.loads(line)))
                    except json.JSONDecodeError:
                        break  # a torn last line from a crash: everything before it is intact
        return self._read_meta(session_id), msgs

    async def append_message(self, session_id: str, message: Message) -> None:
        with open(self._dir(session_id) / "messages.jsonl", "a") as f:
            f.write(json.dumps(message.to_dict()) + "\n")
            f.flush()
            os.fsync(f.fileno())
        s = self._read_meta(session_id)
        s.num_messages += 1
        s.updated_at = time.time()
        self._write_meta(s)

    async def update(self, session_id: str, **fields: Any) -> None:
        s = self._read_meta(session_id)
        for k, v in fields.items():
            setattr(s, k, v)
        s.updated_at = time.time()
        self._write_meta(s)

    def record_config_change(self, session_id: str, what: str, before: Any, after: Any) -> None:
        """A change of model, sampling settings or environment in the middle of a conversation, kept beside the messages
        with the index of the message it took effect after, so that a replay knows which configuration produced which
        turn. The session's own record is brought up to date as well (a resumed session continues with the new one)."""
        s = self._read_meta(session_id)
        with open(self._dir(session_id) / "config_changes.jsonl", "a") as f:
            f.write(json.dumps({"at_message": s.num_messages, "time": time.time(), "what": what, "before": before, "after": after}) + "\n")
        if what == "endpoint" and isinstance(after, dict):
            s.endpoint = after
        elif what == "environment" and isinstance(after, dict):
            s.environment = after
        s.updated_at = time.time()
        self._write_meta(s)

    def config_changes(self, session_id: str) -> list[dict[str, Any]]:
        path = self._dir(session_id) / "config_changes.jsonl"
        if not path.exists():
            return []
        return [json.loads(line) for line in path.read_text().splitlines() if line.strip()]

    async def list(self, filter_tags: dict[str, Any] | None = None, status: str | None = None, limit: int | None = None) -> list[AgentSession]:
        """Sessions, oldest first (ids start with their creation time); optionally only those whose tags contain
        ``filter_tags`` and / or with ``status``; ``limit`` keeps the NEWEST ones. Unreadable folders are skipped."""
        out = []
        for d in sorted(self.root.iterdir()):
            if not (d / "session.json").exists():
                continue
            try:
                s = self._read_meta(d.name)
            except (ValueError, TypeError, OSError):
                continue
            if status is not None and s.status != status:
                continue
            if filter_tags and any(s.tags.get(k) != v for k, v in filter_tags.items()):
                continue
            out.append(s)
        return out[-limit:] if limit else out

    async def list_children(self, parent_id: str) -> list[AgentSession]:
        return [s for s in await self.list() if s.parent_id == parent_id]

    async def lineage(self, session_id: str) -> list[AgentSession]:
        """The session and its ancestors, root first (follows ``parent_id``; a missing ancestor ends the walk)."""
        out, seen = [], set()
        at: str | None = session_id
        while at and at not in seen and (self._dir(at) / "session.json").exists():
            seen.add(at)
            s = self._read_meta(at)
            out.append(s)
            at = s.parent_id
        return out[::-1]

    async def get_latest(self, filter_tags: dict[str, Any] | None = None, status: str | None = None) -> AgentSession | None:
        """The most recently UPDATED session that matches."""
        return max(await self.list(filter_tags, status), key=lambda s: s.updated_at, default=None)

    def get_latest_id_sync(self) -> str | None:
        """For code that is not in an event loop (argument parsing): the id of the most recently updated session."""
        best, best_t = None, -1.0
        for d in self.root.iterdir():
            f = d / "session.json"
            if f.exists() and f.stat().st_mtime > best_t:
                best, best_t = d.name, f.stat().st_mtime
        return best

    def get_config_sync(self, session_id: str) -> dict[str, Any] | None:
        """Endpoint, environment and tags a session was created with (None if there is no such session)."""
        try:
            s = self._read_meta(session_id)
        except (OSError, ValueError, TypeError):
            return None
        return {"endpoint": s.endpoint, "environment": s.environment, "tags": s.tags, "parent_id": s.parent_id}

    async def delete(self, session_id: str) -> bool:
        """Remove one session's folder (its two files, then the folder). Children keep their ``parent_id``; False if
        there was no such session."""
        d = self._dir(session_id)
        if not (d / "session.json").exists() or d.parent != self.root:
            return False
        for f in d.iterdir():
            if f.is_file():
                f.unlink()
        d.rmdir()
        return True

    async def branch(self, session_id: str, at_message: int, reason: str | None = None) -> str:
        """New session that shares the first ``at_message`` messages of ``session_id``; ``reason`` (why the conversation
        forked: an edit, a configuration change, an exploration) is kept in the child's tags."""
        parent, msgs = await self.get(session_id)
        tags = {"branch_reason": reason} if reason else None
        sid = await self.create(parent.endpoint, parent.environment, parent_id=session_id, branch_point=at_message, tags=tags)
        for m in msgs[:at_message]:
            await self.append_message(sid, m)
        return sid

    async def branch_with_edit(self, session_id: str, index: int, new_content: str) -> str:
        """Child session in which message ``index`` says ``new_content`` instead and nothing follows it yet: the
        conversation is replayed from there. The parent keeps the original wording and everything after it."""
        _, msgs = await self.get(session_id)
        if not 0 <= index < len(msgs):
            raise IndexError(f"session {session_id} has {len(msgs)} messages, no message {index}")
        if msgs[index].role not in ("user", "system"):
            raise ValueError(f"message {index} is a {msgs[index].role} message; only user and system messages can be reworded")
        sid = await self.branch(session_id, index, reason="message_edit")
        await self.append_message(sid, Message(msgs[index].role, new_content))
        return sid

    async def root_of(self, session_id: str) -> str:
        return (await self.lineage(session_id))[0].session_id

    async def tree(self, root_id: str) -> dict[str, Any]:
        """``{"session": AgentSession, "children": [subtrees]}`` under ``root_id``, children oldest first."""
        by_parent: dict[str, list[AgentSession]] = {}
        for s in await self.list():
            if s.parent_id:
                by_parent.setdefault(s.parent_id, []).append(s)

        def build(s: AgentSession, seen: frozenset[str]) -> dict[str, Any]:
            kids = sorted(by_parent.get(s.session_id, []), key=lambda c: c.created_at)
            return {"session": s, "children": [build(c, seen | {c.session_id}) for c in kids if c.session_id not in seen]}

        return build(self._read_meta(root_id), frozenset({root_id}))


def format_session_tree(tree: dict[str, Any], current: str | None = None) -> str:
    """The tree as indented lines: id, where it left its parent and why, size, model; ``current`` is marked with ``*``."""
    lines: list[str] = []

    def walk(node: dict[str, Any], prefix: str, last: bool, top: bool) -> None:
        s = node["session"]
        fork = ""
        if s.parent_id is not None:
            fork = f" @{s.branch_point}" + (f" ({s.tags['branch_reason']})" if s.tags.get("branch_reason") else "")
        mark = " *" if s.session_id == current else ""
        lines.append(f"{prefix}{'' if top else ('`-- ' if last else '|-- ')}{s.session_id}{fork}  {s.num_messages} msgs  "
                     f"{s.endpoint.get('model', '?')}  {s.status}{mark}")
        kids = node["children"]
        for i, k in enumerate(kids):
            walk(k, prefix + ("" if top else ("    " if last else "|   ")), i == len(kids) - 1, False)

    walk(tree, "", True, True)
    return "\n".join(lines)


def log_crash(root: str | Path, error: BaseException, context: dict[str, Any] | None = None) -> Path:
    d = Path(root) / "crashes"
    d.mkdir(parents=True, exist_ok=True)
    p = d / f"crash-{time.strftime('%Y%m%d-%H%M%S')}-{uuid.uuid4().hex[:6]}.json"
    p.write_text(json.dumps({"error": f"{type(error).__name__}: {error}",
                             "traceback": "".join(traceback.format_exception(type(error), error, error.__traceback__)),
                             "context": context or {}, "time": time.time()}, indent=2, default=str))
    return p
