"""File-system and REPL environments (rollouts/environments/coding.py:425, repl.py:308-896).

``LocalFilesystemEnvironment`` exposes read (offset / limit, long files and lines cut with a note on how to go on) /
write / edit (exact single match, answers with a diff) / list / glob / grep / bash (own process group, per-call
timeout) / web_fetch inside a sandbox root (paths that escape the root are refused; bash asks for confirmation); the
tool set is a preset or a list, and ``format_tool`` renders a call and its result for the front ends. ``REPLEnvironment`` keeps a
Python namespace across calls and captures stdout; ``MessageParsingREPLEnvironment`` also runs
```python fenced blocks found in the assistant's text.
"""

from __future__ import annotations

import asyncio
import contextlib
import io
import re
import traceback
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Any

from ..dtypes import AgentState, RunConfig, StopReason, Tool, ToolCall, ToolFunction, ToolFunctionParameter, ToolResult


def _tool(name, desc, props, required=()):
    return Tool(ToolFunction(name, desc, ToolFunctionParameter(props, tuple(required))))


IMAGE_TYPES = {".png": "image/png", ".jpg": "image/jpeg", ".jpeg": "image/jpeg", ".gif": "image/gif", ".webp": "image/webp"}
MAX_IMAGE_BYTES = 5 << 20


def sniff_image(path: Path) -> str | None:
    """The image type by the file's first bytes (a wrongly named file is still recognised; a text file called .png is
    not taken for a picture); None for anything else."""
    try:
        with open(path, "rb") as f:
            head = f.read(16)
    except OSError:
        return None
    if head.startswith(b"\x89PNG\r\n\x1a\n"):
        return "image/png"
    if head.startswith(b"\xff\xd8\xff"):
        return "image/jpeg"
    if head.startswith((b"GIF87a", b"GIF89a")):
        return "image/gif"
    if head[:4] == b"RIFF" and head[8:12] == b"WEBP":
        return "image/webp"
    return None
MAX_READ_LINES = 2000
MAX_LINE_CHARS = 2000
MAX_BASH_CHARS = 30_000
TOOL_PRESETS = {"full": ("read", "write", "edit", "list", "glob", "grep", "bash", "web_fetch"),
                "readonly": ("read", "list", "glob", "grep"),
                "no-write": ("read", "list", "glob", "grep", "bash", "web_fetch")}


def unified_diff(old: str, new: str, path: str = "", context: int = 3) -> str:
    import difflib

    return "".join(difflib.unified_diff(old.splitlines(keepends=True), new.splitlines(keepends=True), f"a/{path}", f"b/{path}", n=context))


def _first_lines(text: str, n: int) -> str:
    lines = text.expandtabs(4).splitlines()               # tabs would break the alignment of boxes and diffs
    return "\n".join(lines[:n]) + (f"\n... ({len(lines) - n} more lines)" if len(lines) > n else "")


def format_tool(name: str, args: dict[str, Any], result: ToolResult | None = None, expanded: bool = False) -> str:
    """One tool call as a front end shows it: a header line that reads like the action (``$ ls``, ``read a.py:10-60``,
    ``edit a.py``) and, once there is a result, a body cut to a few lines unless ``expanded`` (the diff for an edit, the
    command's output for bash, the line count for a read)."""
    n = 10**6 if expanded else 12
    if name == "bash":
        head = f"$ {args.get('command', '')}"
    elif name == "read":
        rng = f":{args['offset']}" + (f"-{args['offset'] + args['limit'] - 1}" if args.get("limit") else "") if args.get("offset") else ""
        head = f"read {args.get('path', '')}{rng}"
    elif name in ("write", "edit", "list", "glob", "grep", "web_fetch"):
        what = args.get("path") or args.get("pattern") or args.get("url") or ""
        head = f"{name} {what}" + (f" ({len(str(args.get('content', '')).splitlines())} lines)" if name == "write" else "")
    else:
        head = f"{name}({', '.join(f'{k}={v!r}' for k, v in args.items())})"
    if result is None:
        return head
    if result.is_error:
        return f"{head}\n  error: {_first_lines(result.error or result.content, n)}"
    if name == "read" and not expanded:
        return f"{head}\n  {len(result.content.splitlines())} lines"
    body = result.metadata.get("diff") if name == "edit" and result.metadata.get("diff") else result.content
    return f"{head}\n" + "\n".join("  " + ln for ln in _first_lines(body, n).splitlines())


@dataclass
class LocalFilesystemEnvironment:
    """``tools``: a preset (``full`` / ``readonly`` / ``no-write``) or a list of tool names. ``sandbox``: refuse paths
    outside ``root`` (on by default; off gives the agent the user's whole file system, ``~`` included)."""

    root: str = "."
    allow_bash: bool = True
    bash_timeout: float = 120.0
    tools: str | list[str] | tuple[str, ...] = "full"
    sandbox: bool = True
    fetcher: Any = None                 # async url -> (status, content_type, body); default: urllib

    def __post_init__(self) -> None:
        if isinstance(self.tools, str):
            if self.tools not in TOOL_PRESETS:
                raise ValueError(f"unknown tool preset {self.tools!r}; available: {sorted(TOOL_PRESETS)}")
            names = TOOL_PRESETS[self.tools]
        else:
            unknown = set(self.tools) - set(TOOL_PRESETS["full"])
            if unknown:
                raise ValueError(f"unknown tools {sorted(unknown)}; available: {list(TOOL_PRESETS['full'])}")
            names = tuple(self.tools)
        self._names = tuple(n for n in names if self.allow_bash or n != "bash")

    def get_name(self) -> str:
        return "coding"

    def get_status_info(self) -> dict[str, str] | None:
        cwd, home = str(Path(self.root).resolve()), str(Path.home())
        return {"cwd": "~" + cwd[len(home):] if cwd == home or cwd.startswith(home + "/") else cwd}

    def get_tool_formatter(self, tool_name: str):
        return format_tool if tool_name in TOOL_PRESETS["full"] else None

    def _resolve(self, rel: str) -> Path:
        root = Path(self.root).resolve()
        p = Path(rel).expanduser()
        p = (p if p.is_absolute() else root / p).resolve()
        if self.sandbox and root != p and root not in p.parents:
            raise PermissionError(f"path {rel!r} escapes the sandbox root")
        return p

    def get_tools(self) -> list[Tool]:
        s, i = {"type": "string"}, {"type": "integer"}
        every = {
            "read": _tool("read", f"Read a text file (first {MAX_READ_LINES} lines; offset / limit, 1-based, for the rest)",
                          {"path": s, "offset": i, "limit": i}, ["path"]),
            "write": _tool("write", "Create a file or replace its whole content (parent folders are created)", {"path": s, "content": s}, ["path", "content"]),
            "edit": _tool("edit", "Replace one exact occurrence of old with new (the text must match exactly, whitespace included)",
                          {"path": s, "old": s, "new": s}, ["path", "old", "new"]),
            "list": _tool("list", "List a directory", {"path": s}),
            "glob": _tool("glob", "Files matching a pattern such as **/*.py, newest first", {"pattern": s, "path": s}, ["pattern"]),
            "grep": _tool("grep", "Lines matching a regular expression, as path:line:text", {"pattern": s, "path": s, "glob": s, "max_results": i}, ["pattern"]),
            "bash": _tool("bash", "Run a shell command in the working directory", {"command": s, "timeout": {"type": "number"}}, ["command"]),
            "web_fetch": _tool("web_fetch", "Fetch an http(s) URL and return its text", {"url": s}, ["url"]),
        }
        return [every[n] for n in self._names]

    # ---- tools
    def _read(self, a: dict[str, Any]) -> "str | ToolResult":
        p = self._resolve(a["path"])
        if not p.exists():
            raise FileNotFoundError(f"file not found: {a['path']}")
        if not p.is_file():
            raise IsADirectoryError(f"not a file: {a['path']}")
        mime = sniff_image(p)
        if mime is not None:
            # an image is handed to the model as an image block (the agent loop attaches it to the tool message)
            import base64

            size = p.stat().st_size
            if size > MAX_IMAGE_BYTES:
                raise ValueError(f"image too large to attach: {size} bytes (limit {MAX_IMAGE_BYTES})")
            return ToolResult("", content=f"[image {a['path']}, {size} bytes]",
                              metadata={"image": {"data": base64.b64encode(p.read_bytes()).decode(), "mime_type": mime}})
        try:
            lines = p.read_text(encoding="utf-8").split("\n")
        except UnicodeDecodeError:
            raise ValueError(f"cannot read binary file: {a['path']}") from None
        start = max(int(a.get("offset") or 1) - 1, 0)
        if start >= len(lines) and lines != [""]:
            raise ValueError(f"offset {a.get('offset')} is beyond the end of the file ({len(lines)} lines)")
        end = min(start + int(a.get("limit") or MAX_READ_LINES), len(lines))
        cut = any(len(ln) > MAX_LINE_CHARS for ln in lines[start:end])
        text = "\n".join(ln[:MAX_LINE_CHARS] for ln in lines[start:end])
        notes = ([f"some lines were cut to {MAX_LINE_CHARS} characters"] if cut else []) + \
                ([f"{len(lines) - end} more lines not shown: continue with offset={end + 1}"] if end < len(lines) else [])
        return text + (f"\n\n... ({'; '.join(notes)})" if notes else "")

    def _edit(self, cid: str, a: dict[str, Any]) -> ToolResult:
        p = self._resolve(a["path"])
        old, new = a.get("old", a.get("old_text")), a.get("new", a.get("new_text"))
        if old is None or new is None:
            raise KeyError("old / new")
        text = p.read_text()
        n = text.count(old)
        if n != 1:
            hint = " (check whitespace and line endings; read the file again)" if n == 0 else " (add surrounding lines to make it unique)"
            return ToolResult(cid, is_error=True, error=f"expected exactly one occurrence of the old text, found {n}{hint}")
        if old == new:
            return ToolResult(cid, is_error=True, error="old and new are identical: nothing to change")
        after = text.replace(old, new, 1)
        p.write_text(after)
        return ToolResult(cid, content=f"edited {a['path']}", metadata={"diff": unified_diff(text, after, a["path"])})

    def _glob(self, a: dict[str, Any]) -> str:
        base = self._resolve(a.get("path", "."))
        hits = sorted((p for p in base.glob(a["pattern"]) if p.is_file() and ".git" not in p.parts), key=lambda p: p.stat().st_mtime, reverse=True)
        root = Path(self.root).resolve()
        shown = [str(p.relative_to(root)) if root in p.parents else str(p) for p in hits[:200]]
        return "\n".join(shown) + (f"\n... ({len(hits) - 200} more)" if len(hits) > 200 else "") or "(no files match)"

    def _grep(self, a: dict[str, Any]) -> str:
        rx = re.compile(a["pattern"])
        base, limit = self._resolve(a.get("path", ".")), int(a.get("max_results") or 200)
        files = [base] if base.is_file() else (p for p in sorted(base.rglob(a.get("glob") or "*")) if p.is_file() and ".git" not in p.parts)
        root, out = Path(self.root).resolve(), []
        for f in files:
            try:
                text = f.read_text(encoding="utf-8")
            except (UnicodeDecodeError, OSError):
                continue
            rel = str(f.relative_to(root)) if root in f.parents else str(f)
            for no, line in enumerate(text.splitlines(), 1):
                if rx.search(line):
                    out.append(f"{rel}:{no}:{line[:300]}")
                    if len(out) >= limit:
                        return "\n".join(out) + f"\n... (stopped at {limit} matches)"
        return "\n".join(out) or "(no matches)"

    async def _bash(self, cid: str, a: dict[str, Any]) -> ToolResult:
        import os
        import signal

        limit = float(a.get("timeout") or self.bash_timeout)
        proc = await asyncio.create_subprocess_shell(a["command"], cwd=str(Path(self.root).resolve()), stdout=asyncio.subprocess.PIPE,
                                                     stderr=asyncio.subprocess.STDOUT, start_new_session=True)
        try:
            out, _ = await asyncio.wait_for(proc.communicate(), limit)
        except asyncio.TimeoutError:
            try:
                os.killpg(proc.pid, signal.SIGKILL)      # the group this call started: the shell and what it spawned
            except ProcessLookupError:
                pass
            await proc.wait()
            return ToolResult(cid, is_error=True, error=f"command timed out after {limit:g}s")
        text = out.decode(errors="replace")
        if len(text) > MAX_BASH_CHARS:
            text = f"... ({len(text) - MAX_BASH_CHARS} earlier characters cut)\n" + text[-MAX_BASH_CHARS:]
        if proc.returncode:
            return ToolResult(cid, content=text, is_error=True, error=f"{text}\n(exit code {proc.returncode})".lstrip())
        return ToolResult(cid, content=text or "(no output)")

    async def _web_fetch(self, a: dict[str, Any]) -> str:
        from .interactive import html_to_text, urllib_fetch

        url = str(a["url"])
        if not url.startswith(("http://", "https://")):
            raise ValueError("only http(s) URLs can be fetched")
        status, ctype, body = await (self.fetcher or urllib_fetch)(url)
        if status != 200:
            raise OSError(f"HTTP {status} for {url}")
        text = html_to_text(body) if "html" in ctype.lower() or body.lstrip()[:1] == "<" else body
        return text[:50_000] + (f"\n... ({len(text) - 50_000} more characters)" if len(text) > 50_000 else "")

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        a, cid, name = tool_call.args, tool_call.id, tool_call.name
        if name not in self._names:
            return ToolResult(cid, is_error=True, error=f"unknown tool {name!r}" if name not in TOOL_PRESETS["full"] else f"tool {name!r} is not enabled here")
        try:
            if name == "read":
                got = self._read(a)
                return replace(got, tool_call_id=cid) if isinstance(got, ToolResult) else ToolResult(cid, content=got)
            if name == "write":
                p = self._resolve(a["path"])
                before = p.read_text() if p.is_file() else None
                p.parent.mkdir(parents=True, exist_ok=True)
                p.write_text(a["content"])
                return ToolResult(cid, content=f"wrote {len(a['content'])} characters to {a['path']}",
                                  metadata={"diff": unified_diff(before, a["content"], a["path"])} if before is not None else {"created": True})
            if name == "edit":
                return self._edit(cid, a)
            if name == "list":
                p = self._resolve(a.get("path", "."))
                return ToolResult(cid, content="\n".join(sorted(x.name + ("/" if x.is_dir() else "") for x in p.iterdir())))
            if name == "glob":
                return ToolResult(cid, content=self._glob(a))
            if name == "grep":
                return ToolResult(cid, content=self._grep(a))
            if name == "bash":
                return await self._bash(cid, a)
            return ToolResult(cid, content=await self._web_fetch(a))
        except (OSError, KeyError, ValueError, re.error) as e:      # PermissionError, FileNotFoundError are OSErrors
            return ToolResult(cid, is_error=True, error=f"{type(e).__name__}: {e}")

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return tool_call.name == "bash"

    async def serialize(self) -> dict[str, Any]:
        return {"type": "filesystem", "root": self.root, "allow_bash": self.allow_bash, "bash_timeout": self.bash_timeout,
                "tools": self.tools if isinstance(self.tools, str) else list(self.tools), "sandbox": self.sandbox}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "LocalFilesystemEnvironment":
        return LocalFilesystemEnvironment(data.get("root", "."), data.get("allow_bash", True), data.get("bash_timeout", 120.0),
                                          data.get("tools", "full"), data.get("sandbox", True))


@dataclass
class REPLEnvironment:
    """Persistent Python namespace. ``FINAL(value)`` inside the code ends the episode."""

    namespace: dict[str, Any] = field(default_factory=dict)
    max_output: int = 8000
    final_answer: Any = None
    llm_query: Any = None        # optional callable the code may use as llm_query(prompt)

    def get_tools(self) -> list[Tool]:
        return [_tool("python", "Execute Python; variables persist between calls; print() to see values",
                      {"code": {"type": "string"}}, ["code"])]

    def run_code(self, code: str) -> tuple[str, bool]:
        buf = io.StringIO()
        done = {}

        def FINAL(v: Any) -> None:
            done["v"] = v

        self.namespace.setdefault("__builtins__", __builtins__)
        self.namespace["FINAL"] = FINAL
        if self.llm_query is not None:
            self.namespace["llm_query"] = self.llm_query
        ok = True
        with contextlib.redirect_stdout(buf):
            try:
                exec(compile(code, "<repl>", "exec"), self.namespace)  # noqa: S102 - the purpose of a REPL tool
            except Exception:  # noqa: BLE001
                ok = False
                buf.write(traceback.format_exc(limit=3))
        if "v" in done:
            self.final_answer = done["v"]
        return buf.getvalue()[-self.max_output:], ok

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        if tool_call.name != "python":
            return ToolResult(tool_call.id, is_error=True, error=f"unknown tool {tool_call.name!r}")
        out, ok = self.run_code(str(tool_call.args.get("code", "")))
        stop = StopReason.TASK_COMPLETED if self.final_answer is not None else None
        return ToolResult(tool_call.id, content=out or "(no output)", is_error=not ok, error=None if ok else out, stop_reason=stop)

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return False

    async def serialize(self) -> dict[str, Any]:
        simple = {k: v for k, v in self.namespace.items()
                  if isinstance(v, (int, float, str, bool, list, dict, tuple, type(None))) and not k.startswith("__")}
        return {"type": "repl", "namespace": simple, "final_answer": self.final_answer if isinstance(self.final_answer, (int, float, str, bool, type(None))) else repr(self.final_answer)}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "REPLEnvironment":
        e = REPLEnvironment(dict(data.get("namespace", {})))
        e.final_answer = data.get("final_answer")
        return e


_FENCE = re.compile(r"```(?:python|py)\n(.*?)```", re.DOTALL)


class MessageParsingREPLEnvironment(REPLEnvironment):
    """For models without tool calling: runs fenced python blocks found in the reply text."""

    def extract_code_blocks(self, text: str) -> list[str]:
        return [m.group(1) for m in _FENCE.finditer(text)]

    def run_message(self, text: str) -> str:
        return "\n".join(self.run_code(b)[0] for b in self.extract_code_blocks(text))
