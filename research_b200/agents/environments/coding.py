"""File-system and REPL environments (rollouts/environments/coding.py:425, repl.py:308-896).

``LocalFilesystemEnvironment`` exposes read / write / edit / list / bash inside a sandbox root
(paths that escape the root are refused; bash asks for confirmation). ``REPLEnvironment`` keeps a
Python namespace across calls and captures stdout; ``MessageParsingREPLEnvironment`` also runs
```python fenced blocks found in the assistant's text.
"""

from __future__ import annotations

import asyncio
import contextlib
import io
import re
import traceback
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from ..dtypes import AgentState, RunConfig, StopReason, Tool, ToolCall, ToolFunction, ToolFunctionParameter, ToolResult


def _tool(name, desc, props, required=()):
    return Tool(ToolFunction(name, desc, ToolFunctionParameter(props, tuple(required))))


@dataclass
class LocalFilesystemEnvironment:
    root: str = "."
    allow_bash: bool = True
    bash_timeout: float = 30.0

    def _resolve(self, rel: str) -> Path:
        root = Path(self.root).resolve()
        p = (root / rel).resolve()
        if root != p and root not in p.parents:
            raise PermissionError(f"path {rel!r} escapes the sandbox root")
        return p

    def get_tools(self) -> list[Tool]:
        s = {"type": "string"}
        tools = [_tool("read", "Read a text file", {"path": s}, ["path"]),
                 _tool("write", "Create or overwrite a file", {"path": s, "content": s}, ["path", "content"]),
                 _tool("edit", "Replace one exact occurrence of old with new", {"path": s, "old": s, "new": s}, ["path", "old", "new"]),
                 _tool("list", "List a directory", {"path": s})]
        if self.allow_bash:
            tools.append(_tool("bash", "Run a shell command in the sandbox root", {"command": s}, ["command"]))
        return tools

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        a, cid = tool_call.args, tool_call.id
        try:
            if tool_call.name == "read":
                return ToolResult(cid, content=self._resolve(a["path"]).read_text())
            if tool_call.name == "write":
                p = self._resolve(a["path"])
                p.parent.mkdir(parents=True, exist_ok=True)
                p.write_text(a["content"])
                return ToolResult(cid, content=f"wrote {len(a['content'])} characters to {a['path']}")
            if tool_call.name == "edit":
                p = self._resolve(a["path"])
                text = p.read_text()
                n = text.count(a["old"])
                if n != 1:
                    return ToolResult(cid, is_error=True, error=f"expected exactly one occurrence of the old text, found {n}")
                p.write_text(text.replace(a["old"], a["new"], 1))
                return ToolResult(cid, content=f"edited {a['path']}")
            if tool_call.name == "list":
                p = self._resolve(a.get("path", "."))
                return ToolResult(cid, content="\n".join(sorted(x.name + ("/" if x.is_dir() else "") for x in p.iterdir())))
            if tool_call.name == "bash" and self.allow_bash:
                proc = await asyncio.create_subprocess_shell(a["command"], cwd=str(Path(self.root).resolve()),
                                                             stdout=asyncio.subprocess.PIPE, stderr=asyncio.subprocess.STDOUT)
                try:
                    out, _ = await asyncio.wait_for(proc.communicate(), self.bash_timeout)
                except asyncio.TimeoutError:
                    proc.kill()  # the child this call started
                    return ToolResult(cid, is_error=True, error=f"command timed out after {self.bash_timeout}s")
                text = out.decode(errors="replace")[-20000:]
                return ToolResult(cid, content=text, is_error=proc.returncode != 0, error=text if proc.returncode else None)
            return ToolResult(cid, is_error=True, error=f"unknown tool {tool_call.name!r}")
        except (OSError, KeyError, PermissionError) as e:
            return ToolResult(cid, is_error=True, error=f"{type(e).__name__}: {e}")

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return tool_call.name == "bash"

    async def serialize(self) -> dict[str, Any]:
        return {"type": "filesystem", "root": self.root, "allow_bash": self.allow_bash, "bash_timeout": self.bash_timeout}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "LocalFilesystemEnvironment":
        return LocalFilesystemEnvironment(data.get("root", "."), data.get("allow_bash", True), data.get("bash_timeout", 30.0))


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
