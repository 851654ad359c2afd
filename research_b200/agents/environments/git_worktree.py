"""Coding environment in which every session works in its own git worktree and every file-changing
tool call becomes a commit (rollouts/environments/git_worktree.py:61-620).

``on_session_start`` makes sure the working directory is a repository (initial commit if needed),
creates ``<repo>/.rollouts/worktrees/<session>`` on a branch ``rollouts/<session>`` and redirects the
read / write / edit / list / bash tools of the file-system environment there. The history of a
session is then an ordinary branch that can be diffed, merged or thrown away.
"""

from __future__ import annotations

import asyncio
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from ..dtypes import AgentState, RunConfig, Tool, ToolCall, ToolResult
from .coding import LocalFilesystemEnvironment

_GIT_ID = ["-c", "user.name=rollouts", "-c", "user.email=rollouts@localhost"]


@dataclass
class GitWorktreeEnvironment:
    working_dir: str = "."
    session_id: str | None = None
    worktree_path: str | None = None
    allow_bash: bool = True
    commit_count: int = 0

    def get_name(self) -> str:
        return "git_worktree"

    def get_tool_formatter(self, tool_name: str):
        from .coding import TOOL_PRESETS, format_tool

        return format_tool if tool_name in TOOL_PRESETS["full"] else None

    def get_status_info(self) -> dict[str, str] | None:
        if not self.worktree_path:
            return None
        return {"branch": f"rollouts/{self.session_id}", "commits": str(self.commit_count), "cwd": self.worktree_path}

    async def _git(self, args: list[str], cwd: str | Path | None = None) -> str:
        proc = await asyncio.create_subprocess_exec("git", *_GIT_ID, *args, cwd=str(cwd or self.working_dir),
                                                    stdout=asyncio.subprocess.PIPE, stderr=asyncio.subprocess.PIPE)
        out, err = await proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"git {' '.join(args)} failed: {err.decode(errors='replace').strip()}")
        return out.decode(errors="replace").strip()

    async def on_session_start(self, session_id: str) -> None:
        root = Path(self.working_dir).resolve()
        root.mkdir(parents=True, exist_ok=True)
        if not (root / ".git").exists():
            await self._git(["init", "-q"], root)
        try:
            await self._git(["rev-parse", "--verify", "HEAD"], root)
        except RuntimeError:   # empty repository: a worktree needs a commit to branch from
            await self._git(["add", "-A"], root)
            await self._git(["commit", "-q", "--allow-empty", "-m", "initial state"], root)
        self.session_id = session_id
        wt = root / ".rollouts" / "worktrees" / session_id
        if not wt.exists():
            wt.parent.mkdir(parents=True, exist_ok=True)
            exclude = root / ".git" / "info" / "exclude"
            exclude.parent.mkdir(parents=True, exist_ok=True)
            if ".rollouts/" not in (exclude.read_text() if exclude.exists() else ""):
                with exclude.open("a") as f:
                    f.write("\n.rollouts/\n")
            await self._git(["worktree", "add", "-q", "-b", f"rollouts/{session_id}", str(wt)], root)
        self.worktree_path = str(wt)

    def _fs(self) -> LocalFilesystemEnvironment:
        if not self.worktree_path:
            raise RuntimeError("on_session_start() has not been called")
        return LocalFilesystemEnvironment(self.worktree_path, self.allow_bash)

    def get_tools(self) -> list[Tool]:
        return LocalFilesystemEnvironment(self.worktree_path or self.working_dir, self.allow_bash).get_tools()

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return tool_call.name == "bash"

    async def _auto_commit(self, message: str) -> bool:
        if not await self._git(["status", "--porcelain"], self.worktree_path):
            return False
        await self._git(["add", "-A"], self.worktree_path)
        await self._git(["commit", "-q", "-m", message], self.worktree_path)
        self.commit_count += 1
        return True

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        try:
            result = await self._fs().exec_tool(tool_call, state, run_config)
            if tool_call.name in ("write", "edit", "bash") and not (result.is_error and tool_call.name != "bash"):
                target = tool_call.args.get("path") or str(tool_call.args.get("command", ""))[:60]
                await self._auto_commit(f"{tool_call.name}: {target}")
            return result
        except RuntimeError as e:
            return ToolResult(tool_call.id, is_error=True, error=str(e))

    async def diff_against_base(self) -> str:
        """Everything the session changed, as one patch."""
        base = await self._git(["merge-base", "HEAD", f"rollouts/{self.session_id}"], self.working_dir)
        return await self._git(["diff", base, f"rollouts/{self.session_id}"], self.working_dir)

    async def serialize(self) -> dict[str, Any]:
        return {"env_kind": "git_worktree", "working_dir": self.working_dir, "session_id": self.session_id,
                "worktree_path": self.worktree_path, "allow_bash": self.allow_bash, "commit_count": self.commit_count}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "GitWorktreeEnvironment":
        return GitWorktreeEnvironment(data.get("working_dir", "."), data.get("session_id"), data.get("worktree_path"),
                                      data.get("allow_bash", True), int(data.get("commit_count", 0)))
