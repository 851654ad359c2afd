"""System prompts assembled at run time (rollouts/prompt.py:25-271): a base prompt for the kind of environment, what
the environment says about itself, the tools it ACTUALLY offers, guidelines that follow from that tool set, where the
agent's own documentation lives, the project's context files, and the date and working directory."""

from __future__ import annotations

from datetime import datetime
from pathlib import Path

from .dtypes import Tool
from .paths import get_docs_dir, get_readme_path, get_version

# looked for in every directory from the working directory up to the root; at most one per directory, in this order
PROJECT_CONTEXT_FILES = ("ROLLOUTS.md", "AGENTS.md", "CLAUDE.md")
MAX_CONTEXT_CHARS = 40_000      # per file: a context file is advice, not a corpus

BASE_PROMPTS = {
    "none": "You are a helpful assistant.",
    "calculator": "You solve arithmetic with the calculator tool: one operation per call, then state the result.",
    "coding": ("You are a careful software engineer working in the user's repository. Read before you edit, make the smallest "
               "change that solves the task, run the tests, and say plainly what you verified and what you did not."),
    "git": ("You are a careful software engineer working in a git worktree of the user's repository; every change you make is "
            "committed there. Read before you edit and keep changes small."),
    "research": "Answer with sources. Search, read the pages you cite, and compute with the REPL when numbers matter.",
}
BASE_PROMPTS["coding-git"] = BASE_PROMPTS["git"]

# one line per well-known tool; anything else shows the description its environment gave
TOOL_DESCRIPTIONS = {
    "read": "read a file (optionally a line range)",
    "write": "create a file or replace its whole content",
    "edit": "replace one exact piece of text in a file",
    "bash": "run a shell command in the working directory",
    "glob": "list files by pattern",
    "grep": "search file contents",
}


def load_project_context(cwd: Path, home: Path | None = None) -> list[tuple[Path, str]]:
    """Context files from the user's configuration folder (``~/.research_b200/``, if any) and from every directory
    between the file-system root and ``cwd``, outermost first, so that the most specific advice comes last."""
    found: list[tuple[Path, str]] = []
    seen: set[Path] = set()

    def take(directory: Path) -> None:
        for name in PROJECT_CONTEXT_FILES:
            f = directory / name
            if f.is_file() and f not in seen:
                try:
                    found.append((f, f.read_text(errors="replace")[:MAX_CONTEXT_CHARS]))
                    seen.add(f)
                except OSError:
                    pass
                return

    take((home or Path.home()) / ".research_b200")
    here = Path(cwd).resolve()
    for directory in reversed([here, *here.parents]):
        take(directory)
    return found


def format_tool_list(tools: list[Tool]) -> str:
    return "\n".join(f"- {t.function.name}: {TOOL_DESCRIPTIONS.get(t.function.name, t.function.description or '')}" for t in tools)


def build_tool_guidelines(tools: list[Tool]) -> list[str]:
    """What follows from the tool set: read-only mode when nothing can write, read-before-edit, edit-vs-write."""
    names = {t.function.name for t in tools}
    can_modify = bool(names & {"write", "edit"})
    out = []
    if "read" in names and not can_modify:
        out.append("You are in READ-ONLY mode" + (" with bash access: use bash only for commands that change nothing (git log, grep, "
                                                  "find); do not modify files." if "bash" in names else ": you cannot modify files."))
    if {"read", "edit"} <= names:
        out.append("Read a file before you edit it: edit needs an exact match of the text it replaces.")
    if {"write", "edit"} <= names:
        out.append("Use edit for local changes; write only for new files or complete rewrites.")
    if "bash" in names and can_modify:
        out.append("After changing code, run the project's tests or the command that shows the change works.")
    return out


def build_self_doc_section() -> str:
    return (f"## About this program (research_b200 {get_version()})\n\nOverview: {get_readme_path()}\nDesign notes and measurements: "
            f"{get_docs_dir()}\n\nIf you are asked what you can do, read these files rather than guess.")


def build_system_prompt(env_name: str, tools: list[Tool], cwd: Path | None = None, base_prompt: str | None = None,
                        env_system_prompt: str | None = None, include_self_docs: bool = True, include_project_context: bool = True,
                        now: datetime | None = None) -> str:
    assert env_name, "env_name required"
    where = Path(cwd) if cwd is not None else Path.cwd()
    parts = [base_prompt or BASE_PROMPTS.get(env_name, BASE_PROMPTS["none"])]
    if env_system_prompt:
        parts.append(env_system_prompt)
    if tools:
        parts.append("Available tools:\n" + format_tool_list(tools))
    rules = build_tool_guidelines(tools)
    if rules:
        parts.append("Guidelines:\n" + "\n".join(f"- {r}" for r in rules))
    if include_self_docs:
        parts.append(build_self_doc_section())
    if include_project_context:
        ctx = load_project_context(where)
        if ctx:
            parts.append("# Project context\n\nContext files found for this directory (outermost first):\n" +
                         "".join(f"\n## {p}\n\n{text}\n" for p, text in ctx))
    parts.append(f"Current time: {(now or datetime.now()).strftime('%Y-%m-%d %H:%M:%S')}\nWorking directory: {where}")
    return "\n\n".join(parts)
