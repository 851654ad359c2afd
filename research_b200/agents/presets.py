"""Named agent configurations: system prompt + environment factory + turn budget
(rollouts/agent_presets/)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .environments import (AskUserQuestionEnvironment, BasicEnvironment, BrowsingEnvironment, CalculatorEnvironment,
                           ComposedEnvironment, GitWorktreeEnvironment, LocalFilesystemEnvironment, REPLEnvironment)


@dataclass(frozen=True)
class AgentPreset:
    name: str
    description: str
    system_prompt: str
    environment: Callable[[str], Any]       # working directory -> environment
    max_turns: int = 30


_CODING = ("You are a careful software engineer working in the user's repository. Read before you edit, make the "
           "smallest change that solves the task, run the tests, and say plainly what you verified and what you did not.")

PRESETS: dict[str, AgentPreset] = {p.name: p for p in [
    AgentPreset("chat", "plain conversation, no tools", "You are a helpful assistant.", lambda cwd: BasicEnvironment(), 1),
    AgentPreset("calculator", "arithmetic with a calculator tool", "Use the calculator for every computation.",
                lambda cwd: CalculatorEnvironment(), 10),
    AgentPreset("coding", "read / write / edit / bash in the working directory", _CODING,
                lambda cwd: LocalFilesystemEnvironment(cwd), 50),
    AgentPreset("coding-git", "coding in a per-session git worktree with automatic commits", _CODING,
                lambda cwd: GitWorktreeEnvironment(cwd), 50),
    AgentPreset("coding-interactive", "coding plus questions to the user", _CODING + " Ask when requirements are ambiguous.",
                lambda cwd: ComposedEnvironment([LocalFilesystemEnvironment(cwd), AskUserQuestionEnvironment()]), 50),
    AgentPreset("research", "web search / fetch and a Python scratchpad",
                "Answer with sources. Search, read the pages you cite, compute with the REPL when numbers matter.",
                lambda cwd: ComposedEnvironment([BrowsingEnvironment(), REPLEnvironment()]), 30),
]}


def get_preset(name: str) -> AgentPreset:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; available: {sorted(PRESETS)}")
    return PRESETS[name]
