"""Derived from careful_coder_01_01 (parent 01, self 03): read-only exploration. The tool set has no write, edit or
bash, so the agent can be pointed at a repository (also as a sub-agent started from another session's shell) without
being able to change it."""

from dataclasses import replace

from .careful_coder_01_01 import config as parent_config

SUBAGENT_GUIDANCE = """

## Working as an explorer

You cannot modify files. Your product is an explanation: which files matter, how they connect, where a change would go.
Quote paths and line numbers. When the question is broad, start from the entry points (README, main modules, tests).

A session that needs your findings later can start you from its shell and read your answer back:

    research_b200 chat --preset explorer -p "explain how requests reach the scheduler" --no-session -q > notes.md"""

config = replace(parent_config, name="explorer", tools="readonly", max_turns=40, system_prompt=parent_config.system_prompt + SUBAGENT_GUIDANCE,
                 description="read-only exploration of a repository; safe to run as a sub-agent")
