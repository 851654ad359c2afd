#!/usr/bin/env bash
# Agent presets from the command line (rollouts/examples/preset_usage.sh). A preset bundles a system prompt, an
# environment (tools) and a turn limit; the endpoint is chosen separately.
set -euo pipefail

# plain chat against the in-process engine with a tiny random model (no weights needed)
python -m research_b200.cli chat --provider native --model tiny-qwen2 --preset chat -p "Hello"

# arithmetic with tool calls, tools run without confirmation
python -m research_b200.cli chat --provider native --model tiny-qwen2 --preset calculator -y -p "What is (3 + 4) * 5?"

# coding agent in the current directory against a hosted model (API key from the environment)
# python -m research_b200.cli chat --provider anthropic --model claude-sonnet-4-5 --preset coding --cwd .

# the same inside a per-session git worktree, every tool call committed
# python -m research_b200.cli chat --provider openai --model gpt-4o --preset coding-git --cwd .

# research preset: web search / fetch + Python scratchpad
# python -m research_b200.cli chat --provider openai --model gpt-4o --preset research -p "Who kept Skerry Point lighthouse?"

# sessions are stored; list, show, export and resume them
python -m research_b200.cli sessions list --limit 5
# python -m research_b200.cli chat --session <id> --preset chat
