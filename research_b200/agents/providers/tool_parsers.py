"""Tool-call extraction from raw model text: Hermes ``<tool_call>{json}</tool_call>`` blocks and
bare JSON objects (rollouts/providers/sglang.py:811-961)."""

from __future__ import annotations

import json
import re
import uuid
from typing import Any

from ..dtypes import ToolCall

_HERMES = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.DOTALL)


def _mk(name: str, args: Any) -> ToolCall:
    if isinstance(args, str):
        try:
            args = json.loads(args)
        except json.JSONDecodeError:
            args = {"raw": args}
    return ToolCall(id=f"call_{uuid.uuid4().hex[:10]}", name=name, args=args if isinstance(args, dict) else {"value": args})


def parse_hermes_tool_calls(text: str) -> tuple[str, list[ToolCall]]:
    """Returns (text with the tool-call blocks removed, parsed calls). Malformed blocks are left in the text."""
    calls: list[ToolCall] = []

    def repl(m: re.Match) -> str:
        try:
            obj = json.loads(m.group(1))
            calls.append(_mk(obj["name"], obj.get("arguments", obj.get("parameters", {}))))
            return ""
        except (json.JSONDecodeError, KeyError, TypeError):
            return m.group(0)

    return _HERMES.sub(repl, text).strip(), calls


def parse_json_tool_calls(text: str) -> tuple[str, list[ToolCall]]:
    """A reply that is exactly one JSON object (or list) with ``name`` + ``arguments``."""
    s = text.strip()
    if not (s.startswith("{") or s.startswith("[")):
        return text, []
    try:
        obj = json.loads(s)
    except json.JSONDecodeError:
        return text, []
    items = obj if isinstance(obj, list) else [obj]
    calls = [_mk(o["name"], o.get("arguments", o.get("parameters", {}))) for o in items if isinstance(o, dict) and "name" in o]
    return ("" if calls else text), calls


def parse_tool_calls(text: str) -> tuple[str, list[ToolCall]]:
    rest, calls = parse_hermes_tool_calls(text)
    if calls:
        return rest, calls
    return parse_json_tool_calls(text)


def render_tools_system_prompt(tools: list[Any]) -> str:
    """Hermes-style instruction block listing the available tools."""
    if not tools:
        return ""
    specs = "\n".join(json.dumps(t.to_openai()) for t in tools)
    return ("You may call functions. Available tools:\n<tools>\n" + specs + "\n</tools>\n"
            'To call one, reply with <tool_call>{"name": <name>, "arguments": <json>}</tool_call>.')
