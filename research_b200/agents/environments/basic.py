"""Environments without external dependencies: no tools, calculator, binary search, compose
(rollouts/environments/no_tools.py:21, calculator.py:19, binary_search.py, compose.py:76)."""

from __future__ import annotations

import ast
import operator
from dataclasses import dataclass, field
from typing import Any

from ..dtypes import AgentState, RunConfig, StopReason, Tool, ToolCall, ToolFunction, ToolFunctionParameter, ToolResult


class BasicEnvironment:
    """No tools: the model's first answer ends the episode."""

    def get_tools(self) -> list[Tool]:
        return []

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        return ToolResult(tool_call.id, is_error=True, error=f"no tool named {tool_call.name!r}")

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return False

    async def serialize(self) -> dict[str, Any]:
        return {"type": "basic"}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "BasicEnvironment":
        return BasicEnvironment()


_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv,
        ast.Pow: operator.pow, ast.Mod: operator.mod, ast.FloorDiv: operator.floordiv, ast.USub: operator.neg,
        ast.UAdd: operator.pos}


def safe_eval(expr: str) -> float:
    """Arithmetic only: numbers, + - * / // % ** and parentheses."""
    def ev(node: ast.AST) -> float:
        if isinstance(node, ast.Expression):
            return ev(node.body)
        if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)):
            return node.value
        if isinstance(node, ast.BinOp) and type(node.op) in _OPS:
            a, b = ev(node.left), ev(node.right)
            if isinstance(node.op, ast.Pow) and abs(b) > 64:
                raise ValueError("exponent too large")
            return _OPS[type(node.op)](a, b)
        if isinstance(node, ast.UnaryOp) and type(node.op) in _OPS:
            return _OPS[type(node.op)](ev(node.operand))
        raise ValueError(f"unsupported expression element: {type(node).__name__}")

    return ev(ast.parse(expr, mode="eval"))


def _tool(name: str, desc: str, props: dict[str, Any], required: tuple[str, ...]) -> Tool:
    return Tool(ToolFunction(name, desc, ToolFunctionParameter(props, required)))


@dataclass
class CalculatorEnvironment:
    """Running-value calculator with an explicit ``complete_task`` tool."""

    value: float = 0.0
    history: list[str] = field(default_factory=list)

    def get_tools(self) -> list[Tool]:
        num = {"value": {"type": "number"}}
        return [_tool("add", "Add to the current value", num, ("value",)),
                _tool("subtract", "Subtract from the current value", num, ("value",)),
                _tool("multiply", "Multiply the current value", num, ("value",)),
                _tool("divide", "Divide the current value", num, ("value",)),
                _tool("evaluate", "Evaluate an arithmetic expression", {"expression": {"type": "string"}}, ("expression",)),
                _tool("complete_task", "Finish with a final answer", {"answer": {"type": "number"}}, ())]

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        a = tool_call.args
        try:
            if tool_call.name == "add":
                self.value += float(a["value"])
            elif tool_call.name == "subtract":
                self.value -= float(a["value"])
            elif tool_call.name == "multiply":
                self.value *= float(a["value"])
            elif tool_call.name == "divide":
                if float(a["value"]) == 0:
                    return ToolResult(tool_call.id, is_error=True, error="division by zero")
                self.value /= float(a["value"])
            elif tool_call.name == "evaluate":
                self.value = float(safe_eval(str(a["expression"])))
            elif tool_call.name == "complete_task":
                if "answer" in a:
                    self.value = float(a["answer"])
                return ToolResult(tool_call.id, content=f"final answer: {self.value}", stop_reason=StopReason.TASK_COMPLETED)
            else:
                return ToolResult(tool_call.id, is_error=True, error=f"unknown tool {tool_call.name!r}")
        except (KeyError, ValueError, TypeError, ZeroDivisionError, SyntaxError) as e:
            return ToolResult(tool_call.id, is_error=True, error=f"{type(e).__name__}: {e}")
        self.history.append(f"{tool_call.name}({a}) -> {self.value}")
        return ToolResult(tool_call.id, content=f"current value: {self.value}")

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return False

    async def serialize(self) -> dict[str, Any]:
        return {"type": "calculator", "value": self.value, "history": list(self.history)}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "CalculatorEnvironment":
        return CalculatorEnvironment(float(data.get("value", 0.0)), list(data.get("history", [])))


@dataclass
class BinarySearchEnvironment:
    """Guess a hidden integer with higher/lower feedback."""

    target: int = 42
    low: int = 0
    high: int = 100
    guesses: int = 0
    max_guesses: int = 10

    def get_tools(self) -> list[Tool]:
        return [_tool("guess", f"Guess the number between {self.low} and {self.high}", {"number": {"type": "integer"}}, ("number",))]

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        if tool_call.name != "guess":
            return ToolResult(tool_call.id, is_error=True, error=f"unknown tool {tool_call.name!r}")
        try:
            n = int(tool_call.args["number"])
        except (KeyError, ValueError, TypeError) as e:
            return ToolResult(tool_call.id, is_error=True, error=str(e))
        self.guesses += 1
        if n == self.target:
            return ToolResult(tool_call.id, content=f"correct in {self.guesses} guesses", stop_reason=StopReason.TASK_COMPLETED)
        if self.guesses >= self.max_guesses:
            return ToolResult(tool_call.id, content="out of guesses", stop_reason=StopReason.MAX_TURNS)
        return ToolResult(tool_call.id, content="higher" if n < self.target else "lower")

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return False

    async def serialize(self) -> dict[str, Any]:
        return {"type": "binary_search", "target": self.target, "low": self.low, "high": self.high,
                "guesses": self.guesses, "max_guesses": self.max_guesses}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "BinarySearchEnvironment":
        return BinarySearchEnvironment(**{k: v for k, v in data.items() if k != "type"})


class ComposedEnvironment:
    """Union of several environments; tool names are routed to the one that advertises them."""

    def __init__(self, envs: list[Any]):
        self.envs = list(envs)
        names = [t.function.name for e in self.envs for t in e.get_tools()]
        assert len(names) == len(set(names)), f"duplicate tool names across environments: {names}"

    def get_tools(self) -> list[Tool]:
        return [t for e in self.envs for t in e.get_tools()]

    def _owner(self, name: str):
        for e in self.envs:
            if any(t.function.name == name for t in e.get_tools()):
                return e
        return None

    def get_name(self) -> str:
        return "+".join((getattr(e, "get_name", None) or (lambda e=e: type(e).__name__.replace("Environment", "").lower()))() for e in self.envs)

    def get_system_prompt(self) -> str | None:
        """What the parts say about themselves, in order (parts that say nothing are skipped)."""
        parts = [p for p in ((getattr(e, "get_system_prompt", None) or (lambda: None))() for e in self.envs) if p]
        return "\n\n".join(parts) or None

    async def on_session_start(self, session_id: str) -> None:
        for e in self.envs:
            hook = getattr(e, "on_session_start", None)
            if hook is not None:
                await hook(session_id)

    async def on_assistant_message(self, message, state: AgentState) -> AgentState:
        """Every part that reads assistant messages gets its turn, in order; a part sees (and must return) the COMPOSED
        environment in ``state.environment``. A stop reason set by one part ends the chain."""
        for i, e in enumerate(self.envs):
            hook = getattr(e, "on_assistant_message", None)
            if hook is None:
                continue
            from dataclasses import replace as _replace

            out = await hook(message, _replace(state, environment=e))
            if out.environment is not None and out.environment is not e:
                self.envs[i] = out.environment               # a part may hand back a new copy of itself
            state = _replace(out, environment=self)
            if state.stop is not None:
                break
        return state

    def get_tool_formatter(self, tool_name: str):
        get = getattr(self._owner(tool_name), "get_tool_formatter", None)
        return get(tool_name) if get is not None else None

    def get_status_info(self) -> dict[str, str] | None:
        info: dict[str, str] = {}
        for e in self.envs:
            info.update((getattr(e, "get_status_info", None) or (lambda: None))() or {})
        return info or None

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        e = self._owner(tool_call.name)
        if e is None:
            return ToolResult(tool_call.id, is_error=True, error=f"unknown tool {tool_call.name!r}")
        return await e.exec_tool(tool_call, state, run_config)

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        e = self._owner(tool_call.name)
        return bool(e and e.requires_confirmation(tool_call))

    async def serialize(self) -> dict[str, Any]:
        return {"type": "composed", "envs": [{"cls": f"{type(e).__module__}:{type(e).__name__}", "state": await e.serialize()}
                                             for e in self.envs]}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "ComposedEnvironment":
        import importlib

        envs = []
        for item in data["envs"]:
            mod, cls = item["cls"].split(":")
            envs.append(await getattr(importlib.import_module(mod), cls).deserialize(item["state"]))
        return ComposedEnvironment(envs)


def compose(*environments: Any) -> ComposedEnvironment:
    """``compose(a, b, c)``: one environment with the tools of all; nested compositions are flattened."""
    flat: list[Any] = []
    for e in environments:
        flat += e.envs if isinstance(e, ComposedEnvironment) else [e]
    return ComposedEnvironment(flat)
