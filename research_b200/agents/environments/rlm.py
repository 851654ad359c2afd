"""Recursive-language-model environment (rollouts/environments/repl.py:308-1038): the long input lives in a Python
variable ``context`` instead of the conversation, and the model works on it with four tools:

* ``repl(code)``: run Python in a namespace that persists between calls and holds ``context``, ``llm_query(prompt)``
  and ``agent(task, context=None)`` as plain functions, so that a loop over chunks can ask a model about each one;
* ``llm_query(prompt)``: one question to the sub-model, no tools;
* ``agent(task, context)``: a sub-agent of the same kind over ``context`` (one level deeper, up to ``max_depth``);
* ``final_answer(answer)``: ends the episode.

Code runs in a worker thread; ``llm_query`` / ``agent`` called from that code are handed back to the event loop and
waited for, so nested model calls work from inside user code without blocking the loop. ``MessageParsingRLMEnvironment``
is the same for models without tool calling: it runs ```repl fenced blocks found in the reply and takes
``FINAL(...)`` / ``FINAL_VAR(name)`` written in the text as the answer.
"""

from __future__ import annotations

import asyncio
import io
import re
import traceback
from dataclasses import dataclass, field, replace
from typing import Any

from ..dtypes import (Actor, AgentState, Endpoint, Message, RunConfig, StopReason, Tool, ToolCall, ToolFunction, ToolFunctionParameter,
                      ToolResult, Trajectory)

MAX_OUTPUT_CHARS = 20_000

SYSTEM_PROMPT = """You are working on a task whose input is too long to read at once. It is stored in the Python variable `context`
({n_chars} characters); it is NOT in this conversation.

Tools:
- repl(code): run Python. Variables persist between calls. `context` holds the input. Inside the code you may call
  llm_query(prompt) -> str (ask a model about a passage you paste into the prompt) and agent(task, context=None) -> str
  (hand a sub-task and a piece of the input to a sub-agent). print() what you want to see; output is cut at {max_out} characters.
- llm_query(prompt): the same question-answering call as a tool.
- agent(task, context): the same sub-agent call as a tool.
- final_answer(answer): give the answer and stop.

Work in steps: look at the size and shape of `context` (len, first lines, separators), narrow down with string search or
regular expressions, ask llm_query about short passages where meaning matters, and call final_answer once."""


_LIVE_ENDPOINTS: dict[str, Endpoint] = {}


def _tool(name: str, desc: str, props: dict[str, Any], required: tuple[str, ...]) -> Tool:
    return Tool(ToolFunction(name, desc, ToolFunctionParameter(props, required)))


def run_code(code: str, namespace: dict[str, Any], max_chars: int = MAX_OUTPUT_CHARS, timeout_s: float | None = None) -> tuple[str, bool]:
    """Execute ``code`` in ``namespace`` with what it prints captured; the value of a trailing expression is printed as in
    an interactive session. Returns (output, failed).

    Several of these run at once in worker threads (concurrent evaluation samples, sub-agents), so the process-wide
    ``sys.stdout`` is left alone: the namespace gets its own ``print`` that writes to this call's buffer.

    ``timeout_s`` bounds the run with a per-thread trace function that raises once the time is up (signals only reach
    the main thread, and this runs in workers). It ends Python-level loops; a single blocking call into C is not cut."""
    import ast
    import sys
    import time

    buf, failed = io.StringIO(), False
    deadline = time.monotonic() + timeout_s if timeout_s else None

    def _watch(frame, event, arg):
        if time.monotonic() > deadline:
            raise TimeoutError(f"the code ran longer than {timeout_s:g} s and was stopped")
        return _watch

    def _print(*args: Any, **kw: Any) -> None:
        kw.setdefault("file", buf)
        print(*args, **kw)

    namespace["print"] = _print
    old_trace = sys.gettrace()
    try:
        tree = ast.parse(code, "<repl>", "exec")
        if deadline is not None:
            sys.settrace(_watch)
        last = tree.body.pop() if tree.body and isinstance(tree.body[-1], ast.Expr) else None
        exec(compile(tree, "<repl>", "exec"), namespace)  # noqa: S102 - the purpose of a REPL tool
        if last is not None:
            value = eval(compile(ast.Expression(last.value), "<repl>", "eval"), namespace)  # noqa: S307
            if value is not None:
                _print(repr(value))
    except Exception:  # noqa: BLE001 - reported to the model
        failed = True
        buf.write(traceback.format_exc(limit=4))
    finally:
        if deadline is not None:
            sys.settrace(old_trace)
        namespace.pop("print", None)
    out = buf.getvalue()
    if len(out) > max_chars:
        out = out[:max_chars] + f"\n... ({len(out) - max_chars} more characters cut)"
    return out, failed


@dataclass
class RLMEnvironment:
    context: str = ""
    sub_endpoint: Endpoint | None = None
    max_depth: int = 3
    max_agent_turns: int = 15
    depth: int = 0
    namespace: dict[str, Any] = field(default_factory=dict)
    final_answer: str | None = None
    sub_calls: int = 0                          # llm_query + agent calls made so far (a cost signal for evaluations)
    repl_timeout_s: float | None = 120.0        # one repl call may run this long (sub-model calls inside it count)
    exec_count: int = 0
    last_exec_s: float = 0.0

    def get_name(self) -> str:
        return "repl"

    def get_status_info(self) -> dict[str, str] | None:
        info = {"context": f"{len(self.context):,} chars", "depth": f"{self.depth}/{self.max_depth}"}
        if self.exec_count:
            info["repl"] = f"{self.exec_count} runs, last {self.last_exec_s:.2f}s"
        return info

    def get_system_prompt(self) -> str:
        return SYSTEM_PROMPT.format(n_chars=f"{len(self.context):,}", max_out=f"{MAX_OUTPUT_CHARS:,}")

    def get_tools(self) -> list[Tool]:
        s = {"type": "string"}
        return [_tool("repl", "Run Python code; `context`, llm_query() and agent() are available; variables persist", {"code": s}, ("code",)),
                _tool("llm_query", "Ask the sub-model one question (no tools); paste the passage it needs into the prompt", {"prompt": s}, ("prompt",)),
                _tool("agent", "Give a sub-task and a piece of the input to a sub-agent with the same tools", {"task": s, "context": s}, ("task",)),
                _tool("final_answer", "Submit the final answer and stop", {"answer": s}, ("answer",))]

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return False

    # ---- sub-model calls
    async def _llm_query(self, prompt: str, run_config: RunConfig) -> str:
        from ..agents import rollout

        if self.sub_endpoint is None:
            raise RuntimeError("no sub_endpoint configured for llm_query")
        self.sub_calls += 1
        actor = await rollout(Actor(Trajectory((Message("user", prompt),)), self.sub_endpoint), replace(run_config, on_chunk=None, session_store=None))
        return actor.trajectory.messages[-1].text()

    async def _agent(self, task: str, context: str | None, run_config: RunConfig) -> str:
        from ..agents import run_agent

        if self.depth + 1 >= self.max_depth:
            return f"[maximum depth {self.max_depth} reached: use llm_query for this]"
        if self.sub_endpoint is None:
            raise RuntimeError("no sub_endpoint configured for agent")
        self.sub_calls += 1
        child = type(self)(context=self.context if context is None else context, sub_endpoint=self.sub_endpoint, max_depth=self.max_depth,
                           max_agent_turns=self.max_agent_turns, depth=self.depth + 1)
        start = Trajectory((Message("system", child.get_system_prompt()), Message("user", task)))
        state = AgentState(Actor(start, self.sub_endpoint), child, max_turns=self.max_agent_turns)
        final = (await run_agent(state, replace(run_config, on_chunk=None, session_store=None)))[-1]
        self.sub_calls += final.environment.sub_calls
        if final.environment.final_answer is not None:
            return final.environment.final_answer
        last = next((m.text() for m in reversed(final.actor.trajectory.messages) if m.role == "assistant" and m.text()), "")
        return last or "[the sub-agent ended without an answer]"

    def _bind(self, run_config: RunConfig) -> None:
        """Put ``context`` and the two helper functions into the namespace; the helpers hop from the worker thread the
        code runs in back to the event loop, and turn their own failures into text the code can see."""
        loop = asyncio.get_running_loop()

        def from_thread(coro_fn, *a):
            try:
                return asyncio.run_coroutine_threadsafe(coro_fn(*a, run_config), loop).result()
            except Exception as e:  # noqa: BLE001
                return f"[{coro_fn.__name__.lstrip('_')} error: {e}]"

        self.namespace.setdefault("__builtins__", __builtins__)
        self.namespace["context"] = self.namespace.get("context", self.context)
        self.namespace["llm_query"] = lambda prompt: from_thread(self._llm_query, str(prompt))
        self.namespace["agent"] = lambda task, context=None: from_thread(self._agent, str(task), context)

    async def run_repl(self, code: str, run_config: RunConfig) -> tuple[str, bool]:
        import time

        self._bind(run_config)
        t0 = time.monotonic()
        try:
            return await asyncio.to_thread(run_code, code, self.namespace, MAX_OUTPUT_CHARS, self.repl_timeout_s)
        finally:
            self.exec_count += 1
            self.last_exec_s = time.monotonic() - t0

    # ---- tools
    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        a, cid = tool_call.args, tool_call.id
        try:
            if tool_call.name == "repl":
                code = str(a.get("code", ""))
                if not code.strip():
                    return ToolResult(cid, is_error=True, error="no code given")
                out, failed = await self.run_repl(code, run_config)
                return ToolResult(cid, content=out or "(no output)", is_error=failed, error=out if failed else None)
            if tool_call.name == "llm_query":
                if not str(a.get("prompt", "")).strip():
                    return ToolResult(cid, is_error=True, error="no prompt given")
                return ToolResult(cid, content=await self._llm_query(str(a["prompt"]), run_config))
            if tool_call.name == "agent":
                if not str(a.get("task", "")).strip():
                    return ToolResult(cid, is_error=True, error="no task given")
                return ToolResult(cid, content=await self._agent(str(a["task"]), a.get("context") or None, run_config))
            if tool_call.name == "final_answer":
                self.final_answer = str(a.get("answer", ""))
                return ToolResult(cid, content="answer recorded", stop_reason=StopReason.TASK_COMPLETED)
        except Exception as e:  # noqa: BLE001 - a failing sub-call is an answer to the model, not a crash of the run
            return ToolResult(cid, is_error=True, error=f"{tool_call.name} failed: {e}")
        return ToolResult(cid, is_error=True, error=f"unknown tool {tool_call.name!r}")

    # ---- state
    async def serialize(self) -> dict[str, Any]:
        plain = (int, float, str, bool, list, dict, tuple, type(None))
        keep = {k: v for k, v in self.namespace.items() if isinstance(v, plain) and not k.startswith("__") and k != "context"}
        ep = None
        if self.sub_endpoint is not None:
            # what is stored is JSON and carries no credential; within this process the live endpoint (key, in-process
            # engine) is found again through its token
            token = f"ep-{id(self.sub_endpoint):x}"
            _LIVE_ENDPOINTS[token] = self.sub_endpoint
            ep = {**self.sub_endpoint.to_dict(), "_token": token}
        return {"type": "rlm", "context": self.context, "namespace": keep, "final_answer": self.final_answer, "depth": self.depth,
                "max_depth": self.max_depth, "max_agent_turns": self.max_agent_turns, "sub_calls": self.sub_calls, "sub_endpoint": ep,
                "repl_timeout_s": self.repl_timeout_s, "exec_count": self.exec_count, "last_exec_s": self.last_exec_s}

    @classmethod
    async def deserialize(cls, data: dict[str, Any]) -> "RLMEnvironment":
        ep = None
        if data.get("sub_endpoint"):
            d = dict(data["sub_endpoint"])
            ep = _LIVE_ENDPOINTS.get(d.pop("_token", "")) or Endpoint(**{k: v for k, v in d.items() if k in Endpoint.__dataclass_fields__})
        return cls(context=data.get("context", ""), sub_endpoint=ep, max_depth=data.get("max_depth", 3), max_agent_turns=data.get("max_agent_turns", 15),
                   depth=data.get("depth", 0), namespace=dict(data.get("namespace", {})), final_answer=data.get("final_answer"),
                   sub_calls=data.get("sub_calls", 0), repl_timeout_s=data.get("repl_timeout_s", 120.0), exec_count=data.get("exec_count", 0),
                   last_exec_s=data.get("last_exec_s", 0.0))


_BLOCK = re.compile(r"```(?:repl|python|py)\n(.*?)```", re.DOTALL)
_FINAL_VAR = re.compile(r"FINAL_VAR\(\s*([A-Za-z_]\w*)\s*\)")


def _final_call(text: str) -> str | None:
    """Argument of the last ``FINAL(...)`` outside code fences, parentheses balanced, quotes stripped."""
    prose = _BLOCK.sub("", text)
    at = prose.rfind("FINAL(")
    if at < 0:
        return None
    depth, start = 0, at + len("FINAL(")
    for i in range(start, len(prose)):
        c = prose[i]
        if c == "(":
            depth += 1
        elif c == ")":
            if depth == 0:
                inner = prose[start:i].strip()
                return inner[1:-1] if len(inner) >= 2 and inner[0] == inner[-1] and inner[0] in "\"'" else inner
            depth -= 1
    return None


class MessageParsingRLMEnvironment(RLMEnvironment):
    """For models without tool calling: no tools are advertised; the reply's ```repl blocks are run and their output
    comes back as a user message; ``FINAL(text)`` or ``FINAL_VAR(name)`` in the prose ends the episode."""

    def get_tools(self) -> list[Tool]:
        return []

    def get_system_prompt(self) -> str:
        return (f"The input of your task is stored in the Python variable `context` ({len(self.context):,} characters); it is NOT in this "
                "conversation.\n\nTo run Python, write a fenced block:\n```repl\nprint(len(context))\n```\nVariables persist. Inside the code, "
                "llm_query(prompt) asks a model about a passage and agent(task, context=None) hands a sub-task to a sub-agent; both return "
                f"text. You will get the printed output (cut at {MAX_OUTPUT_CHARS:,} characters) as the next message.\n\nWhen you know the "
                "answer, write FINAL(your answer), or FINAL_VAR(name) to give the value of a variable. Do not put FINAL inside a code block.")

    async def on_assistant_message(self, message: Message, state: AgentState) -> AgentState:
        text = message.text()
        outputs = []
        for code in _BLOCK.findall(text):
            out, failed = await self.run_repl(code, RunConfig())
            outputs.append(("[error]\n" if failed else "") + (out or "(no output)"))
        m = _FINAL_VAR.search(_BLOCK.sub("", text))
        answer = None
        if m is not None:
            if m.group(1) in self.namespace:
                answer = str(self.namespace[m.group(1)])
            else:
                outputs.append(f"[FINAL_VAR: no variable named {m.group(1)!r}]")
        else:
            answer = _final_call(text)
        traj = state.actor.trajectory
        if answer is not None:
            self.final_answer = answer
            return replace(state, environment=self, stop=StopReason.TASK_COMPLETED)
        if outputs:
            traj = traj.append(Message("user", "\n\n".join(f"Output of block {i + 1}:\n{o}" for i, o in enumerate(outputs))))
        return replace(state, actor=replace(state.actor, trajectory=traj), environment=self)
