"""Terminal front ends for the interactive agent and the loop that drives them.

The agent loop emits ``StreamEvent`` objects; a front end renders them and supplies user input and
tool confirmations (rollouts/frontends/protocol.py:19-158). Three implementations:

* ``PlainFrontend`` - line-oriented stdout/stdin, no escape codes (pipes, logs);
* ``JsonFrontend`` - one JSON object per event on stdout, input lines from stdin, for driving the agent
  from another process (rollouts/frontends/json_frontend.py, headless_json.py);
* ``AnsiFrontend`` - a terminal UI drawn with ANSI escape codes only (no curses, no external toolkit):
  coloured roles, dimmed reasoning, boxed tool calls with truncated results, fenced-code highlighting,
  a spinner while the model is thinking and a status line with model / turn / token counts
  (the roles of rollouts/frontends/tui_frontend.py and tui/agent_renderer.py).

``InteractiveRunner`` is the front-end-agnostic chat loop (rollouts/frontends/runner.py:117): read a line,
handle slash commands, run the agent until it stops, persist to the session store, repeat.
"""

from __future__ import annotations

import asyncio
import itertools
import json
import shutil
import sys
import time
from dataclasses import asdict, replace
from typing import Any, Callable, Protocol, TextIO, runtime_checkable

from ..agents.agents import run_agent
from ..agents.dtypes import (Actor, AgentState, Endpoint, LLMCallStart, Message, RunConfig, StopReason, StreamDone, StreamError,
                             StreamEvent, TextDelta, ThinkingDelta, ToolCall, ToolCallDelta, ToolCallEnd, ToolCallError, ToolCallStart,
                             ToolExecutionStart, ToolResultReceived, Trajectory)


@runtime_checkable
class Frontend(Protocol):
    async def start(self) -> None: ...
    async def stop(self) -> None: ...
    async def handle_event(self, event: StreamEvent) -> None: ...
    async def get_input(self, prompt: str = "") -> str: ...
    async def confirm_tool(self, tool_call: ToolCall) -> bool: ...
    def show_loader(self, text: str) -> None: ...
    def hide_loader(self) -> None: ...
    def set_status(self, **fields: Any) -> None: ...


async def _readline(stream: TextIO) -> str:
    line = await asyncio.get_running_loop().run_in_executor(None, stream.readline)
    if line == "":
        raise EOFError
    return line.rstrip("\n")


class PlainFrontend:
    """Unadorned text on ``out``; input lines from ``inp``."""

    def __init__(self, out: TextIO | None = None, inp: TextIO | None = None, show_thinking: bool = False,
                 auto_confirm: bool = True):
        self.out, self.inp = out or sys.stdout, inp or sys.stdin
        self.show_thinking, self.auto_confirm = show_thinking, auto_confirm
        self._mid_line = False
        self.status: dict[str, Any] = {}
        self.environment: Any = None          # set by the runner: its get_tool_formatter(name) renders calls / results
        self._calls: dict[str, tuple[str, dict[str, Any]]] = {}

    def _formatted(self, event: StreamEvent, expanded: bool = False) -> str | None:
        """The environment's own rendering of a tool call (``ToolCallEnd``) or of its result (``ToolResultReceived``),
        None when the environment offers no formatter for that tool."""
        from ..agents.dtypes import ToolResult

        if isinstance(event, ToolCallEnd):
            self._calls[event.tool_call_id] = (event.name, event.args)
            name, args, result = event.name, event.args, None
        else:
            if event.tool_call_id not in self._calls:
                return None
            name, args = self._calls.pop(event.tool_call_id)
            result = ToolResult(event.tool_call_id, event.content, event.is_error, event.content if event.is_error else None,
                                metadata=dict(event.details))
        get = getattr(self.environment, "get_tool_formatter", None)
        fmt = get(name) if get is not None else None
        return fmt(name, args, result, expanded) if fmt is not None else None

    def _w(self, s: str) -> None:
        self.out.write(s)
        self.out.flush()
        if s:
            self._mid_line = not s.endswith("\n")

    def _fresh_line(self) -> None:
        if self._mid_line:
            self._w("\n")

    async def start(self) -> None: ...

    async def stop(self) -> None:
        self._fresh_line()

    async def handle_event(self, event: StreamEvent) -> None:
        if isinstance(event, TextDelta):
            self._w(event.delta)
        elif isinstance(event, ThinkingDelta):
            if self.show_thinking:
                self._w(event.delta)
        elif isinstance(event, ToolCallEnd):
            self._fresh_line()
            text = self._formatted(event)
            self._w(f"[tool] {text}\n" if text is not None else f"[tool] {event.name}({json.dumps(event.args, ensure_ascii=False)})\n")
        elif isinstance(event, ToolResultReceived):
            self._fresh_line()
            tag = "error" if event.is_error else "result"
            text = self._formatted(event)
            self._w(f"[{tag}] {text}\n" if text is not None else f"[{tag}] {_truncate(event.content, 2000)}\n")
        elif isinstance(event, StreamError):
            self._fresh_line()
            self._w(f"[error] {event.error}\n")
        elif isinstance(event, StreamDone):
            self._fresh_line()

    async def get_input(self, prompt: str = "") -> str:
        self._fresh_line()
        self._w(prompt)
        return await _readline(self.inp)

    async def confirm_tool(self, tool_call: ToolCall) -> bool:
        if self.auto_confirm:
            return True
        ans = await self.get_input(f"run {tool_call.name}({json.dumps(tool_call.args, ensure_ascii=False)})? [y/N] ")
        return ans.strip().lower() in ("y", "yes")

    def show_loader(self, text: str) -> None: ...

    def hide_loader(self) -> None: ...

    def set_status(self, **fields: Any) -> None:
        self.status.update(fields)


class JsonFrontend(PlainFrontend):
    """Newline-delimited JSON: every event is ``{"type": ..., ...}``; requests for input are events too
    (``input_request`` / ``confirm_request``) and are answered by one line on ``inp``."""

    def _emit(self, obj: dict[str, Any]) -> None:
        self.out.write(json.dumps(obj, ensure_ascii=False, default=str) + "\n")
        self.out.flush()

    async def start(self) -> None:
        self._emit({"type": "start", "timestamp": time.time()})

    async def stop(self) -> None:
        self._emit({"type": "stop", "timestamp": time.time(), **{k: v for k, v in self.status.items()}})

    async def handle_event(self, event: StreamEvent) -> None:
        self._emit(asdict(event))

    async def get_input(self, prompt: str = "") -> str:
        self._emit({"type": "input_request", "prompt": prompt})
        line = await _readline(self.inp)
        try:                      # either a bare line or {"text": "..."}
            obj = json.loads(line)
            if isinstance(obj, dict) and "text" in obj:
                return str(obj["text"])
        except ValueError:
            pass
        return line

    async def confirm_tool(self, tool_call: ToolCall) -> bool:
        if self.auto_confirm:
            return True
        self._emit({"type": "confirm_request", "tool": tool_call.name, "args": tool_call.args, "id": tool_call.id})
        return (await _readline(self.inp)).strip().lower() in ("y", "yes", "true", '{"ok": true}')

    def show_loader(self, text: str) -> None:
        self._emit({"type": "loader", "text": text})


# ------------------------------------------------------------------------------------------ ANSI rendering
class Theme:
    RESET, BOLD, DIM, ITALIC = "\x1b[0m", "\x1b[1m", "\x1b[2m", "\x1b[3m"
    USER, ASSISTANT, TOOL, ERROR, CODE, STATUS = "\x1b[36m", "\x1b[0m", "\x1b[33m", "\x1b[31m", "\x1b[32m", "\x1b[7m"
    CLEAR_LINE, HIDE_CURSOR, SHOW_CURSOR = "\r\x1b[2K", "\x1b[?25l", "\x1b[?25h"


_THEMES = {
    "dark": dict(USER="\x1b[36m", ASSISTANT="\x1b[0m", TOOL="\x1b[33m", ERROR="\x1b[31m", CODE="\x1b[32m", STATUS="\x1b[7m", DIM="\x1b[2m"),
    # on a light background dim yellow and green wash out: darker blue / magenta, and no dimming of secondary text
    "light": dict(USER="\x1b[34m", ASSISTANT="\x1b[0m", TOOL="\x1b[35m", ERROR="\x1b[31m", CODE="\x1b[34m", STATUS="\x1b[7m", DIM="\x1b[90m"),
    "none": dict(USER="", ASSISTANT="", TOOL="", ERROR="", CODE="", STATUS="", DIM="", RESET="", BOLD="", ITALIC=""),
}


def apply_theme(name: str) -> None:
    """Switch the colours of the ANSI front end (``dark`` | ``light`` | ``none``). Cursor and line control stay as they are."""
    if name not in _THEMES:
        raise ValueError(f"unknown theme {name!r}: {sorted(_THEMES)}")
    for k, v in {"RESET": "\x1b[0m", "BOLD": "\x1b[1m", "ITALIC": "\x1b[3m", **_THEMES[name]}.items():
        setattr(Theme, k, v)


def _truncate(text: str, limit: int) -> str:
    return text if len(text) <= limit else text[:limit] + f"... (+{len(text) - limit} chars)"


def truncate_lines(text: str, max_lines: int, width: int) -> list[str]:
    """First ``max_lines`` display lines of ``text`` (long lines cut to ``width``) and a count of what was dropped."""
    lines = text.splitlines() or [""]
    shown = [ln if len(ln) <= width else ln[:max(width - 1, 1)] + "…" for ln in lines[:max_lines]]
    if len(lines) > max_lines:
        shown.append(f"… {len(lines) - max_lines} more lines")
    return shown


def colour_diff_line(line: str) -> str:
    """One line of a unified diff (possibly indented by a formatter): additions green, removals red, hunk headers dim."""
    s = line.lstrip()
    if s.startswith(("+++", "---")):
        return f"{Theme.DIM}{line}{Theme.RESET}"
    if s.startswith("+"):
        return f"{Theme.CODE}{line}{Theme.RESET}"
    if s.startswith("-"):
        return f"{Theme.ERROR}{line}{Theme.RESET}"
    if s.startswith("@@"):
        return f"{Theme.DIM}{line}{Theme.RESET}"
    return line


def box(title: str, body_lines: list[str], width: int, color: str = "") -> str:
    """A one-line-border box around ``body_lines``; ``width`` is the total width in columns."""
    inner = max(width - 4, 8)
    top = f"┌─ {title[:inner - 2]} " + "─" * max(inner - len(title[:inner - 2]) - 1, 0) + "┐"
    rows = [f"│ {ln[:inner].ljust(inner)} │" for ln in body_lines]
    bottom = "└" + "─" * (inner + 2) + "┘"
    reset = Theme.RESET if color else ""
    return "\n".join(f"{color}{r}{reset}" for r in [top, *rows, bottom])


class FenceHighlighter:
    """Streaming colouriser for Markdown code fences: text arrives in arbitrary pieces, lines inside a
    ``` fence are coloured, everything else passes through. Partial lines are emitted at once (the colour
    state only changes at line starts), so streaming stays character-granular."""

    def __init__(self, code_color: str = Theme.CODE, reset: str = Theme.RESET):
        self.code_color, self.reset = code_color, reset
        self.in_code = False
        self._line = ""          # the current (unfinished) line as seen so far

    def feed(self, piece: str) -> str:
        out = []
        for ch in piece:
            at_start = self._line == ""
            self._line += ch
            if ch == "\n":
                if self._line.lstrip().startswith("```"):
                    self.in_code = not self.in_code
                    out.append(self.reset if not self.in_code else "")
                self._line = ""
                out.append(ch)
                continue
            if at_start and self.in_code:
                out.append(self.code_color)
            out.append(ch)
        return "".join(out)


class AnsiFrontend(PlainFrontend):
    """Escape-code terminal UI. All drawing goes through ``_w`` so tests can capture it from ``out``."""

    SPIN = "⠋⠙⠹⠸⠼⠴⠦⠧⠇⠏"

    def __init__(self, out: TextIO | None = None, inp: TextIO | None = None, show_thinking: bool = True,
                 auto_confirm: bool = False, width: int | None = None, max_result_lines: int = 12):
        super().__init__(out, inp, show_thinking, auto_confirm)
        self.width = width or shutil.get_terminal_size((100, 24)).columns
        self.max_result_lines = max_result_lines
        self._fence = FenceHighlighter()
        self._tool_names: dict[str, str] = {}
        self._editor = None                  # the prompt's line editor, created on first use at a terminal
        self.completer = None                # set by the runner: slash commands and paths
        self._loader_task: asyncio.Task | None = None
        self._loader_text = ""
        self._mode = ""           # "", "text", "thinking"
        self._t_stream = 0.0
        self._chars = 0

    async def start(self) -> None:
        self._w(f"{Theme.BOLD}research_b200 chat{Theme.RESET}  {Theme.DIM}/help for commands, ctrl-d to quit{Theme.RESET}\n")

    async def stop(self) -> None:
        self.hide_loader()
        self._fresh_line()
        self._w(Theme.SHOW_CURSOR + Theme.RESET)

    # ---- loader / status
    def show_loader(self, text: str) -> None:
        self.hide_loader()
        self._loader_text = text
        try:
            loop = asyncio.get_running_loop()
        except RuntimeError:
            return
        self._loader_task = loop.create_task(self._spin())

    async def _spin(self) -> None:
        t0 = time.monotonic()
        try:
            for frame in itertools.cycle(self.SPIN):
                self.out.write(f"{Theme.CLEAR_LINE}{Theme.DIM}{frame} {self._loader_text} {time.monotonic() - t0:4.1f}s{Theme.RESET}")
                self.out.flush()
                await asyncio.sleep(0.08)
        except asyncio.CancelledError:
            self.out.write(Theme.CLEAR_LINE)
            self.out.flush()

    def hide_loader(self) -> None:
        if self._loader_task is not None:
            self._loader_task.cancel()
            self._loader_task = None
            self.out.write(Theme.CLEAR_LINE)
            self.out.flush()

    def status_line(self) -> str:
        s = self.status
        parts = [str(s.get("model", "")), f"turn {s.get('turn', 0)}", f"{s.get('input_tokens', 0)}→{s.get('output_tokens', 0)} tok"]
        if s.get("cost"):
            parts.append(f"${s['cost']:.4f}")
        if s.get("session_id"):
            parts.append(str(s["session_id"])[:12])
        text = "  ".join(p for p in parts if p)
        return f"{Theme.STATUS} {text[:self.width - 2].ljust(self.width - 2)} {Theme.RESET}"

    # ---- events
    def _enter(self, mode: str) -> None:
        if mode == self._mode:
            return
        self.hide_loader()
        if self._mode == "thinking":
            self._w(Theme.RESET)
        self._fresh_line()
        if mode == "thinking":
            self._w(f"{Theme.DIM}{Theme.ITALIC}")
        elif mode == "text":
            self._t_stream, self._chars = time.monotonic(), 0
        self._mode = mode

    async def handle_event(self, event: StreamEvent) -> None:
        if isinstance(event, TextDelta):
            self._enter("text")
            self._chars += len(event.delta)
            self._w(self._fence.feed(event.delta))
        elif isinstance(event, ThinkingDelta):
            if self.show_thinking:
                self._enter("thinking")
                self._w(event.delta)
        elif isinstance(event, LLMCallStart):
            if self._mode == "":
                self.show_loader("waiting for the model")
        elif isinstance(event, ToolCallStart):
            self._enter("")
            self._tool_names[event.tool_call_id] = event.name
            self.show_loader(f"{event.name}: receiving arguments")
        elif isinstance(event, ToolCallDelta):
            if event.partial_args:                  # the arguments as far as they have arrived, in the loader line
                name = self._tool_names.get(event.tool_call_id, "tool")
                shown = ", ".join(f"{k}={str(v)[:40]!r}" for k, v in list(event.partial_args.items())[:3])
                self._loader_text = f"{name}({shown[:self.width - len(name) - 12]}…"
        elif isinstance(event, ToolCallError):
            self._enter("")
            self._w(f"{Theme.ERROR}{event.tool_name}: {event.error}{Theme.RESET}\n")
        elif isinstance(event, ToolExecutionStart):
            self.show_loader(f"running {event.tool_name}")
        elif isinstance(event, ToolCallEnd):
            self._enter("")
            self._formatted(event)                  # remembers the call for its result
            args = json.dumps(event.args, ensure_ascii=False, indent=2)
            self._w(box(f"tool: {event.name}", truncate_lines(args, 10, self.width - 4), self.width, Theme.TOOL) + "\n")
            self.show_loader(f"running {event.name}")
        elif isinstance(event, ToolResultReceived):
            self._enter("")
            color = Theme.ERROR if event.is_error else Theme.DIM
            title = "error" if event.is_error else "result"
            body = self._formatted(event) or event.content
            lines = truncate_lines(body, self.max_result_lines, self.width - 4)
            if event.details.get("diff") and not event.is_error:
                self._w("\n".join(colour_diff_line(ln) for ln in lines) + "\n")      # a diff reads better unboxed: removed red, added green
            else:
                self._w(box(title, lines, self.width, color) + "\n")
        elif isinstance(event, StreamError):
            self._enter("")
            self._w(f"{Theme.ERROR}error: {event.error}{Theme.RESET}\n")
        elif isinstance(event, StreamDone):
            self._enter("")
            self._w(Theme.RESET)

    async def get_input(self, prompt: str = "") -> str:
        self._enter("")
        self._w(self.status_line() + "\n")
        if self._is_tty():
            # a real terminal: the line editor (history, word motions, multi-line, completion) in raw mode
            from .widgets import LineEditor, read_line_raw

            if self._editor is None:
                self._editor = LineEditor(completer=self.completer)
            self._editor.completer = self.completer
            return await asyncio.to_thread(read_line_raw, self._editor, f"{Theme.USER}{Theme.BOLD}{prompt or '> '}{Theme.RESET}",
                                           self.inp.fileno(), self._w, self.width)
        self._w(f"{Theme.USER}{Theme.BOLD}{prompt or '> '}{Theme.RESET}")
        return await _readline(self.inp)

    def _is_tty(self) -> bool:
        try:
            return bool(self.inp.isatty() and self.out.isatty()) and self.inp.fileno() >= 0
        except (AttributeError, ValueError, OSError):
            return False

    async def confirm_tool(self, tool_call: ToolCall) -> bool:
        if self.auto_confirm:
            return True
        self.hide_loader()
        self._fresh_line()
        self._w(f"{Theme.TOOL}allow {tool_call.name}? [y/N/a(lways)] {Theme.RESET}")
        ans = (await _readline(self.inp)).strip().lower()
        if ans in ("a", "always"):
            self.auto_confirm = True
            return True
        return ans in ("y", "yes")


# ------------------------------------------------------------------------------------------ the chat loop
HELP = """/help               this text
/quit               leave (ctrl-d works too)
/clear              start a new conversation (keeps the system prompt)
/model NAME         switch the model of the endpoint
/temperature X      sampling temperature
/thinking [on|off|N] extended thinking (N = token budget) and whether it is shown
/status             session, turns, token counts
/save PATH          write the conversation as JSON lines
/retry              drop the last assistant turn and ask again
/slice SPEC         continue on a sliced copy (0:4, summarize:4:20, 20:)
/env [NAME]         show or switch the environment (the agent's tools)
/session [ID]       recent sessions, or continue in another one
/branch [N]         fork the conversation (after N messages) into a new session
/edit [N] TEXT      reword a user message (default: the last) and continue from there in a new session
/tree               the tree of sessions this conversation belongs to
/commands           every command, including those from .research_b200/commands/*.md"""


class InteractiveRunner:
    """Chat loop over any ``Frontend``: prompts, slash commands, tool confirmation, session persistence."""

    def __init__(self, endpoint: Endpoint, frontend: Frontend, environment: Any = None, system_prompt: str | None = None,
                 session_store: Any = None, session_id: str | None = None, max_turns: int = 20,
                 initial_prompt: str | None = None, single_turn: bool = False, trajectory: Trajectory | None = None,
                 session_tags: dict[str, Any] | None = None, cwd: str = ".", file_commands: list | None = None):
        from .slash_commands import load_file_commands

        self.endpoint, self.frontend, self.environment = endpoint, frontend, environment
        self.session_tags = session_tags
        self.cwd = cwd
        self.file_commands = load_file_commands(cwd) if file_commands is None else file_commands
        self.current_exchange: "asyncio.Future | None" = None
        if hasattr(frontend, "environment"):
            frontend.environment = environment
        if hasattr(frontend, "completer"):
            from .slash_commands import BUILTIN_COMMANDS
            from .widgets import make_completer

            every = BUILTIN_COMMANDS + self.file_commands
            frontend.completer = make_completer([c.name for c in every], cwd, {c.name: c.arg_hint for c in every if c.arg_hint})
        self.system_prompt = system_prompt
        self.store, self.session_id = session_store, session_id
        self.max_turns, self.initial_prompt, self.single_turn = max_turns, initial_prompt, single_turn
        base = trajectory or Trajectory(tuple([Message("system", system_prompt)] if system_prompt else []))
        self.state = AgentState(actor=Actor(base, endpoint), environment=environment, max_turns=max_turns, session_id=session_id)
        self.turns = 0
        self.commands: dict[str, Callable[[str], Any]] = {
            "help": self._cmd_help, "clear": self._cmd_clear, "model": self._cmd_model, "temperature": self._cmd_temperature,
            "thinking": self._cmd_thinking, "status": self._cmd_status, "save": self._cmd_save, "retry": self._cmd_retry,
            "slice": self._cmd_slice, "env": self._cmd_env, "commands": self._cmd_commands, "session": self._cmd_session,
            "branch": self._cmd_branch, "edit": self._cmd_edit, "tree": self._cmd_tree}

    # ---- slash commands: return text to print; "retry" returns a prompt to resend
    def _cmd_help(self, arg: str) -> str:
        return HELP

    def _cmd_clear(self, arg: str) -> str:
        msgs = tuple(m for m in self.state.actor.trajectory.messages if m.role == "system")
        self.state = replace(self.state, actor=Actor(Trajectory(msgs), self.endpoint), turn_idx=0, stop=None, session_id=None,
                             pending_tool_calls=())
        return "conversation cleared"

    def _cmd_model(self, arg: str) -> str:
        if not arg:
            return f"model: {self.endpoint.model}"
        self.set_endpoint(replace(self.endpoint, model=arg))
        return f"model set to {arg}"

    def _cmd_temperature(self, arg: str) -> str:
        try:
            t = float(arg)
        except ValueError:
            return "usage: /temperature 0.7"
        self.set_endpoint(replace(self.endpoint, temperature=t))
        return f"temperature set to {t}"

    def _log_config_change(self, what: str, before: Any, after: Any) -> None:
        # every exchange is its own agent run with a fixed endpoint and environment; a change between two runs is
        # recorded in the session so that the conversation can be replayed with the configuration each turn had
        record = getattr(self.store, "record_config_change", None)
        if record is not None and self.state.session_id and before != after:
            record(self.state.session_id, what, before, after)

    def set_endpoint(self, endpoint: Endpoint) -> None:
        self._log_config_change("endpoint", self.endpoint.to_dict(), endpoint.to_dict())
        self.endpoint = endpoint
        self.state = replace(self.state, actor=replace(self.state.actor, endpoint=endpoint))

    def set_environment(self, environment: Any) -> None:
        name = lambda e: {"name": e.get_name() if hasattr(e, "get_name") else type(e).__name__} if e is not None else None  # noqa: E731
        self._log_config_change("environment", name(self.environment), name(environment))
        self.environment = environment
        self.state = replace(self.state, environment=environment)
        if hasattr(self.frontend, "environment"):
            self.frontend.environment = environment

    def _cmd_thinking(self, arg: str):
        from .slash_commands import handle_thinking

        return handle_thinking(self, arg)

    def _cmd_slice(self, arg: str):
        from .slash_commands import handle_slice

        return handle_slice(self, arg)

    def _cmd_env(self, arg: str):
        from .slash_commands import handle_env

        return handle_env(self, arg)

    def _cmd_session(self, arg: str):
        from .slash_commands import handle_session

        return handle_session(self, arg)

    def _cmd_branch(self, arg: str):
        from .slash_commands import handle_branch

        return handle_branch(self, arg)

    def _cmd_edit(self, arg: str):
        from .slash_commands import handle_edit

        return handle_edit(self, arg)

    def _cmd_tree(self, arg: str):
        from .slash_commands import handle_tree

        return handle_tree(self, arg)

    def _cmd_commands(self, arg: str) -> str:
        from .slash_commands import BUILTIN_COMMANDS

        rows = [(f"/{c.name}" + (f" {c.arg_hint}" if c.arg_hint else ""), c.description, c.source) for c in BUILTIN_COMMANDS + self.file_commands]
        w = max(len(r[0]) for r in rows)
        return "\n".join(f"{r[0]:<{w}}  {r[1]}" + (f"  {r[2]}" if r[2] != "(builtin)" else "") for r in rows)

    def _cmd_status(self, arg: str) -> str:
        u = self.state.usage
        return (f"session {self.state.session_id or '-'}  turns {self.turns}  messages {len(self.state.actor.trajectory.messages)}  "
                f"tokens in/out {u.input_tokens}/{u.output_tokens}")

    def _cmd_save(self, arg: str) -> str:
        if not arg:
            return "usage: /save conversation.jsonl"
        with open(arg, "w") as f:
            for m in self.state.actor.trajectory.messages:
                f.write(json.dumps(m.to_dict(), ensure_ascii=False) + "\n")
        return f"saved {len(self.state.actor.trajectory.messages)} messages to {arg}"

    def _cmd_retry(self, arg: str):
        msgs = list(self.state.actor.trajectory.messages)
        while msgs and msgs[-1].role != "user":
            msgs.pop()
        if not msgs:
            return "nothing to retry"
        last_user = msgs.pop()
        self.state = replace(self.state, actor=Actor(Trajectory(tuple(msgs)), self.endpoint), stop=None, pending_tool_calls=())
        return ("retry", last_user.text())

    # ---- loop
    def _run_config(self) -> RunConfig:
        fe = self.frontend

        async def on_chunk(ev: StreamEvent) -> None:
            await fe.handle_event(ev)

        async def confirm(call: ToolCall, state: AgentState, rc: RunConfig) -> bool:
            return await fe.confirm_tool(call)

        async def on_input(prompt: str) -> str:
            return await fe.get_input(prompt)

        return RunConfig(on_chunk=on_chunk, confirm_tool=confirm, on_input=on_input, session_store=self.store,
                         session_tags=self.session_tags)

    @staticmethod
    def _interrupt_with_sigint(task: "asyncio.Future") -> Callable[[], None]:
        """While ``task`` runs, SIGINT cancels it instead of raising KeyboardInterrupt in the event loop. Returns the function
        that puts the previous behaviour back. Where signal handlers cannot be installed (not the main thread, not Unix)
        nothing changes."""
        import signal

        loop = asyncio.get_running_loop()
        try:
            loop.add_signal_handler(signal.SIGINT, task.cancel)
        except (NotImplementedError, RuntimeError, ValueError):
            return lambda: None

        def restore() -> None:
            try:
                loop.remove_signal_handler(signal.SIGINT)
            except (NotImplementedError, RuntimeError, ValueError):
                pass

        return restore

    def _publish_status(self) -> None:
        u = self.state.usage
        self.frontend.set_status(model=self.endpoint.model or self.endpoint.provider, turn=self.turns, input_tokens=u.input_tokens,
                                 output_tokens=u.output_tokens, cost=u.cost.input + u.cost.output + u.cost.cache_read + u.cost.cache_write,
                                 session_id=self.state.session_id)

    async def _one_exchange(self, text: str) -> None:
        traj = self.state.actor.trajectory.append(Message("user", text))
        self.state = replace(self.state, actor=replace(self.state.actor, trajectory=traj, endpoint=self.endpoint), stop=None, turn_idx=0)
        if self.store is not None and self.state.session_id:
            await self.store.append_message(self.state.session_id, traj.messages[-1])
        self.frontend.show_loader("thinking")
        # the exchange runs as a task of its own so that ctrl-c (SIGINT) ends THIS exchange and the chat goes on: the
        # conversation continues from the user's message, whatever the interrupted turn had produced is dropped
        task = asyncio.ensure_future(run_agent(self.state, self._run_config()))
        self.current_exchange = task
        restore = self._interrupt_with_sigint(task)
        try:
            states = await task
            self.state = states[-1]
        except asyncio.CancelledError:
            if not task.cancelled():
                raise                                # the runner itself is being cancelled
            await self.frontend.handle_event(StreamError(error="interrupted"))
            self.state = replace(self.state, stop=StopReason.ABORTED, pending_tool_calls=())
        except Exception as e:  # noqa: BLE001 - a provider failure ends the exchange, not the chat
            await self.frontend.handle_event(StreamError(error=f"{type(e).__name__}: {e}"))
            self.state = replace(self.state, stop=StopReason.ERROR)
        finally:
            restore()
            self.current_exchange = None
            self.frontend.hide_loader()
        self.turns += 1
        self._publish_status()

    async def run(self) -> AgentState:
        fe = self.frontend
        await fe.start()
        self._publish_status()
        pending = self.initial_prompt
        try:
            while True:
                if pending is None:
                    try:
                        pending = await fe.get_input("> ")
                    except (EOFError, KeyboardInterrupt):
                        break
                text, pending = pending.strip(), None
                if not text:
                    continue
                if text.startswith("/"):
                    name, _, arg = text[1:].partition(" ")
                    if name in ("quit", "exit", "q"):
                        break
                    from .slash_commands import SlashCommandResult, expand_file_command, find_similar_command

                    fn = self.commands.get(name)
                    if fn is None:
                        expanded = expand_file_command(text, self.file_commands)
                        if expanded is not None:          # a command from a file is a prompt: it goes to the model
                            await self._one_exchange(expanded)
                            if self.single_turn:
                                break
                            continue
                        near = find_similar_command(name, sorted(self.commands) + [c.name for c in self.file_commands])
                        res = f"unknown command /{name}" + (f" (did you mean /{near}?)" if near else "") + " (try /commands)"
                    else:
                        res = fn(arg.strip())
                        if asyncio.iscoroutine(res):
                            res = await res
                    if isinstance(res, SlashCommandResult):
                        if res.persist and self.store is not None and self.state.session_id:
                            session, _ = await self.store.get(self.state.session_id)
                            await self.store.update(self.state.session_id, tags={**session.tags, **res.persist})
                        if res.expanded_text:
                            if res.message:
                                await fe.handle_event(TextDelta(delta=res.message + "\n"))
                                await fe.handle_event(StreamDone())
                            pending = res.expanded_text
                            continue
                        res = res.message or ""
                    if isinstance(res, tuple) and res[0] == "retry":
                        pending = res[1]
                    else:
                        await fe.handle_event(TextDelta(delta=str(res) + "\n"))
                        await fe.handle_event(StreamDone())
                    continue
                await self._one_exchange(text)
                if self.single_turn:
                    break
        finally:
            await fe.stop()
        return self.state


class HeadlessJsonFrontend(PlainFrontend):
    """Turn-level NDJSON in both directions, for scripts and external user interfaces (rollouts/frontends/headless_json.py:42-413).
    Unlike ``JsonFrontend`` (every stream event as it happens) this one speaks in whole turns::

        -> {"type": "system", "subtype": "init", "session_id": "...", "tools": [...], "environment": "coding"}
        <- {"type": "user", "text": "fix the failing test"}                 (or a bare line of text; "/quit" ends)
        -> {"type": "assistant", "message": {"content": [{"type": "text", ...}, {"type": "tool_use", ...}]}}
        -> {"type": "user", "message": {"content": [{"type": "tool_result", "tool_use_id": ..., "content": ..., "is_error": false}]}}
        -> {"type": "input_request"}                                         (the agent waits for the next line)
        -> {"type": "result", "subtype": "success", "num_turns": 2, "duration_ms": 1234, ...status}

    Slash commands typed as user text are answered by the runner and appear as ``assistant`` text like any other output."""

    def __init__(self, out: TextIO | None = None, inp: TextIO | None = None, include_thinking: bool = False, auto_confirm: bool = True, **_):
        super().__init__(out, inp, include_thinking, auto_confirm)
        self.include_thinking = include_thinking
        self._text: list[str] = []
        self._thinking: list[str] = []
        self._calls: list[dict[str, Any]] = []
        self.num_turns = 0
        self._t0 = time.time()

    def _emit(self, obj: dict[str, Any]) -> None:
        self.out.write(json.dumps(obj, ensure_ascii=False, default=str) + "\n")
        self.out.flush()

    def _flush_turn(self) -> None:
        content: list[dict[str, Any]] = []
        thinking = "".join(self._thinking).strip()
        if thinking and self.include_thinking:
            content.append({"type": "thinking", "thinking": thinking})
        text = "".join(self._text).strip()
        if text:
            content.append({"type": "text", "text": text})
        content += self._calls
        if content:
            self._emit({"type": "assistant", "message": {"content": content}})
            self.num_turns += 1
        self._text, self._thinking, self._calls = [], [], []

    async def start(self) -> None:
        env = self.environment
        tools = [t.function.name for t in env.get_tools()] if env is not None and hasattr(env, "get_tools") else []
        name = env.get_name() if env is not None and hasattr(env, "get_name") else ("none" if env is None else type(env).__name__)
        self._t0 = time.time()
        self._emit({"type": "system", "subtype": "init", "session_id": self.status.get("session_id") or "", "tools": tools, "environment": name})

    async def stop(self) -> None:
        self._flush_turn()
        self._emit({"type": "result", "subtype": "success", "num_turns": self.num_turns, "duration_ms": int((time.time() - self._t0) * 1000),
                    **{k: v for k, v in self.status.items()}})

    async def handle_event(self, event: StreamEvent) -> None:
        if isinstance(event, TextDelta):
            self._text.append(event.delta)
        elif isinstance(event, ThinkingDelta):
            self._thinking.append(event.delta)
        elif isinstance(event, ToolCallEnd):
            self._calls.append({"type": "tool_use", "id": event.tool_call_id, "name": event.name, "input": dict(event.args)})
        elif isinstance(event, ToolResultReceived):
            self._flush_turn()
            self._emit({"type": "user", "message": {"content": [{"type": "tool_result", "tool_use_id": event.tool_call_id, "content": event.content,
                                                                "is_error": event.is_error}]}})
        elif isinstance(event, StreamDone):
            self._flush_turn()
        elif isinstance(event, StreamError):
            self._flush_turn()
            self._emit({"type": "error", "error": str(event.error)})

    async def get_input(self, prompt: str = "") -> str:
        self._flush_turn()
        self._emit({"type": "input_request"})
        line = await _readline(self.inp)
        try:
            obj = json.loads(line)
            if isinstance(obj, dict):
                return str(obj.get("text", obj.get("content", "")))
        except ValueError:
            pass
        return line

    async def confirm_tool(self, tool_call: ToolCall) -> bool:
        if self.auto_confirm:
            return True
        self._flush_turn()
        self._emit({"type": "confirm_request", "tool": tool_call.name, "input": tool_call.args, "id": tool_call.id})
        answer = (await _readline(self.inp)).strip()
        try:
            obj = json.loads(answer)
            return bool(obj.get("allow", obj.get("ok", False))) if isinstance(obj, dict) else bool(obj)
        except ValueError:
            return answer.lower() in ("y", "yes", "true")


def make_frontend(kind: str, **kw: Any) -> Frontend:
    """``plain`` | ``json`` (every event) | ``headless`` (whole turns, two-way) | ``ansi`` (``auto`` = ansi on a terminal, plain otherwise)."""
    if kind == "auto":
        kind = "ansi" if sys.stdout.isatty() else "plain"
    return {"plain": PlainFrontend, "none": PlainFrontend, "json": JsonFrontend, "headless": HeadlessJsonFrontend, "ansi": AnsiFrontend,
            "tui": AnsiFrontend}[kind](**kw)
