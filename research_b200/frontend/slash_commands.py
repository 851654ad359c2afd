"""Slash commands of the interactive chat beyond the basic ones (rollouts/frontends/tui/slash_commands.py:28-830):

* ``/thinking [on|off|N]``: extended thinking of the model (a token budget), and whether it is shown;
* ``/slice SPEC``: continue on a sliced copy of the conversation (``0:4, summarize:4:20, 20:``) in a child session;
* ``/env [NAME]``: show or switch the environment (the tools the agent has) without leaving the conversation;
* ``/commands``: list everything, built in or from files;
* commands from files: every ``*.md`` under ``~/.research_b200/commands/`` (user) and ``./.research_b200/commands/``
  (project; wins on a name clash) is a command named after the file (``review.md`` -> ``/review``, ``git/pr.md`` ->
  ``/git:pr``). Optional front matter gives ``description`` and ``argument-hint``; the body is a prompt in which ``$1``,
  ``$2`` ... and ``$@`` / ``$ARGUMENTS`` stand for the arguments. Such a command is not executed here: its expanded text
  is sent to the model as the user's message.
"""

from __future__ import annotations

import difflib
import re
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Any

DEFAULT_THINKING_BUDGET = 10_000


@dataclass(frozen=True)
class SlashCommand:
    name: str
    description: str
    arg_hint: str | None = None
    content: str | None = None           # file commands: the prompt template
    source: str = "(builtin)"            # (builtin) | (user) | (project)


@dataclass
class SlashCommandResult:
    handled: bool = True                 # False: not a command after all, send the text to the model as it is
    message: str | None = None           # shown to the user
    expanded_text: str | None = None     # send this to the model instead
    persist: dict[str, Any] | None = None  # session tags to store


BUILTIN_COMMANDS = [SlashCommand("help", "what can be typed here"), SlashCommand("clear", "forget the conversation (keeps the system prompt)"),
                    SlashCommand("model", "show or switch the model", "[provider/model]"), SlashCommand("temperature", "set the sampling temperature", "<float>"),
                    SlashCommand("thinking", "extended thinking", "[on|off|budget]"), SlashCommand("status", "session, turns, tokens"),
                    SlashCommand("save", "write the conversation to a JSONL file", "<file>"), SlashCommand("retry", "resend the last user message"),
                    SlashCommand("slice", "continue on a sliced copy of the conversation", "[0:5, summarize:5:20, 20:]"),
                    SlashCommand("env", "show or switch the environment", "[name]"), SlashCommand("commands", "list all commands"),
                    SlashCommand("session", "list recent sessions, or continue in another one", "[id]"),
                    SlashCommand("branch", "fork the conversation here (or after N messages) into a new session", "[n]"),
                    SlashCommand("edit", "reword a user message (default: the last one) and continue from there in a new session", "[n] <new text>"),
                    SlashCommand("tree", "the tree of sessions this conversation belongs to"),
                    SlashCommand("quit", "leave")]


# ------------------------------------------------------------------------------------------- commands from files
def parse_frontmatter(text: str) -> tuple[dict[str, str], str]:
    """``---`` / ``key: value`` lines / ``---`` at the top of a file -> (dict, rest). No front matter: ({}, text)."""
    if not text.startswith("---"):
        return {}, text
    end = text.find("\n---", 3)
    if end < 0:
        return {}, text
    meta = {}
    for line in text[3:end].splitlines():
        key, sep, value = line.partition(":")
        if sep and key.strip():
            meta[key.strip()] = value.strip().strip("\"'")
    return meta, text[end + 4:].lstrip("\n").rstrip() + "\n" if text[end + 4:].strip() else ""


def parse_command_args(text: str) -> list[str]:
    """Whitespace-separated arguments; single or double quotes group words (the quotes are dropped)."""
    args, cur, quote, open_arg = [], "", None, False
    for ch in text:
        if quote:
            if ch == quote:
                quote = None
            else:
                cur += ch
        elif ch in "\"'":
            quote, open_arg = ch, True
        elif ch.isspace():
            if cur or open_arg:
                args.append(cur)
            cur, open_arg = "", False
        else:
            cur += ch
    if cur or open_arg:
        args.append(cur)
    return args


def substitute_args(template: str, args: list[str]) -> str:
    out = template.replace("$ARGUMENTS", " ".join(args)).replace("$@", " ".join(args))
    return re.sub(r"\$(\d+)", lambda m: args[int(m.group(1)) - 1] if 0 < int(m.group(1)) <= len(args) else "", out)


def load_commands_from_dir(directory: Path, source: str) -> list[SlashCommand]:
    out = []
    if not directory.is_dir():
        return out
    for f in sorted(directory.rglob("*.md")):
        try:
            meta, body = parse_frontmatter(f.read_text())
        except OSError:
            continue
        name = ":".join(f.relative_to(directory).with_suffix("").parts)
        first = next((ln.strip().lstrip("# ") for ln in body.splitlines() if ln.strip()), "")
        out.append(SlashCommand(name, meta.get("description") or first[:60], meta.get("argument-hint") or None, body, source))
    return out


def load_file_commands(cwd: str | Path | None = None, home: Path | None = None) -> list[SlashCommand]:
    """User commands, then project commands; a project command replaces a user command of the same name."""
    by_name = {c.name: c for c in load_commands_from_dir((home or Path.home()) / ".research_b200" / "commands", "(user)")}
    by_name.update({c.name: c for c in load_commands_from_dir(Path(cwd or ".") / ".research_b200" / "commands", "(project)")})
    return list(by_name.values())


def expand_file_command(text: str, commands: list[SlashCommand]) -> str | None:
    """``/name args`` -> the command's prompt with the arguments filled in; None if ``name`` is not a file command."""
    if not text.startswith("/"):
        return None
    name, _, rest = text[1:].partition(" ")
    cmd = next((c for c in commands if c.name == name and c.content is not None), None)
    return substitute_args(cmd.content, parse_command_args(rest)).strip() if cmd else None


def find_similar_command(name: str, known: list[str]) -> str | None:
    close = difflib.get_close_matches(name, known, n=1, cutoff=0.6)
    return close[0] if close else next((k for k in known if k.startswith(name)), None)


def get_command_arg_hint(name: str, commands: list[SlashCommand]) -> str | None:
    return next((c.arg_hint for c in commands if c.name == name), None)


# ------------------------------------------------------------------------------------------- built-ins that need the runner
def thinking_budget(endpoint: Any) -> int | None:
    t = endpoint.extra_params.get("thinking")
    return int(t.get("budget_tokens", 0)) or None if isinstance(t, dict) and t.get("type") == "enabled" else None


def handle_thinking(runner: Any, arg: str) -> SlashCommandResult:
    """No argument: report. ``on`` / ``off`` / a number of tokens: set the request's thinking budget (``reasoning_effort`` for
    providers that take an effort level instead) and show or hide the thinking text."""
    ep, arg = runner.endpoint, arg.strip().lower()
    if not arg:
        b = thinking_budget(ep)
        return SlashCommandResult(message=f"thinking: {'on, budget ' + str(b) + ' tokens' if b else 'off'}" +
                                  (f", effort {ep.reasoning_effort}" if ep.reasoning_effort else ""))
    if arg in ("off", "0", "false", "no"):
        extra = {k: v for k, v in ep.extra_params.items() if k != "thinking"}
        runner.set_endpoint(replace(ep, extra_params=extra, reasoning_effort=None))
        if hasattr(runner.frontend, "show_thinking"):
            runner.frontend.show_thinking = False
        return SlashCommandResult(message="thinking off", persist={"thinking": "off"})
    if arg in ("on", "true", "yes"):
        budget = thinking_budget(ep) or DEFAULT_THINKING_BUDGET
    elif arg.isdigit() and int(arg) >= 1024:
        budget = int(arg)
    else:
        return SlashCommandResult(message="usage: /thinking [on|off|<budget in tokens, at least 1024>]")
    effort = "low" if budget < 4096 else "medium" if budget < 16384 else "high"
    runner.set_endpoint(replace(ep, extra_params={**ep.extra_params, "thinking": {"type": "enabled", "budget_tokens": budget}},
                                reasoning_effort=effort, max_tokens=max(ep.max_tokens, budget + 1024)))
    if hasattr(runner.frontend, "show_thinking"):
        runner.frontend.show_thinking = True
    return SlashCommandResult(message=f"thinking on, budget {budget} tokens", persist={"thinking": budget})


async def handle_slice(runner: Any, arg: str) -> SlashCommandResult:
    from ..agents.dtypes import Actor, Trajectory
    from ..agents.slice import apply_slice, parse_slice_spec

    msgs = list(runner.state.actor.trajectory.messages)
    if not arg.strip():
        return SlashCommandResult(message=f"{len(msgs)} messages. usage: /slice 0:4, summarize:4:{max(len(msgs) - 4, 4)}, {max(len(msgs) - 4, 4)}:   "
                                          "(ranges, summarize:a:b[:\"goal\"], compact:a:b, inject:\"text\")")
    try:
        segments = parse_slice_spec(arg)
        new = await apply_slice(msgs, segments)
    except (ValueError, IndexError) as e:
        return SlashCommandResult(message=f"cannot slice: {e}")
    if not new:
        return SlashCommandResult(message="that slice would leave no messages")
    sid = None
    if runner.store is not None:
        sid = await runner.store.create(runner.endpoint.to_dict(), await runner.environment.serialize() if runner.environment else None,
                                        parent_id=runner.state.session_id, branch_point=len(msgs), tags={**(runner.session_tags or {}), "slice": arg})
        for m in new:
            await runner.store.append_message(sid, m)
    runner.state = replace(runner.state, actor=Actor(Trajectory(tuple(new)), runner.endpoint), session_id=sid, stop=None, pending_tool_calls=())
    return SlashCommandResult(message=f"{len(msgs)} -> {len(new)} messages" + (f"; now in session {sid}" if sid else ""))


def current_env_name(env: Any) -> str:
    if env is None:
        return "none"
    get = getattr(env, "get_name", None)
    return get() if get is not None else type(env).__name__.replace("Environment", "").lower()


async def handle_env(runner: Any, arg: str) -> SlashCommandResult:
    """``/env``: what is active. ``/env list``: what exists. ``/env coding+ask_user [tool preset]``: switch, in a child session
    that branches from here (the parent keeps the conversation as it was under the old tools)."""
    from ..agents.presets import ENVIRONMENTS, environment_from_spec

    arg = arg.strip()
    current = getattr(runner, "env_spec", None) or current_env_name(runner.environment)
    if not arg:
        tools = [t.function.name for t in runner.environment.get_tools()] if runner.environment is not None else []
        return SlashCommandResult(message=f"environment: {current} (tools: {', '.join(tools) or 'none'}); "
                                          f"available: {', '.join(sorted(ENVIRONMENTS))}")
    if arg == "list":
        return SlashCommandResult(message="available environments (combine with +):\n" + "\n".join(f"  {n}" for n in sorted(ENVIRONMENTS)))
    spec, _, tools = arg.partition(" ")
    if spec == current and not tools.strip():
        return SlashCommandResult(message=f"already using env: {spec}")
    try:
        env = environment_from_spec(spec, runner.cwd, tools.strip() or None)
    except KeyError as e:
        first = spec.split("+")[0]
        near = find_similar_command(first, sorted(ENVIRONMENTS)) if first not in ENVIRONMENTS else None
        return SlashCommandResult(message=str(e).strip("'\"") + (f" (did you mean {near}?)" if near else ""))
    except ValueError as e:
        return SlashCommandResult(message=str(e))
    if hasattr(env, "on_session_start"):
        await env.on_session_start(runner.state.session_id or "chat")
    runner.set_environment(env)
    runner.env_spec = spec
    note = ""
    if runner.store is not None and runner.state.session_id:
        msgs = runner.state.actor.trajectory.messages
        child = await runner.store.create(runner.endpoint.to_dict(), await env.serialize(), parent_id=runner.state.session_id, branch_point=len(msgs),
                                          tags={**(runner.session_tags or {}), "env": spec})
        for m in msgs:
            await runner.store.append_message(child, m)
        runner.state = replace(runner.state, session_id=child)
        note = f"; now in session {child}"
    return SlashCommandResult(message=f"environment: {spec} (tools: {', '.join(t.function.name for t in env.get_tools()) or 'none'}){note}",
                              persist={"env": spec})


async def handle_session(runner: Any, arg: str) -> SlashCommandResult:
    """No argument: the ten most recent sessions. An id (a unique prefix is enough): continue in that session, with its
    messages, its endpoint settings where they were stored, and its environment restored from what the session recorded."""
    from ..agents.agents import resume_session
    from ..agents.doctor import format_time_ago
    from ..agents.dtypes import Endpoint

    if runner.store is None:
        return SlashCommandResult(message="this chat stores no sessions (--no-session)")
    sessions = sorted(await runner.store.list(), key=lambda s: s.updated_at, reverse=True)
    arg = arg.strip()
    if not arg:
        rows = [f"{'*' if s.session_id == runner.state.session_id else ' '} {s.session_id}  {s.num_messages:>3} msgs  {format_time_ago(s.updated_at):>9}  "
                f"{s.endpoint.get('model', '?')}" for s in sessions[:10]]
        return SlashCommandResult(message="\n".join(rows) or "no sessions yet")
    hits = [s for s in sessions if s.session_id.startswith(arg)]
    if len(hits) != 1:
        return SlashCommandResult(message=f"{len(hits)} sessions match {arg!r}" + (": " + ", ".join(s.session_id for s in hits[:5]) if hits else ""))
    target = hits[0]
    stored = {k: v for k, v in target.endpoint.items() if k in Endpoint.__dataclass_fields__ and k not in ("api_key", "oauth_token", "engine")}
    endpoint = replace(runner.endpoint, **stored) if stored.get("provider") == runner.endpoint.provider else runner.endpoint
    env_cls = type(runner.environment) if runner.environment is not None else None
    try:
        state = await resume_session(target.session_id, runner.store, endpoint, env_cls if target.environment is not None else None, runner.max_turns)
    except Exception as e:  # noqa: BLE001 - a session written by another environment type, a damaged file ...
        return SlashCommandResult(message=f"cannot continue {target.session_id}: {type(e).__name__}: {e}")
    runner.set_endpoint(endpoint)
    if state.environment is not None:
        runner.set_environment(state.environment)
    runner.state = replace(state, environment=runner.environment, stop=None)
    return SlashCommandResult(message=f"now in session {target.session_id} ({len(state.actor.trajectory.messages)} messages, model {endpoint.model or endpoint.provider})")


async def handle_branch(runner: Any, arg: str) -> SlashCommandResult:
    if runner.store is None or not runner.state.session_id:
        return SlashCommandResult(message="nothing stored to branch from yet")
    msgs = runner.state.actor.trajectory.messages
    try:
        n = int(arg) if arg.strip() else len(msgs)
    except ValueError:
        return SlashCommandResult(message="usage: /branch [number of messages to keep]")
    if not 0 < n <= len(msgs):
        return SlashCommandResult(message=f"keep between 1 and {len(msgs)} messages")
    from ..agents.dtypes import Actor, Trajectory

    parent = runner.state.session_id
    sid = await runner.store.branch(parent, n)
    runner.state = replace(runner.state, actor=Actor(Trajectory(tuple(msgs[:n])), runner.endpoint), session_id=sid, stop=None, pending_tool_calls=())
    return SlashCommandResult(message=f"branched after message {n}: now in session {sid} (parent {parent})")


async def handle_edit(runner: Any, arg: str) -> SlashCommandResult:
    """``/edit new text`` rewords the last user message, ``/edit 3 new text`` message 3: the conversation forks into a
    child session that ends just before that message, and the new wording is sent."""
    msgs = runner.state.actor.trajectory.messages
    head, _, rest = arg.strip().partition(" ")
    if head.isdigit() and rest.strip():
        index, text = int(head), rest.strip()
    else:
        index, text = next((i for i in range(len(msgs) - 1, -1, -1) if msgs[i].role == "user"), -1), arg.strip()
    if not text:
        return SlashCommandResult(message="usage: /edit [message number] <new text>")
    if not 0 <= index < len(msgs) or msgs[index].role != "user":
        users = [i for i, m in enumerate(msgs) if m.role == "user"]
        return SlashCommandResult(message=f"message {index} is not a user message (user messages: {users})" if users else "no user message to edit yet")
    from ..agents.dtypes import Actor, Trajectory

    note = f"reworded message {index}"
    sid = runner.state.session_id
    if runner.store is not None and sid:
        parent = sid
        sid = await runner.store.branch(parent, index, reason="message_edit")      # the runner appends the new wording itself
        note += f": now in session {sid} (parent {parent})"
    runner.state = replace(runner.state, actor=Actor(Trajectory(tuple(msgs[:index])), runner.endpoint), session_id=sid, stop=None,
                           pending_tool_calls=())
    return SlashCommandResult(message=note, expanded_text=text)


async def handle_tree(runner: Any, arg: str) -> SlashCommandResult:
    if runner.store is None or not runner.state.session_id:
        return SlashCommandResult(message="this conversation is not stored")
    from ..agents.store import format_session_tree

    root = await runner.store.root_of(runner.state.session_id)
    return SlashCommandResult(message=format_session_tree(await runner.store.tree(root), current=runner.state.session_id))
