"""The agent loop: ``run_agent`` -> ``run_agent_step`` -> ``rollout`` (model call) ->
``process_pending_tools`` (environment), with stop handlers, cancellation, session persistence
and resume (surface of rollouts/agents.py:208-1021, asyncio instead of trio).

State is immutable: every step returns a new ``AgentState``. ``rollout`` routes on
``endpoint.provider``; with ``RunConfig.use_tito`` the token-level providers are used so that
``Choice.token_ids`` / log-probs are the engine's own (no re-tokenisation).
"""

from __future__ import annotations

import asyncio
import time
import uuid
from dataclasses import replace
from typing import Any

from .dtypes import (Actor, AgentState, ImageContent, LLMCallStart, Message, TextContent, RunConfig, StopReason, StreamDone, StreamEvent, TextDelta, ThinkingDelta, ToolCall,
                     ToolCallEnd, ToolConfirmResult, ToolExecutionStart, ToolResult, ToolResultReceived, Trajectory)


# ------------------------------------------------------------------------------ stop handlers
def handle_stop_max_turns(state: AgentState) -> AgentState:
    if state.turn_idx >= state.max_turns:
        return replace(state, stop=StopReason.MAX_TURNS)
    return state


def handle_stop_on_empty_message(state: AgentState) -> AgentState:
    msgs = state.actor.trajectory.messages
    if msgs and msgs[-1].role == "assistant" and not msgs[-1].text().strip() and not msgs[-1].get_tool_calls():
        return replace(state, stop=StopReason.NO_TOOL_CALLS)
    return state


def compose_stop_handlers(*handlers):
    def composed(state: AgentState) -> AgentState:
        for h in handlers:
            state = h(state)
            if state.stop is not None:
                break
        return state

    return composed


def inject_turn_warning(warning_at: int = 2, text: str | None = None):
    """For ``RunConfig.on_step_start``: when exactly ``warning_at`` turns are left (of ``state.max_turns``), a user message
    says so, once, so that the model wraps up instead of being cut off (rollouts/agents.py:167-205)."""
    assert warning_at > 0

    def handler(state: AgentState) -> AgentState:
        if state.max_turns - state.turn_idx != warning_at or state.max_turns <= warning_at:
            return state
        note = Message("user", text or f"You have {warning_at} turn{'s' if warning_at != 1 else ''} left. Finish the task now and give your final answer.")
        return replace(state, actor=replace(state.actor, trajectory=state.actor.trajectory.append(note)))

    return handler


def estimated_tokens(state: AgentState) -> int:
    """Tokens this episode has used: the providers' own counts when they reported any, else a quarter of the characters
    in the conversation."""
    if state.usage.total_tokens:
        return state.usage.total_tokens
    return sum(len(m.text()) + sum(len(str(c.args)) for c in m.tool_calls) for m in state.actor.trajectory.messages) // 4


def handle_stop_token_budget(max_tokens: int):
    def handler(state: AgentState) -> AgentState:
        return replace(state, stop=StopReason.BUDGET_EXCEEDED) if estimated_tokens(state) >= max_tokens else state

    return handler


def handle_stop_cost_budget(max_cost_usd: float, cost_fn=None):
    """Stop once the episode's cost reaches the budget; the default cost is what the providers' usage records add up to."""
    def handler(state: AgentState) -> AgentState:
        cost = cost_fn(state) if cost_fn is not None else state.usage.cost.total
        return replace(state, stop=StopReason.BUDGET_EXCEEDED) if cost >= max_cost_usd else state

    return handler


def make_tool_reminder(text: str = "Use the available tools to make progress on the task, or give your final answer.", max_reminders: int = 2):
    """For ``RunConfig.handle_no_tool``: instead of ending the episode when the model answers without a tool call, remind
    it, at most ``max_reminders`` times in a row; after that the episode ends as usual."""
    async def handler(state: AgentState, run_config: RunConfig) -> AgentState:
        msgs = state.actor.trajectory.messages
        streak = 0
        for m in reversed(msgs[:-1]):
            if m.role == "user" and m.metadata.get("reminder"):
                streak += 1
            elif m.role in ("tool",) or (m.role == "user" and not m.metadata.get("reminder")):
                break
        if streak >= max_reminders:
            return replace(state, stop=StopReason.NO_TOOL_CALLS)
        note = Message("user", text, metadata={"reminder": True})
        if run_config.session_store is not None and state.session_id:
            await run_config.session_store.append_message(state.session_id, note)
        return replace(state, actor=replace(state.actor, trajectory=state.actor.trajectory.append(note)))

    return handler


def make_confirm_with_feedback(ask, out=print):
    """A ``RunConfig.confirm_tool`` for terminals: ``y`` runs the call, ``n`` refuses it and asks why (the reason reaches the
    model as a user message after the refused result), anything else skips silently. ``ask(prompt) -> str`` may be a plain
    or an async function."""
    async def _ask(prompt: str) -> str:
        r = ask(prompt)
        return (await r) if asyncio.iscoroutine(r) else r

    async def confirm(call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolConfirmResult:
        out(f"\nrun {call.name}({call.args})?\n  [y] yes   [n] no, and say why   [s] skip")
        choice = (await _ask("choice: ")).strip().lower()
        if choice == "y":
            return ToolConfirmResult(True)
        if choice == "n":
            why = (await _ask("why not / what instead: ")).strip()
            return ToolConfirmResult(False, ToolResult(call.id, is_error=True, error="rejected by the user"), why or None)
        return ToolConfirmResult(False, ToolResult(call.id, is_error=True, error="skipped by the user"))

    return confirm


async def stdout_handler(event: StreamEvent) -> None:
    """The plainest ``on_chunk``: text and thinking as they stream, one line per tool call and result."""
    if isinstance(event, (TextDelta, ThinkingDelta)):
        print(event.delta, end="", flush=True)
    elif isinstance(event, ToolCallEnd):
        print(f"\n[tool] {event.name}({event.args})", flush=True)
    elif isinstance(event, ToolResultReceived):
        print(f"[{'error' if event.is_error else 'result'}] {event.content[:500]}", flush=True)
    elif isinstance(event, StreamDone):
        print(flush=True)


async def handle_no_tool_stop(state: AgentState, run_config: RunConfig) -> AgentState:
    """Default when the model answers without calling a tool: the episode is over."""
    return replace(state, stop=StopReason.NO_TOOL_CALLS)


async def handle_no_tool_continue(state: AgentState, run_config: RunConfig) -> AgentState:
    return state


# ------------------------------------------------------------------------------ model call
async def rollout(actor: Actor, run_config: RunConfig) -> Actor:
    """One model call: appends the assistant message and the completion to the trajectory."""
    from .providers import get_provider

    fn = get_provider(actor.endpoint.provider, token_level=run_config.use_tito)
    if run_config.api_limiter is not None:
        async with run_config.api_limiter:
            return await fn(actor, run_config)
    return await fn(actor, run_config)


# ------------------------------------------------------------------------------ tools
async def process_pending_tools(state: AgentState, run_config: RunConfig) -> AgentState:
    """Execute pending tool calls one by one; each runs against a freshly deserialised copy of the
    environment so a tool that raises cannot leave half-applied state behind."""
    env = state.environment
    traj = state.actor.trajectory
    for i in range(state.next_tool_idx, len(state.pending_tool_calls)):
        call = state.pending_tool_calls[i]
        if run_config.cancel_event is not None and run_config.cancel_event.is_set():
            return replace(state, actor=replace(state.actor, trajectory=traj), environment=env, next_tool_idx=i,
                           stop=StopReason.ABORTED)
        ok, feedback, refused = True, None, None
        if env is not None and env.requires_confirmation(call) and run_config.confirm_tool is not None:
            answer = await run_config.confirm_tool(call, state, run_config)
            if isinstance(answer, ToolConfirmResult):
                ok, refused, feedback = answer.proceed, answer.tool_result, answer.user_message
            else:
                ok = bool(answer)
        if env is None:
            result = ToolResult(call.id, is_error=True, error=f"no environment to run tool {call.name!r}")
        elif not ok:
            result = refused or ToolResult(call.id, is_error=True, error="tool call rejected by the user")
        else:
            try:
                if run_config.on_chunk is not None:
                    await run_config.on_chunk(ToolExecutionStart(tool_call_id=call.id, tool_name=call.name))
                snapshot = await env.serialize()
                work_env = await type(env).deserialize(snapshot)
                if run_config.tool_limiter is not None:
                    async with run_config.tool_limiter:
                        result = await work_env.exec_tool(call, state, run_config)
                else:
                    result = await work_env.exec_tool(call, state, run_config)
                env = work_env
            except asyncio.CancelledError:
                raise
            except Exception as e:  # noqa: BLE001 - tool failures are fed back to the model
                result = ToolResult(call.id, is_error=True, error=f"{type(e).__name__}: {e}")
        content = result.content if not result.is_error else f"Error: {result.error or result.content}"
        image = result.metadata.get("image") if not result.is_error else None
        if isinstance(image, dict) and image.get("data"):
            # a tool that returns a picture (a screenshot, an image file that was read): text and image blocks together
            body: Any = [TextContent(content), ImageContent(image["data"], image.get("mime_type", "image/png"))]
        else:
            body = content
        traj = traj.append(Message("tool", body, tool_call_id=call.id, name=call.name))
        if run_config.on_chunk is not None:
            await run_config.on_chunk(ToolResultReceived(tool_call_id=call.id, content=content, is_error=result.is_error,
                                                         details={k: v for k, v in result.metadata.items() if k != "image"}))
        if run_config.session_store is not None and state.session_id:
            await run_config.session_store.append_message(state.session_id, traj.messages[-1])
        if feedback:
            # the user said why not: every remaining call of this turn gets its (refused) result first, so that the
            # conversation stays well-formed, then the guidance follows as a user message
            for rest in state.pending_tool_calls[i + 1:]:
                traj = traj.append(Message("tool", "Error: not run (the user interrupted this turn)", tool_call_id=rest.id, name=rest.name))
            traj = traj.append(Message("user", feedback))
            if run_config.session_store is not None and state.session_id:
                for m in traj.messages[-(len(state.pending_tool_calls) - i):]:
                    await run_config.session_store.append_message(state.session_id, m)
            return replace(state, actor=replace(state.actor, trajectory=traj), environment=env, pending_tool_calls=(), next_tool_idx=0)
        if result.stop_reason is not None:
            return replace(state, actor=replace(state.actor, trajectory=traj), environment=env,
                           pending_tool_calls=(), next_tool_idx=0, stop=result.stop_reason)
    return replace(state, actor=replace(state.actor, trajectory=traj), environment=env, pending_tool_calls=(), next_tool_idx=0)


# ------------------------------------------------------------------------------ steps
async def run_agent_step(state: AgentState, run_config: RunConfig) -> AgentState:
    """One turn: finish pending tools, call the model, queue its tool calls."""
    if state.pending_tool_calls:
        state = await process_pending_tools(state, run_config)
        if state.stop is not None:
            return state
    stop_handler = run_config.handle_stop or handle_stop_max_turns
    state = stop_handler(state)
    if state.stop is not None:
        return state
    if run_config.on_step_start is not None:
        state = run_config.on_step_start(state)
    tools = tuple(state.environment.get_tools()) if state.environment is not None else ()
    if run_config.on_chunk is not None:
        await run_config.on_chunk(LLMCallStart())
    actor = await rollout(replace(state.actor, tools=tools), run_config)
    last = actor.trajectory.messages[-1]
    if run_config.session_store is not None and state.session_id:
        await run_config.session_store.append_message(state.session_id, last)
    usage = state.usage + actor.trajectory.completions[-1].usage if actor.trajectory.completions else state.usage
    state = replace(state, actor=actor, turn_idx=state.turn_idx + 1, usage=usage)
    hook = getattr(state.environment, "on_assistant_message", None)
    if hook is not None:
        # an environment that reads the reply itself (code blocks or answers written as text, by models without tool
        # calling) may append messages, change its own state, or set a stop reason; messages it adds are stored too
        before = len(state.actor.trajectory.messages)
        state = await hook(last, state)
        if run_config.session_store is not None and state.session_id:
            for m in state.actor.trajectory.messages[before:]:
                await run_config.session_store.append_message(state.session_id, m)
        if state.stop is not None:
            return state
        if len(state.actor.trajectory.messages) > before and not last.get_tool_calls():
            return state                      # the environment answered: next turn, not "no tool calls"
    calls = tuple(last.get_tool_calls())
    if calls:
        state = replace(state, pending_tool_calls=calls, next_tool_idx=0)
        return await process_pending_tools(state, run_config)
    handler = run_config.handle_no_tool or handle_no_tool_stop
    return await handler(state, run_config)


async def run_agent(state: AgentState, run_config: RunConfig | None = None) -> list[AgentState]:
    """Run until a stop reason is set; returns every intermediate state (last one is final)."""
    run_config = run_config or RunConfig()
    if run_config.session_store is not None and state.session_id is None:
        sid = await run_config.session_store.create(state.actor.endpoint.to_dict(),
                                                    await state.environment.serialize() if state.environment else None,
                                                    tags=dict(run_config.session_tags) if run_config.session_tags else None)
        state = replace(state, session_id=sid)
        for m in state.actor.trajectory.messages:
            await run_config.session_store.append_message(sid, m)
    states = [state]
    try:
        while state.stop is None:
            if run_config.cancel_event is not None and run_config.cancel_event.is_set():
                state = replace(state, stop=StopReason.ABORTED)
                states.append(state)
                break
            state = await run_agent_step(state, run_config)
            states.append(state)
    except asyncio.CancelledError:
        state = replace(state, stop=StopReason.ABORTED)
        states.append(state)
        if run_config.session_store is not None and state.session_id:
            await asyncio.shield(run_config.session_store.update(state.session_id, status="aborted"))
        raise
    if run_config.on_chunk is not None:
        await run_config.on_chunk(StreamDone(stop_reason=state.stop.value if state.stop else "stop"))
    if run_config.session_store is not None and state.session_id:
        await run_config.session_store.update(state.session_id, status=state.stop.value if state.stop else "done")
    return states


async def resume_session(session_id: str, store: Any, endpoint, environment_cls=None, max_turns: int = 10) -> AgentState:
    """Rebuild an ``AgentState`` from a stored session (messages + serialised environment).

    A session that stopped between an assistant message with tool calls and their results
    resumes by re-queuing exactly the calls that have no result yet."""
    session, messages = await store.get(session_id)
    env = None
    if environment_cls is not None and session.environment is not None:
        env = await environment_cls.deserialize(session.environment)
    traj = Trajectory(tuple(messages))
    pending: tuple[ToolCall, ...] = ()
    if messages:
        last_assistant = max((i for i, m in enumerate(messages) if m.role == "assistant"), default=-1)
        if last_assistant >= 0:
            done = {m.tool_call_id for m in messages[last_assistant + 1:] if m.role == "tool"}
            pending = tuple(c for c in messages[last_assistant].get_tool_calls() if c.id not in done)
    turns = sum(1 for m in messages if m.role == "assistant")
    return AgentState(actor=Actor(traj, endpoint), environment=env, turn_idx=turns, max_turns=max_turns,
                      pending_tool_calls=pending, session_id=session_id)


def new_id(prefix: str = "id") -> str:
    return f"{prefix}_{uuid.uuid4().hex[:12]}_{int(time.time())}"
