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

from .dtypes import (Actor, AgentState, Message, RunConfig, StopReason, StreamDone, ToolCall, ToolResult,
                     ToolResultReceived, Trajectory)


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
        ok = True
        if env is not None and env.requires_confirmation(call) and run_config.confirm_tool is not None:
            ok = await run_config.confirm_tool(call, state, run_config)
        if env is None:
            result = ToolResult(call.id, is_error=True, error=f"no environment to run tool {call.name!r}")
        elif not ok:
            result = ToolResult(call.id, is_error=True, error="tool call rejected by the user")
        else:
            try:
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
        traj = traj.append(Message("tool", content, tool_call_id=call.id, name=call.name))
        if run_config.on_chunk is not None:
            await run_config.on_chunk(ToolResultReceived(tool_call_id=call.id, content=content, is_error=result.is_error,
                                                         details=dict(result.metadata)))
        if run_config.session_store is not None and state.session_id:
            await run_config.session_store.append_message(state.session_id, traj.messages[-1])
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
    tools = tuple(state.environment.get_tools()) if state.environment is not None else ()
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
