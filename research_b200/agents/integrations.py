"""Adapters for "verifiers"-style environments (the Prime Intellect environment hub), so their datasets, rubrics and
multi-turn logic drive this framework's ``evaluate`` and agent loop (dev/integration-evaluation/local.py:40-160 is the
reference's driver; the ``rollouts.integrations.prime.prime_reward_fn`` it imports is not in the reference tree, so the
contract below is taken from how that driver and its configs use it).

Nothing here imports the ``verifiers`` package: the environment is duck-typed.

* dataset: ``env.dataset`` or ``env.eval_dataset``, rows with ``prompt`` (chat list) or ``question``, plus ``answer`` /
  ``info`` / ``task``;
* rubric: ``env.rubric.score_rollout(prompt=, completion=, answer=, state=, task=, info=)`` (plain or coroutine)
  returning a number, a mapping or an object with ``reward`` (and optionally ``metrics``); or, failing that,
  ``rubric.reward_funcs`` with ``rubric.reward_weights``, each function called with the arguments it names;
* multi-turn: ``env.is_completed(messages, state)`` and ``env.env_response(messages, state) -> (messages, state)``.
"""

from __future__ import annotations

import asyncio
import inspect
from dataclasses import replace
from typing import Any, Callable, Iterable

from .dtypes import AgentState, Message, Metric, RunConfig, Score, StopReason, Trajectory


def to_chat(messages: Iterable[Message]) -> list[dict[str, Any]]:
    out = []
    for m in messages:
        d: dict[str, Any] = {"role": m.role, "content": m.text()}
        if m.tool_calls:
            d["tool_calls"] = [{"id": c.id, "type": "function", "function": {"name": c.name, "arguments": c.args}} for c in m.tool_calls]
        if m.tool_call_id:
            d["tool_call_id"] = m.tool_call_id
        out.append(d)
    return out


def dataset_rows(env: Any, limit: int | None = None) -> list[dict[str, Any]]:
    """Rows of the environment's dataset (``dataset`` first, then ``eval_dataset``), as plain dicts."""
    for attr in ("dataset", "eval_dataset"):
        ds = getattr(env, attr, None)
        if ds is not None:
            rows = [dict(r) for r in ds]
            return rows[:limit] if limit is not None else rows
    raise ValueError("the environment has neither a dataset nor an eval_dataset")


def prepare_messages(row: dict[str, Any], system_prompt: str | None = None) -> list[Message]:
    """Chat-list ``prompt`` rows as they are; ``question`` rows as one user message (after the system prompt)."""
    prompt = row.get("prompt")
    if isinstance(prompt, (list, tuple)) and prompt:
        return [Message(role=p["role"], content=p["content"]) for p in prompt]
    text = prompt if isinstance(prompt, str) else row.get("question", "")
    head = [Message("system", system_prompt)] if system_prompt else []
    return head + [Message("user", str(text))]


async def _maybe_await(x: Any) -> Any:
    return await x if inspect.isawaitable(x) else x


def _call_with_known_args(fn: Callable[..., Any], available: dict[str, Any]) -> Any:
    sig = inspect.signature(fn)
    if any(p.kind is inspect.Parameter.VAR_KEYWORD for p in sig.parameters.values()):
        return fn(**available)
    return fn(**{k: v for k, v in available.items() if k in sig.parameters})


def _as_score(result: Any) -> Score:
    if isinstance(result, Score):
        return result
    if isinstance(result, (int, float)):
        return Score((Metric("reward", float(result), 1.0),))
    reward = result.get("reward") if isinstance(result, dict) else getattr(result, "reward", None)
    metrics = (result.get("metrics") if isinstance(result, dict) else getattr(result, "metrics", None)) or {}
    if reward is None:
        raise TypeError(f"cannot read a reward from a rubric result of type {type(result).__name__}")
    return Score((Metric("reward", float(reward), 1.0),) + tuple(Metric(str(k), float(v), 0.0) for k, v in metrics.items()))


def split_prompt_completion(traj: Trajectory, row: dict[str, Any]) -> tuple[list[dict], list[dict]]:
    """The rubric sees the prompt and, separately, everything the episode added to it: the split is at the first
    assistant message (system prompts added by the caller count as prompt)."""
    n = next((i for i, m in enumerate(traj.messages) if m.role == "assistant"), len(traj.messages))
    chat = to_chat(traj.messages)
    return chat[:n], chat[n:]


def prime_reward_fn(env: Any, state_of: Callable[[Trajectory, dict[str, Any]], dict[str, Any]] | None = None) -> Callable[..., Any]:
    """``score_fn(trajectory, row) -> Score`` for ``EvalConfig`` from the environment's rubric. ``state_of`` builds the
    rubric's ``state`` argument (default: the trajectory's metadata plus the turn count)."""
    rubric = getattr(env, "rubric", None)
    if rubric is None:
        raise ValueError("the environment has no rubric")

    async def score(traj: Trajectory, row: dict[str, Any]) -> Score:
        prompt, completion = split_prompt_completion(traj, row)
        state = state_of(traj, row) if state_of else {**traj.metadata, "turn": sum(m.role == "assistant" for m in traj.messages)}
        args = {"prompt": prompt, "completion": completion, "answer": row.get("answer", ""), "state": state,
                "task": row.get("task", "default"), "info": row.get("info", {}), "parser": getattr(env, "parser", None)}
        if hasattr(rubric, "score_rollout"):
            return _as_score(await _maybe_await(_call_with_known_args(rubric.score_rollout, args)))
        funcs = list(getattr(rubric, "reward_funcs", []) or [])
        if not funcs:
            raise ValueError("the rubric has neither score_rollout nor reward_funcs")
        weights = list(getattr(rubric, "reward_weights", []) or [1.0] * len(funcs))
        metrics = []
        for fn, w in zip(funcs, weights):
            v = await _maybe_await(_call_with_known_args(fn, args))
            metrics.append(Metric(getattr(fn, "__name__", "reward"), float(v), float(w)))
        total = sum(m.value * m.weight for m in metrics)
        # verifiers sums weighted rewards (no division by the weights): keep that number as the reward
        return Score((Metric("reward", total, 1.0),) + tuple(replace(m, weight=0.0) for m in metrics))

    return score


def multiturn_handler(env: Any, state: dict[str, Any] | None = None) -> Callable[[AgentState, RunConfig], Any]:
    """A ``RunConfig.handle_no_tool`` that lets the environment answer the assistant: stop when ``is_completed`` says
    so, otherwise append what ``env_response`` returns and go on. The environment's own state dict lives in the
    closure (one handler per episode)."""
    env_state: dict[str, Any] = dict(state or {})

    async def handle(agent_state: AgentState, run_config: RunConfig) -> AgentState:
        chat = to_chat(agent_state.actor.trajectory.messages)
        env_state["turn"] = env_state.get("turn", 0) + 1
        if await _maybe_await(env.is_completed(chat, env_state)):
            return replace(agent_state, stop=StopReason.TASK_COMPLETED)
        reply, new_state = await _maybe_await(env.env_response(chat, env_state))
        if isinstance(new_state, dict):
            env_state.update(new_state)
        msgs = [Message(role=r.get("role", "user"), content=r.get("content", "")) for r in (reply if isinstance(reply, list) else [reply])]
        if not msgs:
            return replace(agent_state, stop=StopReason.TASK_COMPLETED)
        traj = agent_state.actor.trajectory.append(*msgs)
        traj = replace(traj, metadata={**traj.metadata, "env_state": dict(env_state)})
        return replace(agent_state, actor=replace(agent_state.actor, trajectory=traj))

    return handle


def eval_config_for(env: Any, endpoint: Any, max_turns: int | None = None, system_prompt: str | None = None, **kw: Any):
    """An ``EvalConfig`` wired to the environment: its prompts, its rubric and (for multi-turn environments) its
    replies. A fresh reply handler is made per call of ``run_config_factory``; ``evaluate`` itself uses one shared
    ``RunConfig``, so multi-turn environments should be evaluated with ``max_concurrent=1`` or through
    ``evaluate_env``."""
    from .dtypes import EvalConfig

    turns = max_turns or int(getattr(env, "max_turns", 1) or 1)
    return EvalConfig(endpoint=endpoint, score_fn=prime_reward_fn(env), prepare_messages=lambda row: prepare_messages(row, system_prompt),
                      max_turns=max(turns, 1), **kw)


async def evaluate_env(env: Any, endpoint: Any, limit: int | None = None, max_turns: int | None = None, max_concurrent: int = 4,
                       system_prompt: str | None = None, eval_name: str = "verifiers_eval", output_dir: str | None = None):
    """Evaluate ``endpoint`` on the environment's dataset; every episode gets its own reply handler."""
    from .evaluation import EvalReport, compute_summary_metrics, evaluate_sample

    rows = dataset_rows(env, limit)
    multi = hasattr(env, "env_response") and hasattr(env, "is_completed")
    sem = asyncio.Semaphore(max_concurrent)

    async def one(i: int, row: dict[str, Any]):
        cfg = eval_config_for(env, endpoint, max_turns, system_prompt, eval_name=eval_name, n_retries=0,
                              run_config=RunConfig(handle_no_tool=multiturn_handler(env, {"answer": row.get("answer", ""), "info": row.get("info", {})})
                                                   if multi else None))
        async with sem:
            return await evaluate_sample(row, str(row.get("id", i)), cfg)

    samples = list(await asyncio.gather(*[one(i, r) for i, r in enumerate(rows)]))
    report = EvalReport(eval_name, samples, compute_summary_metrics(samples), {"endpoint": endpoint.to_dict(), "environment": type(env).__name__})
    if output_dir:
        report.save(output_dir)
    return report


class StatefulToolEnvironment:
    """A verifiers-style *stateful tool* environment (``oai_tools`` + ``env_response(messages, state)``, e.g. a kernel
    bench that compiles and times what the model wrote) as an agent environment (dev/integration-evaluation/configs/
    prime_backend_bench.py:140-400): its tools are advertised as they are; a tool call is replayed to the wrapped
    environment as an assistant message with that call and the first ``tool`` message it answers with is the result; an
    assistant message WITHOUT tool calls is also shown to it (environments that parse code from text answer with user
    messages, which are appended). What the wrapped code prints goes to ``logger`` instead of the terminal."""

    def __init__(self, env: Any, state: dict[str, Any] | None = None, messages: list[dict[str, Any]] | None = None, logger: Any = None):
        import logging

        self.env, self.state, self.messages = env, dict(state or {}), list(messages or [])
        self.logger = logger or logging.getLogger(f"{__name__}.{type(env).__name__}")

    def get_name(self) -> str:
        return type(self.env).__name__

    def get_tools(self):
        from .dtypes import Tool, ToolFunction, ToolFunctionParameter

        out = []
        for t in getattr(self.env, "oai_tools", None) or []:
            if t.get("type") != "function":
                continue
            f = t["function"]
            params = f.get("parameters") or {}
            out.append(Tool(ToolFunction(f["name"], f.get("description", ""), ToolFunctionParameter(params.get("properties", {}), tuple(params.get("required", []))))))
        return out

    def requires_confirmation(self, tool_call) -> bool:
        return False

    async def _respond(self):
        from ..utils.print_capture import intercept_prints

        with intercept_prints(self.logger):
            new_messages, new_state = await _maybe_await(self.env.env_response(list(self.messages), self.state))
        if isinstance(new_state, dict):
            self.state = new_state
        new_messages = list(new_messages)
        # either the whole conversation comes back (longer than what was sent) or only the reply
        fresh = new_messages[len(self.messages):] if len(new_messages) > len(self.messages) and new_messages[:len(self.messages)] == self.messages else new_messages
        self.messages += fresh
        return fresh

    async def exec_tool(self, tool_call, state: AgentState, run_config: RunConfig):
        import json

        from .dtypes import ToolResult

        self.messages.append({"role": "assistant", "content": None, "tool_calls": [
            {"id": tool_call.id, "type": "function", "function": {"name": tool_call.name, "arguments": json.dumps(tool_call.args)}}]})
        try:
            fresh = await self._respond()
        except Exception as e:  # noqa: BLE001 - the environment's failure is the tool's answer
            return ToolResult(tool_call.id, is_error=True, error=f"{type(e).__name__}: {e}")
        reply = next((m for m in fresh if m.get("role") == "tool"), None)
        if reply is None:
            return ToolResult(tool_call.id, is_error=True, error="the environment gave no tool response")
        done = bool(await _maybe_await(self.env.is_completed(self.messages, self.state))) if hasattr(self.env, "is_completed") else False
        return ToolResult(tool_call.id, content=str(reply.get("content", "")), stop_reason=StopReason.TASK_COMPLETED if done else None,
                          metadata={"env_state_keys": sorted(self.state)})

    async def on_assistant_message(self, message: Message, state: AgentState) -> AgentState:
        if message.get_tool_calls():
            return state                                        # exec_tool will show the call to the environment
        self.messages.append({"role": "assistant", "content": message.text()})
        fresh = await self._respond()
        if hasattr(self.env, "is_completed") and await _maybe_await(self.env.is_completed(self.messages, self.state)):
            return replace(state, environment=self, stop=StopReason.TASK_COMPLETED)
        replies = [Message(m.get("role", "user"), m.get("content", "")) for m in fresh if m.get("role") in ("user", "system")]
        traj = state.actor.trajectory.append(*replies) if replies else state.actor.trajectory
        return replace(state, actor=replace(state.actor, trajectory=traj), environment=self)

    async def serialize(self) -> dict[str, Any]:
        """The live wrapped environment cannot be stored: within a process it is found again through a token; a stored
        session keeps the conversation it had with it (for inspection, not for resumption)."""
        token = f"env-{id(self.env):x}"
        _LIVE_ENVS[token] = (self.env, self.logger)
        plain = {k: v for k, v in self.state.items() if isinstance(v, (int, float, str, bool, list, dict, type(None)))}
        return {"type": "stateful_tool", "token": token, "messages": self.messages, "state": plain, "_state_ref": _keep(self.state)}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "StatefulToolEnvironment":
        env, logger = _LIVE_ENVS.get(data.get("token", ""), (None, None))
        if env is None:
            raise RuntimeError("the wrapped environment of this session is gone (it lives only inside the process that created it)")
        return StatefulToolEnvironment(env, _STATES.get(data.get("_state_ref", ""), data.get("state", {})), data.get("messages", []), logger)


_LIVE_ENVS: dict[str, tuple[Any, Any]] = {}
_STATES: dict[str, dict[str, Any]] = {}


def _keep(state: dict[str, Any]) -> str:
    """Environment state may hold objects (compiled kernels, result records) that JSON cannot carry: the full dict is kept
    in the process and referred to by a key."""
    key = f"state-{id(state):x}-{len(_STATES)}"
    _STATES[key] = dict(state)
    while len(_STATES) > 256:
        _STATES.pop(next(iter(_STATES)))
    return key
