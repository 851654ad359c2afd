"""Trajectory transforms and multi-agent pipelines (rollouts/pipeline.py:39-410).

Pure transforms (compact, summarise, filter, inject), a fan-out runner that executes several agents
on copies of a state with bounded concurrency, reducers that pick one result (best score,
majority vote, model judge) and ``run_agent_pipeline`` that chains stages, feeding each stage's
final trajectory into the next.
"""

from __future__ import annotations

import asyncio
from collections import Counter
from dataclasses import dataclass, field, replace
from typing import Any, Awaitable, Callable

from .agents import run_agent
from .dtypes import Actor, AgentState, Message, RunConfig, Trajectory


# ------------------------------------------------------------------------------ trajectory transforms
def compact_trajectory(trajectory: Trajectory, keep_last_n: int = 5, keep_system: bool = True) -> Trajectory:
    msgs = list(trajectory.messages)
    head = [msgs.pop(0)] if keep_system and msgs and msgs[0].role == "system" else []
    return replace(trajectory, messages=tuple(head + msgs[-keep_last_n:]))


def summarize_trajectory(trajectory: Trajectory, summary: str, keep_last_n: int = 2, keep_system: bool = True) -> Trajectory:
    """Replace everything but the system prompt and the last ``keep_last_n`` messages by one summary message."""
    msgs = list(trajectory.messages)
    head = [msgs.pop(0)] if keep_system and msgs and msgs[0].role == "system" else []
    tail = msgs[-keep_last_n:] if keep_last_n else []
    note = Message("user", f"[Summary of the earlier conversation]\n{summary}")
    return replace(trajectory, messages=tuple(head + [note] + tail))


def filter_trajectory(trajectory: Trajectory, predicate: Callable[[Message], bool]) -> Trajectory:
    return replace(trajectory, messages=tuple(m for m in trajectory.messages if predicate(m)))


def inject_message(trajectory: Trajectory, message: Message, position: int = -1) -> Trajectory:
    msgs = list(trajectory.messages)
    msgs.insert(len(msgs) if position == -1 else position, message)
    return replace(trajectory, messages=tuple(msgs))


# ------------------------------------------------------------------------------ fan-out / reduce
async def run_parallel_agents(states: list[AgentState], run_config: RunConfig | None = None, max_concurrent: int = 4,
                              return_exceptions: bool = True) -> list[list[AgentState] | BaseException]:
    sem = asyncio.Semaphore(max_concurrent)

    async def one(s: AgentState):
        async with sem:
            return await run_agent(s, run_config)

    return await asyncio.gather(*(one(s) for s in states), return_exceptions=return_exceptions)


def _final_text(states: list[AgentState]) -> str:
    for m in reversed(states[-1].actor.trajectory.messages):
        if m.role == "assistant":
            return m.text().strip()
    return ""


def reduce_select_best(results: list[list[AgentState]], score_fn: Callable[[list[AgentState]], float]) -> list[AgentState]:
    assert results, "nothing to select from"
    return max(results, key=score_fn)


def reduce_majority_vote(results: list[list[AgentState]], answer_fn: Callable[[list[AgentState]], str] = _final_text) -> list[AgentState]:
    answers = [answer_fn(r) for r in results]
    winner, _ = Counter(answers).most_common(1)[0]
    return results[answers.index(winner)]


async def reduce_llm_judge(results: list[list[AgentState]], judge: Callable[[Actor, RunConfig], Awaitable[Actor]], endpoint,
                           question: str = "Which candidate answer is best?") -> list[AgentState]:
    """Ask a model to pick; ``judge`` is any rollout function (a provider or a scripted stand-in)."""
    listing = "\n\n".join(f"Candidate {i + 1}:\n{_final_text(r)}" for i, r in enumerate(results))
    prompt = f"{question}\n\n{listing}\n\nReply with the number of the best candidate only."
    actor = await judge(Actor(Trajectory((Message("user", prompt),)), endpoint), RunConfig())
    digits = "".join(ch for ch in actor.trajectory.messages[-1].text() if ch.isdigit())
    idx = int(digits) - 1 if digits else 0
    return results[idx if 0 <= idx < len(results) else 0]


# ------------------------------------------------------------------------------ staged pipeline
@dataclass
class AgentStage:
    name: str
    endpoint: Any
    environment_factory: Callable[[], Any] | None = None
    system_prompt: str | None = None
    max_turns: int = 10
    n_parallel: int = 1
    reducer: Callable[[list[list[AgentState]]], list[AgentState]] = reduce_majority_vote
    transform: Callable[[Trajectory], Trajectory] | None = None     # applied to the incoming trajectory
    run_config: RunConfig = field(default_factory=RunConfig)


async def run_agent_pipeline(stages: list[AgentStage], initial: Trajectory) -> tuple[Trajectory, dict[str, list[AgentState]]]:
    """Run stages in order; returns the final trajectory and every stage's chosen state list."""
    traj, chosen = initial, {}
    for st in stages:
        if st.transform is not None:
            traj = st.transform(traj)
        msgs = [m for m in traj.messages if m.role != "system"] if st.system_prompt else list(traj.messages)
        if st.system_prompt:
            msgs = [Message("system", st.system_prompt)] + msgs
        base = Trajectory(tuple(msgs), traj.completions, traj.rewards, dict(traj.metadata))
        states = [AgentState(Actor(base, st.endpoint), st.environment_factory() if st.environment_factory else None,
                             max_turns=st.max_turns) for _ in range(st.n_parallel)]
        results = [r for r in await run_parallel_agents(states, st.run_config, st.n_parallel) if not isinstance(r, BaseException)]
        if not results:
            raise RuntimeError(f"stage {st.name!r}: every agent failed")
        best = results[0] if len(results) == 1 else st.reducer(results)
        chosen[st.name] = best
        traj = best[-1].actor.trajectory
    return traj, chosen
