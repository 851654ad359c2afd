"""Dataset evaluation: run an agent per sample with bounded concurrency and sample-level retry,
score the trajectory, write a report (rollouts/evaluation.py:130-994)."""

from __future__ import annotations

import asyncio
import json
import statistics
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterable

from .agents import run_agent
from .dtypes import Actor, AgentState, EvalConfig, Message, Score, Trajectory
from .providers.base import NonRetryableError, ProviderError


@dataclass
class EvalSample:
    sample_id: str
    input: dict[str, Any]
    trajectory: Trajectory
    score: Score
    stop_reason: str | None = None
    error: str | None = None
    attempts: int = 1
    duration_s: float = 0.0
    metadata: dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return {"sample_id": self.sample_id, "input": self.input, "trajectory": self.trajectory.to_dict(),
                "score": self.score.to_dict(), "stop_reason": self.stop_reason, "error": self.error,
                "attempts": self.attempts, "duration_s": self.duration_s, "metadata": self.metadata}


@dataclass
class EvalReport:
    eval_name: str
    samples: list[EvalSample]
    summary: dict[str, float]
    config: dict[str, Any] = field(default_factory=dict)
    timestamp: float = field(default_factory=time.time)

    def save(self, output_dir: str | Path) -> Path:
        d = Path(output_dir) / self.eval_name
        d.mkdir(parents=True, exist_ok=True)
        (d / "report.json").write_text(json.dumps({"eval_name": self.eval_name, "summary": self.summary,
                                                   "config": self.config, "timestamp": self.timestamp,
                                                   "num_samples": len(self.samples)}, indent=2, default=str))
        with open(d / "samples.jsonl", "w") as f:
            for s in self.samples:
                f.write(json.dumps(s.to_dict(), default=str) + "\n")
        Trajectory.save_jsonl([s.trajectory for s in self.samples], d / "trajectories.jsonl")
        return d


def compute_summary_metrics(samples: list[EvalSample]) -> dict[str, float]:
    if not samples:
        return {"num_samples": 0.0}
    rewards = [s.score.reward for s in samples]
    out = {"num_samples": float(len(samples)), "mean_reward": statistics.fmean(rewards),
           "error_rate": sum(1 for s in samples if s.error) / len(samples),
           "mean_duration_s": statistics.fmean(s.duration_s for s in samples)}
    if len(rewards) > 1:
        out["std_reward"] = statistics.stdev(rewards)
    names = {m.name for s in samples for m in s.score.metrics}
    for n in sorted(names):
        vals = [m.value for s in samples for m in s.score.metrics if m.name == n]
        out[f"mean_{n}"] = statistics.fmean(vals)
    return out


async def evaluate_sample(row: dict[str, Any], sample_id: str, config: EvalConfig) -> EvalSample:
    """One agent run + scoring, retried on transient provider errors."""
    t0 = time.time()
    last_err: str | None = None
    for attempt in range(config.n_retries + 1):
        try:
            msgs = config.prepare_messages(row) if config.prepare_messages else [Message("user", str(row.get("prompt", row.get("question", ""))))]
            env = config.environment_factory(row) if config.environment_factory else None
            if asyncio.iscoroutine(env):
                env = await env
            state = AgentState(Actor(Trajectory(tuple(msgs)), config.endpoint), env, max_turns=config.max_turns)
            states = await run_agent(state, config.run_config)
            final = states[-1]
            score = config.score_fn(final.actor.trajectory, row)
            if asyncio.iscoroutine(score):
                score = await score
            if not isinstance(score, Score):
                from .dtypes import Metric

                score = Score((Metric("reward", float(score), 1.0),))
            return EvalSample(sample_id, row, final.actor.trajectory, score, final.stop.value if final.stop else None,
                              None, attempt + 1, time.time() - t0)
        except NonRetryableError as e:
            last_err = f"{type(e).__name__}: {e}"
            break
        except (ProviderError, asyncio.TimeoutError, ConnectionError) as e:
            last_err = f"{type(e).__name__}: {e}"
            if attempt < config.n_retries:
                await asyncio.sleep(config.retry_delays[min(attempt, len(config.retry_delays) - 1)])
    return EvalSample(sample_id, row, Trajectory(), Score(), None, last_err, config.n_retries + 1, time.time() - t0)


async def evaluate(dataset: Iterable[dict[str, Any]], config: EvalConfig) -> EvalReport:
    rows = list(dataset)
    if config.max_samples is not None:
        rows = rows[:config.max_samples]
    sem = asyncio.Semaphore(config.max_concurrent)

    async def one(i: int, row: dict[str, Any]) -> EvalSample:
        async with sem:
            return await evaluate_sample(row, str(row.get("id", i)), config)

    samples = list(await asyncio.gather(*[one(i, r) for i, r in enumerate(rows)]))
    report = EvalReport(config.eval_name, samples, compute_summary_metrics(samples),
                        {"endpoint": config.endpoint.to_dict(), "max_turns": config.max_turns})
    if config.output_dir:
        report.save(config.output_dir)
    return report


def group_by(samples: list[EvalSample], key: Callable[[EvalSample], Any]) -> dict[Any, list[EvalSample]]:
    out: dict[Any, list[EvalSample]] = {}
    for s in samples:
        out.setdefault(key(s), []).append(s)
    return out


def summarize(groups: dict[Any, list[EvalSample]]) -> dict[Any, dict[str, float]]:
    return {k: compute_summary_metrics(v) for k, v in groups.items()}


_ = asdict
