"""Evaluation on GSM8K-style problems (rollouts/examples/eval/gsm8k/base_config.py:35-700): single-turn (answer in
``\\boxed{}``) or multi-turn with the calculator tools, against any endpoint: the in-process engine (``provider="native"``),
an HTTP server, a hosted API, or a scripted model for dry runs."""

from __future__ import annotations

import asyncio
from dataclasses import dataclass
from typing import Any

from examples.rl.gsm8k.base_config import SYSTEM_PROMPT, extract_boxed_answer, load_problems, normalize_answer, truth_of
from research_b200.agents.dtypes import Endpoint, EvalConfig, Message, Metric, Score, Trajectory
from research_b200.agents.environments import CalculatorEnvironment
from research_b200.agents.evaluation import EvalReport, evaluate


@dataclass(frozen=True)
class GSM8KConfig:
    endpoint: Endpoint = Endpoint(provider="mock")
    dataset: str | None = None
    num_samples: int = 20
    seed: int = 0
    use_tools: bool = False
    max_turns: int = 6
    max_concurrent: int = 4
    output_dir: str | None = None
    eval_name: str = "gsm8k"


def score_trajectory(traj: Trajectory, row: dict[str, Any]) -> Score:
    answers = [m.text() for m in traj.messages if m.role == "assistant"]
    text = answers[-1] if answers else ""
    boxed = extract_boxed_answer(text)
    got = normalize_answer(boxed if boxed is not None else text)
    if got is None:                                     # tool runs: the last tool result is the calculator's value
        tools = [m.text() for m in traj.messages if m.role == "tool"]
        got = normalize_answer(tools[-1]) if tools else None
    want = truth_of(row)
    correct = float(got is not None and want is not None and abs(got - want) < 1e-6)
    return Score((Metric("correct", correct, 1.0), Metric("boxed", float(boxed is not None), 0.0),
                  Metric("turns", float(len(answers)), 0.0)))


def run_eval(config: GSM8KConfig) -> EvalReport:
    rows = load_problems(config.dataset, config.num_samples, config.seed)
    system = SYSTEM_PROMPT if not config.use_tools else SYSTEM_PROMPT + " Use the calculator tools for every arithmetic step."
    ec = EvalConfig(endpoint=config.endpoint, score_fn=score_trajectory,
                    environment_factory=(lambda row: CalculatorEnvironment()) if config.use_tools else None,
                    prepare_messages=lambda row: [Message("system", system), Message("user", row["question"])],
                    max_turns=config.max_turns if config.use_tools else 1, max_concurrent=config.max_concurrent,
                    output_dir=config.output_dir, eval_name=config.eval_name, n_retries=0)
    return asyncio.run(evaluate(rows, ec))
