"""Dry run of the evaluation pipeline with a scripted model that solves the synthetic problems by reading the numbers
(python examples/eval/gsm8k/eval_scripted_01_01.py). Replace the endpoint to evaluate a real model:
``Endpoint(provider="native", engine=engine)`` or ``Endpoint(provider="openai", model=..., api_key=...)``."""

import re
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from examples.eval.gsm8k.base_config import GSM8KConfig, run_eval  # noqa: E402
from research_b200.agents.dtypes import Endpoint  # noqa: E402
from research_b200.agents.providers import ScriptedLLM, register_provider  # noqa: E402


async def reads_the_numbers(actor, run_config):
    question = next(m.text() for m in actor.trajectory.messages if m.role == "user")
    a, b, c = (int(x) for x in re.findall(r"\d+", question)[:3])
    return await ScriptedLLM([f"{a} * {b} = {a * b}, minus {c}: \\boxed{{{a * b - c}}}"])(actor, run_config)


if __name__ == "__main__":
    register_provider("mock", reads_the_numbers)
    report = run_eval(GSM8KConfig(endpoint=Endpoint(provider="mock"), num_samples=10, output_dir="results/eval/gsm8k_scripted"))
    print(report.summary)
    assert report.summary["mean_reward"] == 1.0
