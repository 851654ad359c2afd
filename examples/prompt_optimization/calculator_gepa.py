"""Prompt optimisation with GEPA on an arithmetic task (rollouts/examples/prompt_optimization/calculator_gepa.py): the
candidate is a system prompt; a reflection model reads scored traces and proposes a better instruction. Here both the
task model and the reflection model are scripted so the loop runs offline; plug in real ``generate`` / ``reflect``
coroutines (any provider) to optimise an actual prompt."""

import asyncio
import random
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from research_b200.agents.prompt_optimization import GEPAConfig, optimize_prompt  # noqa: E402


def make_set(n: int, seed: int) -> list[dict]:
    rng = random.Random(seed)
    rows = []
    for _ in range(n):
        a, b = rng.randint(2, 30), rng.randint(2, 30)
        rows.append({"input": f"{a} + {b}", "answer": str(a + b)})
    return rows


async def generate(system: str, user: str) -> str:
    """A stand-in task model: it only answers with the bare number when the instruction asks for that."""
    a, b = (int(x) for x in user.split("+"))
    return str(a + b) if "only the number" in system.lower() else f"The sum of {a} and {b} is {a + b}, I think."


def score(sample: dict, text: str) -> tuple[float, str]:
    ok = text.strip() == sample["answer"]
    return float(ok), "exact" if ok else f"expected the bare number {sample['answer']}, got {text!r}"


async def reflect(prompt: str) -> str:
    """A stand-in reflection model: reads the feedback in the prompt and proposes the obvious fix."""
    return "```\nAdd the two numbers. Reply with only the number, nothing else.\n```" if "bare number" in prompt else "```\nAdd the numbers.\n```"


def run(max_evaluations: int = 80):
    return asyncio.run(optimize_prompt("You are a helpful calculator.", "{input}", generate, score, make_set(12, 0), make_set(8, 1), reflect,
                                       GEPAConfig(max_evaluations=max_evaluations, minibatch_size=4, seed=0)))


if __name__ == "__main__":
    result = run()
    print(f"best validation score {result.best_score:.2f} with system prompt: {result.best_candidate['system']!r}")
