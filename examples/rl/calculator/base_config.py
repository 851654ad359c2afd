"""Multi-turn tool-use RL (rollouts/examples/rl/calculator/base_config.py:1-132): the policy drives
``CalculatorEnvironment`` through tool calls over several turns; every turn is generated token-in / token-out by the
in-process engine and the reward compares the calculator's final value (or the stated answer) with the truth."""

from __future__ import annotations

import random
import re
from typing import Any

from examples.common import default_tokenizer
from examples.rl.base_config import small_config
from research_b200.agents.dtypes import Metric, Score
from research_b200.agents.environments import CalculatorEnvironment
from research_b200.training.grpo import GRPOConfig, grpo_train

SYSTEM_PROMPT = ("You are a calculator assistant. Use one tool call per turn, in the form "
                 '<tool_call>{"name": "add", "arguments": {"value": 3}}</tool_call>, and finish with complete_task.')


def make_problems(n: int, seed: int = 0) -> tuple[list[list[dict[str, str]]], list[float]]:
    rng = random.Random(seed)
    prompts, truths = [], []
    for _ in range(n):
        a, b, c = rng.randint(1, 20), rng.randint(1, 20), rng.randint(2, 5)
        prompts.append([{"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": f"Compute ({a} + {b}) * {c}."}])
        truths.append(float((a + b) * c))
    return prompts, truths


def calculator_score_fn(sample: Any) -> Score:
    want = float(sample.ground_truth or 0.0)
    text = str((sample.metadata or {}).get("response_text", "")) + " " + " ".join(str(m) for m in (sample.metadata or {}).get("messages", []))
    numbers = [float(x) for x in re.findall(r"-?\d+(?:\.\d+)?", text)]
    hit = float(any(abs(x - want) < 1e-6 for x in numbers[-4:]))
    used_tool = float("tool_call" in text or (sample.metadata or {}).get("stop_reason") == "task_completed")
    return Score((Metric("correct", hit, 1.0), Metric("used_tool", used_tool, 0.1)))


# the tool schemas are part of the prompt: about 1.6 k characters with the character tokenizer
DEFAULT = small_config("calculator_grpo", max_turns=3, use_tito=False, max_tokens=32, max_seq_len=2048, kv_blocks=2048, batch_size=2)


def train(config: GRPOConfig | None = None, num_samples: int = 32, tokenizer: Any = None, device: str | None = None):
    config = config or DEFAULT
    prompts, truths = make_problems(num_samples, config.seed)
    return grpo_train(config, prompts, calculator_score_fn, environment_cls=CalculatorEnvironment, tokenizer=tokenizer or default_tokenizer(),
                      ground_truths=truths, device=device)
