"""Grade-school-math RL (rollouts/examples/rl/gsm8k/base_config.py:1-160): word problems, final answer in ``\\boxed{}``,
reward 1 for the right number plus a small format bonus. ``load_problems`` reads a GSM8K-style JSONL
(``question`` / ``answer`` with ``#### 42``) when given one; offline it writes seeded two-step arithmetic problems in
the same format."""

from __future__ import annotations

import json
import random
import re
from pathlib import Path
from typing import Any

from examples.common import default_tokenizer, response_text
from examples.rl.base_config import small_config
from research_b200.agents.dtypes import Metric, Score
from research_b200.training.grpo import GRPOConfig, grpo_train

SYSTEM_PROMPT = "Solve the problem step by step and give the final number as \\boxed{answer}."
ITEMS = ["apples", "pencils", "marbles", "tickets", "stamps"]


def synthetic_problems(n: int, seed: int = 0) -> list[dict[str, str]]:
    rng = random.Random(seed)
    rows = []
    for _ in range(n):
        a, b, c, item = rng.randint(3, 30), rng.randint(2, 9), rng.randint(1, 20), rng.choice(ITEMS)
        rows.append({"question": f"Tom has {a} boxes with {b} {item} each and gives away {c} {item}. How many {item} are left?",
                     "answer": f"{a} * {b} = {a * b}. {a * b} - {c} = {a * b - c}. #### {a * b - c}"})
    return rows


def load_problems(path: str | Path | None = None, n: int = 64, seed: int = 0) -> list[dict[str, str]]:
    if path and Path(path).exists():
        rows = [json.loads(x) for x in Path(path).read_text().splitlines() if x.strip()]
        return rows[:n]
    return synthetic_problems(n, seed)


def extract_boxed_answer(text: str) -> str | None:
    m = re.findall(r"\\boxed\{([^{}]*)\}", text)
    return m[-1].strip() if m else None


def normalize_answer(answer: str | None) -> float | None:
    if answer is None:
        return None
    cleaned = re.sub(r"[,$%\s]", "", answer)
    m = re.search(r"-?\d+(?:\.\d+)?", cleaned)
    return float(m.group()) if m else None


def truth_of(row: dict[str, str]) -> float | None:
    return normalize_answer(row["answer"].split("####")[-1])


def gsm8k_score_fn(sample: Any, tokenizer: Any = None) -> Score:
    text = response_text(sample, tokenizer)
    boxed = extract_boxed_answer(text)
    got = normalize_answer(boxed) if boxed is not None else normalize_answer((re.findall(r"-?\d[\d,]*(?:\.\d+)?", text) or [None])[-1])
    want = sample.ground_truth
    correct = float(got is not None and want is not None and abs(got - float(want)) < 1e-6)
    return Score((Metric("correct", correct, 1.0), Metric("boxed", float(boxed is not None), 0.1)))


DEFAULT = small_config("gsm8k_grpo", max_tokens=48, max_seq_len=384)


def train(config: GRPOConfig | None = None, num_samples: int = 64, dataset: str | None = None, tokenizer: Any = None, device: str | None = None):
    config = config or DEFAULT
    tokenizer = tokenizer or default_tokenizer()
    rows = load_problems(dataset, num_samples, config.seed)
    prompts = [[{"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": r["question"]}] for r in rows]
    return grpo_train(config, prompts, lambda s: gsm8k_score_fn(s, tokenizer), tokenizer=tokenizer, ground_truths=[truth_of(r) for r in rows], device=device)
