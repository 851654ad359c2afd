"""Alphabet-sort RL (rollouts/examples/rl/alphabet_sort/base_config.py:1-248): sort a list of names alphabetically,
one per line inside ``<sorted>`` tags; reward = fraction of positions that are right, with a bonus for an exact list."""

from __future__ import annotations

import random
from typing import Any

from examples.common import default_tokenizer, parse_tag, response_text, strip_thinking
from examples.rl.base_config import small_config
from research_b200.agents.dtypes import Metric, Score
from research_b200.training.grpo import GRPOConfig, grpo_train

SYSTEM_PROMPT = "Sort the names alphabetically. Answer with one name per line inside <sorted> tags."
NAMES = "ada bo cy dee eli fay gus hal ivy jo kit lee mae ned oz pia quin rae sy tess".split()


def make_tasks(n: int, seed: int = 0, k: tuple[int, int] = (3, 5)) -> tuple[list[list[dict[str, str]]], list[list[str]]]:
    rng = random.Random(seed)
    lists = [rng.sample(NAMES, rng.randint(*k)) for _ in range(n)]
    prompts = [[{"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": ", ".join(x)}] for x in lists]
    return prompts, [sorted(x) for x in lists]


def sort_score_fn(sample: Any, tokenizer: Any = None) -> Score:
    want: list[str] = list(sample.ground_truth or [])
    raw = response_text(sample, tokenizer)
    parsed = parse_tag(raw, "sorted")
    got = [x.strip() for x in (parsed if parsed is not None else strip_thinking(raw)).replace(",", "\n").split("\n") if x.strip()]
    right = sum(a == b for a, b in zip(got, want)) / max(len(want), 1)
    exact = float(got == want)
    return Score((Metric("position_accuracy", right, 0.8), Metric("exact", exact, 0.2), Metric("has_tags", float(parsed is not None), 0.0)))


DEFAULT = small_config("alphabet_sort_grpo", max_tokens=32)


def train(config: GRPOConfig | None = None, num_samples: int = 64, tokenizer: Any = None, device: str | None = None):
    config = config or DEFAULT
    tokenizer = tokenizer or default_tokenizer()
    prompts, truths = make_tasks(num_samples, config.seed)
    return grpo_train(config, prompts, lambda s: sort_score_fn(s, tokenizer), tokenizer=tokenizer, ground_truths=truths, device=device)
