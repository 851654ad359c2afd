"""Reverse-text RL (rollouts/examples/rl/reverse_text/base_config.py:1-176): single turn, "reverse this string", answer
inside ``<reversed_text>`` tags, reward = LCS ratio between the parsed answer and the true reversal. The reference pulls
sentences from a hub dataset; offline the prompts are seeded pseudo-sentences (pass ``texts`` for real ones)."""

from __future__ import annotations

import random
from typing import Any

from examples.common import default_tokenizer, lcs_ratio, parse_tag, response_text, strip_thinking
from examples.rl.base_config import small_config
from research_b200.agents.dtypes import Metric, Score
from research_b200.training.grpo import GRPOConfig, grpo_train

SYSTEM_PROMPT = "Reverse the text character-by-character. Put your answer in <reversed_text> tags."
WORDS = "the of and river stone cloud paper silver engine garden winter signal copper orbit tensor kernel".split()


def make_texts(n: int, seed: int = 0, words: tuple[int, int] = (2, 4)) -> list[str]:
    rng = random.Random(seed)
    return [" ".join(rng.choice(WORDS) for _ in range(rng.randint(*words))) for _ in range(n)]


def make_prompts(texts: list[str]) -> tuple[list[list[dict[str, str]]], list[str]]:
    """Chat prompts and the expected answers."""
    return ([[{"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": t}] for t in texts], [t[::-1] for t in texts])


def reverse_text_score_fn(sample: Any, tokenizer: Any = None) -> Score:
    expected = sample.ground_truth or ""
    raw = response_text(sample, tokenizer)
    parsed = parse_tag(raw, "reversed_text", "final")
    answer = parsed if parsed is not None else strip_thinking(raw)
    return Score((Metric("similarity", lcs_ratio(answer, expected), 1.0), Metric("exact_match", float(answer == expected), 0.0),
                  Metric("has_tags", float(parsed is not None), 0.0)))


DEFAULT = small_config("reverse_text_grpo", temperature=0.7, max_tokens=32)


def train(config: GRPOConfig | None = None, num_samples: int = 64, texts: list[str] | None = None, tokenizer: Any = None,
          device: str | None = None) -> list[dict[str, float]]:
    config = config or DEFAULT
    tokenizer = tokenizer or default_tokenizer()
    prompts, truths = make_prompts(texts or make_texts(num_samples, config.seed))
    return grpo_train(config, prompts, lambda s: reverse_text_score_fn(s, tokenizer), tokenizer=tokenizer, ground_truths=truths, device=device)
