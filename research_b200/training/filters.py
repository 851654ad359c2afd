"""Dynamic-sampling filters over one GRPO group (all samples of one prompt).

A filter returns True to keep the group. Same catalogue as the reference
(rollouts/training/filters.py:21-271): reward spread, minimum reward, response diversity,
length sanity, any-success, the combined quality+diversity check, and two factories.
"""

from __future__ import annotations

import statistics
from typing import Callable

from .types import Sample


def check_reward_nonzero_std(samples: list[Sample]) -> bool:
    """Groups whose rewards are all equal carry no GRPO signal (every advantage is zero)."""
    if len(samples) < 2:
        return True
    return statistics.pstdev(s.reward for s in samples) > 1e-6


def check_min_reward(samples: list[Sample], threshold: float = 0.5) -> bool:
    return bool(samples) and max(s.reward for s in samples) >= threshold


def _response_key(s: Sample):
    if s.response_length:
        return tuple(s.tokens[-s.response_length:])
    return s.response or tuple(s.tokens)


def check_response_diversity(samples: list[Sample], min_unique_ratio: float = 0.5) -> bool:
    if not samples:
        return False
    return len({_response_key(s) for s in samples}) / len(samples) >= min_unique_ratio


def check_reasonable_length(samples: list[Sample], min_tokens: int = 1, max_tokens: int = 8192) -> bool:
    for s in samples:
        n = s.response_length or len(s.tokens)
        if n < min_tokens or n > max_tokens:
            return False
    return bool(samples)


def check_any_success(samples: list[Sample]) -> bool:
    return any(s.reward > 0 for s in samples)


def check_quality_and_diversity(samples: list[Sample]) -> bool:
    return check_reward_nonzero_std(samples) and check_response_diversity(samples) and check_reasonable_length(samples)


def make_threshold_filter(threshold: float) -> Callable[[list[Sample]], bool]:
    def filter_fn(samples: list[Sample]) -> bool:
        return check_min_reward(samples, threshold)

    return filter_fn


def make_length_filter(min_tokens: int, max_tokens: int) -> Callable[[list[Sample]], bool]:
    def filter_fn(samples: list[Sample]) -> bool:
        return check_reasonable_length(samples, min_tokens, max_tokens)

    return filter_fn
