"""Synchronous rollout batches and the Sample -> RolloutBatch conversion
(rollouts/training/rollout_gen/rollout_generation.py:21-260)."""

from __future__ import annotations

from typing import Any, Iterator

from ..datasets.data_buffer import DataBuffer
from ..types import RolloutBatch, RolloutConfig, Sample


def extract_sample_fields(samples: list[Sample]) -> tuple[list, list, list]:
    return [s.tokens for s in samples], [s.loss_mask for s in samples], [s.reward for s in samples]


def extract_group_indices(samples: list[Sample]) -> list[int]:
    return [s.group_index if s.group_index is not None else i for i, s in enumerate(samples)]


def extract_rollout_log_probs(samples: list[Sample]) -> list[list[float]] | None:
    if not samples or any(s.rollout_log_probs is None for s in samples):
        return None
    return [list(s.rollout_log_probs) for s in samples]  # type: ignore[arg-type]


def compute_response_lengths(loss_masks: list[list[float]]) -> list[int]:
    return [int(sum(1 for m in mask if m > 0)) for mask in loss_masks]


def build_batch_metadata(samples: list[Sample], **extra: Any) -> dict[str, Any]:
    n = max(len(samples), 1)
    return {"num_samples": len(samples), "mean_reward": sum(s.reward for s in samples) / n,
            "mean_tokens": sum(len(s.tokens) for s in samples) / n, **extra}


def convert_to_batch(samples: list[Sample], **metadata: Any) -> RolloutBatch:
    tokens, masks, rewards = extract_sample_fields(samples)
    return RolloutBatch(tokens=tokens, loss_masks=masks, rewards=rewards, response_lengths=compute_response_lengths(masks),
                        group_indices=extract_group_indices(samples), rollout_log_probs=extract_rollout_log_probs(samples),
                        samples=list(samples), metadata=build_batch_metadata(samples, **metadata))


def apply_sample_transforms(samples: list[Sample], config: RolloutConfig) -> list[Sample]:
    """Score every sample (``score.reward`` -> ``sample.reward``) then keep groups that pass the filter."""
    if config.score_fn is not None:
        for s in samples:
            score = config.score_fn(s)
            s.score = score
            s.reward = float(getattr(score, "reward", score))
    if config.filter_fn is None:
        return samples
    groups: dict[int, list[Sample]] = {}
    for i, s in enumerate(samples):
        groups.setdefault(s.group_index if s.group_index is not None else i, []).append(s)
    return [s for g in groups.values() if config.filter_fn(g) for s in g]


def generate_rollout_batches(data_buffer: DataBuffer, config: RolloutConfig, **kwargs: Any) -> Iterator[RolloutBatch]:
    """Endless generator of scored, filtered rollout batches."""
    assert config.generate_fn is not None, "RolloutConfig.generate_fn is required"
    step = 0
    while True:
        groups = data_buffer.get_sample_groups(config.batch_size, config.n_samples_per_prompt)
        prompts = [g[0].prompt for g in groups for _ in g]
        flat = [s for g in groups for s in g]
        out = config.generate_fn(prompts, **kwargs)
        for src, dst in zip(flat, out):
            dst.group_index, dst.index = src.group_index, src.index
            if dst.ground_truth is None:
                dst.ground_truth = src.ground_truth
        samples = apply_sample_transforms(list(out), config)
        yield convert_to_batch(samples, step=step)
        step += 1
