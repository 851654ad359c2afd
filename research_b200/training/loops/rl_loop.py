"""Generic RL loop: rollouts -> advantages -> batch -> backend step -> periodic weight sync
(rollouts/training/loops/rl_loop.py:20-200)."""

from __future__ import annotations

from typing import Any, Callable

import torch

from ..losses import compute_group_advantages
from ..metrics import MetricsLogger
from ..types import RLTrainingConfig, RolloutBatch


def compute_advantages(rewards: list[float], baseline: float = 0.0, group_indices: list[int] | None = None) -> torch.Tensor:
    if group_indices:
        return compute_group_advantages(rewards, group_indices)
    return torch.tensor(rewards, dtype=torch.float32) - baseline


def prepare_grpo_batch(batch: RolloutBatch, advantages: torch.Tensor, max_seq_len: int | None = None,
                       pad_token_id: int = 0) -> dict[str, Any]:
    """Right-padded tensors; ``old_logprobs`` is the masked mean of the rollout log-probs per sequence."""
    n = min(max(len(t) for t in batch.tokens), max_seq_len or 1 << 30)
    B = len(batch.tokens)
    ids = torch.full((B, n), pad_token_id, dtype=torch.long)
    mask = torch.zeros(B, n)
    old = torch.zeros(B)
    for i, (toks, lm) in enumerate(zip(batch.tokens, batch.loss_masks)):
        t = toks[:n]
        ids[i, :len(t)] = torch.tensor(t)
        m = list(lm)[:n]
        mask[i, :len(m)] = torch.tensor(m, dtype=torch.float32)
        if batch.rollout_log_probs is not None:
            lps = batch.rollout_log_probs[i]
            resp = [j for j, v in enumerate(m) if v > 0]
            # rollout log-probs cover the response tokens in order
            vals = lps[:len(resp)]
            old[i] = sum(vals) / max(len(vals), 1)
    out = {"input_ids": ids, "labels": ids.clone(), "loss_mask": mask, "advantages": advantages.float()}
    if batch.rollout_log_probs is not None:
        out["old_logprobs"] = old
    return out


async def run_rl_training(backend, rollout_manager, config: RLTrainingConfig,
                          sync_fn: Callable[[], Any] | None = None, metrics_logger: MetricsLogger | None = None,
                          max_seq_len: int | None = None) -> list[dict[str, float]]:
    history = []
    for step in range(config.num_steps):
        batch = await rollout_manager.generate_batch()
        adv = compute_advantages(batch.rewards, config.baseline, batch.group_indices)
        fb = await backend.forward_backward(prepare_grpo_batch(batch, adv, max_seq_len)).result()
        opt = await backend.optim_step().result()
        m = {**fb, **opt, "mean_reward": sum(batch.rewards) / max(len(batch.rewards), 1)}
        history.append(m)
        if metrics_logger is not None and step % config.log_every == 0:
            metrics_logger.log(m, step)
        if sync_fn is not None and (step + 1) % config.sync_every == 0:
            r = sync_fn()
            if hasattr(r, "__await__"):
                await r
        if config.checkpoint_every and (step + 1) % config.checkpoint_every == 0 and getattr(backend, "checkpoint_dir", None):
            backend.save_checkpoint(step + 1, m)
    return history
