"""Supervised fine-tuning loop over any ``TrainingBackend`` (rollouts/training/loops/sft_loop.py:19-199)."""

from __future__ import annotations

from typing import Any

import torch

from ..metrics import MetricsLogger
from ..types import Sample, SFTTrainingConfig


def collate_batch(samples: list[Sample], pad_token_id: int = 0, max_len: int | None = None) -> dict[str, Any]:
    """Right-pad to the longest sample: ``input_ids``, ``labels``, ``loss_mask``, ``attention_mask``."""
    n = min(max(len(s.tokens) for s in samples), max_len or 1 << 30)
    ids = torch.full((len(samples), n), pad_token_id, dtype=torch.long)
    mask = torch.zeros(len(samples), n)
    attn = torch.zeros(len(samples), n, dtype=torch.long)
    for i, s in enumerate(samples):
        t = s.tokens[:n]
        ids[i, :len(t)] = torch.tensor(t)
        lm = (s.loss_mask or [1.0] * len(s.tokens))[:n]
        mask[i, :len(lm)] = torch.tensor(lm, dtype=torch.float32)
        attn[i, :len(t)] = 1
    return {"input_ids": ids, "labels": ids.clone(), "loss_mask": mask, "attention_mask": attn}


def prepare_sft_batch(samples: list[Sample]) -> dict[str, Any]:
    """Sequence packing: one row ``[1, total]`` plus ``cu_seqlens`` and per-token ``position_ids``."""
    toks, mask, pos, cu = [], [], [], [0]
    for s in samples:
        toks.extend(s.tokens)
        lm = list(s.loss_mask or [1.0] * len(s.tokens))
        lm[0] = 0.0  # the first token of a document has no in-document context to be predicted from
        mask.extend(lm)
        pos.extend(range(len(s.tokens)))
        cu.append(len(toks))
    ids = torch.tensor([toks], dtype=torch.long)
    return {"input_ids": ids, "labels": ids.clone(), "loss_mask": torch.tensor([mask]),
            "cu_seqlens": torch.tensor(cu, dtype=torch.int32), "position_ids": torch.tensor([pos], dtype=torch.long)}


async def run_sft_training(backend, samples: list[Sample], config: SFTTrainingConfig,
                           metrics_logger: MetricsLogger | None = None, pad_token_id: int = 0) -> list[dict[str, float]]:
    """``num_steps`` optimizer steps over ``samples`` (cycled); returns the per-step metrics."""
    assert samples, "no training samples"
    history: list[dict[str, float]] = []
    for step in range(config.num_steps):
        lo = (step * config.batch_size) % len(samples)
        picked = [samples[(lo + i) % len(samples)] for i in range(config.batch_size)]
        batch = collate_batch(picked, pad_token_id)
        fb = await backend.forward_backward(batch).result()
        opt = await backend.optim_step().result()
        m = {**fb, **opt}
        history.append(m)
        if metrics_logger is not None and step % config.log_every == 0:
            metrics_logger.log(m, step)
        if config.checkpoint_every and (step + 1) % config.checkpoint_every == 0 and getattr(backend, "checkpoint_dir", None):
            backend.save_checkpoint(step + 1, m)
    return history
