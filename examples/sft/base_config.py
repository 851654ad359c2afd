"""Supervised fine-tuning examples (rollouts/examples/sft/base_config.py:1-367): build chat samples, mask the loss to the
assistant turns, run ``run_sft_training`` over a single-GPU (or CPU) backend, checkpoint."""

from __future__ import annotations

import asyncio
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from examples.common import default_tokenizer
from research_b200.training.backends import create_backend_with_scheduler
from research_b200.training.datasets.sft import load_sft_dataset
from research_b200.training.loops.sft_loop import run_sft_training
from research_b200.training.metrics import JSONLLogger
from research_b200.training.types import SFTTrainingConfig, TrainerConfig


@dataclass(frozen=True)
class SFTExampleConfig:
    experiment_name: str = "sft"
    model_name: str = "tiny-qwen2"
    lr: float = 1e-3
    warmup_steps: int = 2
    num_steps: int = 20
    batch_size: int = 8
    micro_batch_size: int | None = None
    max_length: int = 256
    output_dir: str = "results/sft"
    checkpoint_every: int = 0
    seed: int = 0
    extra: dict[str, Any] = field(default_factory=dict)


def train(config: SFTExampleConfig, rows: list[dict[str, Any]], tokenizer: Any = None, device: str | None = None):
    """``rows``: chat rows (``messages`` / ``conversations`` / ``prompt`` + ``response``). Returns (history, backend)."""
    tokenizer = tokenizer or default_tokenizer()
    samples = load_sft_dataset(rows, tokenizer, max_length=config.max_length)
    assert samples, "no usable rows"
    out = Path(config.output_dir) / config.experiment_name
    backend = create_backend_with_scheduler(config.model_name, total_steps=config.num_steps, warmup_steps=config.warmup_steps,
                                            device=device, loss_fn="sft", lr=config.lr, seed=config.seed,
                                            checkpoint_dir=out / "checkpoints",
                                            trainer_config=TrainerConfig(micro_batch_size=config.micro_batch_size))
    loop = SFTTrainingConfig(num_steps=config.num_steps, batch_size=config.batch_size, log_every=1, checkpoint_every=config.checkpoint_every)
    hist = asyncio.run(run_sft_training(backend, samples, loop, JSONLLogger(out), pad_token_id=getattr(tokenizer, "pad_token_id", 0) or 0))
    return hist, backend
