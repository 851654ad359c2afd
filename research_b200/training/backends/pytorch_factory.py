"""Three-tier construction helpers (rollouts/training/backends/pytorch_factory.py:55-499).

Tier 1: primitives (``parse_dtype``, ``load_model_weights``, optimizer/loss/scheduler choices).
Tier 2: ``create_pytorch_backend`` one call.
Tier 3: ``create_backend_with_scheduler`` adds warm-up + cosine decay.
"""

from __future__ import annotations

from pathlib import Path
from typing import Callable

import torch

from ...models.config import ModelConfig, get_preset
from ...models.weights import init_random_weights, load_safetensors_dir
from ..losses import LOGPROB_LOSSES
from ..types import TrainerConfig
from .native import warmup_cosine
from .pytorch import PyTorchTrainingBackend


def parse_dtype(name: str | torch.dtype) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    table = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
             "half": torch.float16, "fp32": torch.float32, "float32": torch.float32, "float": torch.float32}
    key = name.lower().replace("torch.", "")
    assert key in table, f"unknown dtype {name!r}; expected one of {sorted(table)}"
    return table[key]


def load_model_weights(model_name: str, seed: int = 0, device=None) -> tuple[dict[str, torch.Tensor], ModelConfig]:
    """A checkpoint directory (HF safetensors) or the name of a built-in preset (random init). Presets above 12 B
    parameters come back as a lazy mapping that builds one tensor at a time (on ``device`` when given), so that no
    process ever holds a second full copy of such a model."""
    if Path(model_name).is_dir():
        return load_safetensors_dir(model_name)
    cfg = get_preset(model_name)
    if cfg.num_params() > 12e9:
        from ...models.weights import LazyRandomWeights

        return LazyRandomWeights(cfg, seed=seed, device=device or "cpu"), cfg
    return init_random_weights(cfg, seed=seed), cfg


def create_adamw_optimizer(lr: float = 1e-5, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0) -> dict:
    """Hyper-parameters of the fused sharded AdamW (betas default to the reference's (0.9, 0.95))."""
    return {"lr": lr, "betas": tuple(betas), "eps": eps, "weight_decay": weight_decay}


def create_cross_entropy_loss() -> str:
    return "ce"


def create_loss(name: str) -> str:
    assert name in LOGPROB_LOSSES, f"unknown loss {name!r}; expected one of {sorted(LOGPROB_LOSSES)}"
    return name


def create_warmup_cosine_scheduler(warmup_steps: int, total_steps: int, min_lr_ratio: float = 0.1) -> Callable[[int], float]:
    return warmup_cosine(warmup_steps, total_steps, min_lr_ratio)


def create_pytorch_backend(model_name: str, checkpoint_dir: str | Path | None = None, device: str | None = None,
                           dtype: str = "bfloat16", loss_fn: str = "grpo", lr: float = 1e-5, weight_decay: float = 0.0,
                           trainer_config: TrainerConfig | None = None, seed: int = 0, **kw) -> PyTorchTrainingBackend:
    parse_dtype(dtype)
    weights, cfg = load_model_weights(model_name, seed)
    return PyTorchTrainingBackend(cfg, weights, device=device, loss_fn=create_loss(loss_fn),
                                  checkpoint_dir=checkpoint_dir, trainer_config=trainer_config,
                                  **create_adamw_optimizer(lr=lr, weight_decay=weight_decay), **kw)


def create_backend_with_scheduler(model_name: str, total_steps: int, warmup_steps: int = 0, min_lr_ratio: float = 0.1,
                                  **kw) -> PyTorchTrainingBackend:
    return create_pytorch_backend(model_name, lr_schedule=create_warmup_cosine_scheduler(warmup_steps, total_steps, min_lr_ratio), **kw)
