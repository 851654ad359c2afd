"""Training: types, losses, filters, backends, loops, rollout generation, GRPO driver.

Names are resolved lazily so that ``import research_b200.training`` stays cheap
(the reference does the same, rollouts/training/__init__.py:26-136)."""

from __future__ import annotations

import importlib

_LAZY = {
    "Sample": ".types", "RolloutBatch": ".types", "RolloutConfig": ".types", "TrainerConfig": ".types",
    "SFTTrainingConfig": ".types", "RLTrainingConfig": ".types", "TrainFuture": ".types",
    "ImmediateTrainFuture": ".types", "Status": ".types",
    "GRPOConfig": ".grpo", "grpo_train": ".grpo",
    "run_rl_training": ".loops.rl_loop", "run_sft_training": ".loops.sft_loop",
    "AsyncRolloutManager": ".rollout_gen.async_rollout_manager", "RolloutManager": ".rollout_gen.rollout_manager",
    "DataBuffer": ".datasets.data_buffer", "BufferState": ".datasets.data_buffer",
    "TrainingBackend": ".backends.protocol", "PyTorchTrainingBackend": ".backends.pytorch",
    "FSDPTrainingBackend": ".backends.fsdp", "FSDPConfig": ".backends.fsdp",
    "create_pytorch_backend": ".backends.pytorch_factory",
    "grpo_loss": ".losses", "grpo_loss_clipped": ".losses", "grpo_loss_masked": ".losses", "sft_loss": ".losses",
    "pretrain_loss": ".losses", "ppo_loss": ".losses", "compute_group_advantages": ".losses",
    "JSONLLogger": ".metrics", "WandbLogger": ".metrics", "CompositeLogger": ".metrics", "MetricsLogger": ".metrics",
    "sync_weights_to_engines": ".weight_sync", "NativeEngine": ".weight_sync", "SGLangEngine": ".weight_sync",
    "VLLMEngine": ".weight_sync",
}


def __getattr__(name: str):
    if name in _LAZY:
        return getattr(importlib.import_module(_LAZY[name], __name__), name)
    raise AttributeError(name)


__all__ = sorted(_LAZY)
