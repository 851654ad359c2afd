from .rl_loop import compute_advantages, prepare_grpo_batch, run_rl_training
from .sft_loop import collate_batch, prepare_sft_batch, run_sft_training

__all__ = ["compute_advantages", "prepare_grpo_batch", "run_rl_training", "collate_batch", "prepare_sft_batch",
           "run_sft_training"]
