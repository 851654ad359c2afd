from .async_rollout_manager import AsyncRolloutManager, generate_rollout_batch
from .rollout_generation import (apply_sample_transforms, build_batch_metadata, compute_response_lengths,
                                 convert_to_batch, extract_group_indices, extract_rollout_log_probs,
                                 extract_sample_fields, generate_rollout_batches)
from .rollout_manager import RolloutManager

__all__ = ["AsyncRolloutManager", "generate_rollout_batch", "apply_sample_transforms", "build_batch_metadata",
           "compute_response_lengths", "convert_to_batch", "extract_group_indices", "extract_rollout_log_probs",
           "extract_sample_fields", "generate_rollout_batches", "RolloutManager"]
