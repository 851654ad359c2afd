"""Synchronous manager kept for older call sites (rollouts/training/rollout_gen/rollout_manager.py:49)."""

from __future__ import annotations

import warnings
from dataclasses import dataclass

from ..datasets.data_buffer import DataBuffer
from ..types import RolloutBatch, RolloutConfig
from .rollout_generation import generate_rollout_batches


@dataclass
class RolloutManager:
    data_buffer: DataBuffer
    config: RolloutConfig

    def __post_init__(self) -> None:
        warnings.warn("RolloutManager is superseded by AsyncRolloutManager", DeprecationWarning, stacklevel=2)
        self._it = generate_rollout_batches(self.data_buffer, self.config)

    def __iter__(self):
        return self

    def __next__(self) -> RolloutBatch:
        return next(self._it)

    def state_dict(self) -> dict:
        return {"buffer_state": self.data_buffer.save_state()}

    def load_state_dict(self, state: dict) -> None:
        self.data_buffer.load_state(state["buffer_state"])
