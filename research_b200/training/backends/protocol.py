"""The four-method training backend surface (rollouts/training/backends/protocol.py:16-67)."""

from __future__ import annotations

from typing import Any, Protocol, runtime_checkable

from ..types import TrainFuture


@runtime_checkable
class TrainingBackend(Protocol):
    def forward_backward(self, batch: dict[str, Any]) -> TrainFuture[dict[str, float]]: ...
    def optim_step(self) -> TrainFuture[dict[str, float]]: ...
    def get_weights(self) -> TrainFuture[dict[str, Any]]: ...
    def load_weights(self, weights: dict[str, Any]) -> TrainFuture[None]: ...
