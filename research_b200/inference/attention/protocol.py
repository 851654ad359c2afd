"""Attention backend protocol (rollouts/inference/attention/protocol.py:10)."""

from __future__ import annotations

from typing import Protocol, runtime_checkable

import torch

from ..types import InferenceContext


@runtime_checkable
class AttentionBackend(Protocol):
    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layer_idx: int, ctx: InferenceContext) -> torch.Tensor: ...
