"""``Attention`` module: a thin ``nn.Module`` that forwards to a backend (rollouts/inference/attention/layer.py:10)."""

from __future__ import annotations

import torch
from torch import nn

from ..types import InferenceContext
from .protocol import AttentionBackend


class Attention(nn.Module):
    def __init__(self, backend: AttentionBackend, layer_idx: int):
        super().__init__()
        self.backend = backend
        self.layer_idx = layer_idx

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ctx: InferenceContext) -> torch.Tensor:
        return self.backend.forward(q, k, v, self.layer_idx, ctx)
