"""KV cache geometry (rollouts/inference/attention/config.py:9-45)."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class CacheConfig:
    num_layers: int
    num_kv_heads: int
    head_dim: int
    num_blocks: int
    block_size: int = 16
    dtype: torch.dtype = torch.bfloat16
    device: str = "cuda"
    sliding_window: int = 0

    @property
    def num_slots(self) -> int:
        return self.num_blocks * self.block_size

    @property
    def bytes_per_block(self) -> int:
        return 2 * self.num_layers * self.num_kv_heads * self.block_size * self.head_dim * torch.finfo(self.dtype).bits // 8

    @property
    def total_bytes(self) -> int:
        return self.bytes_per_block * self.num_blocks

    @staticmethod
    def blocks_for_budget(num_layers: int, num_kv_heads: int, head_dim: int, budget_bytes: int, block_size: int = 16,
                          dtype: torch.dtype = torch.bfloat16) -> int:
        per = 2 * num_layers * num_kv_heads * block_size * head_dim * torch.finfo(dtype).bits // 8
        return max(1, budget_bytes // per)
