"""Paged attention backend on the sm_100a kernels.

Owns ``[L, num_blocks, Hkv, 16, D]`` K and V tensors. ``forward`` stores the new K/V at the
context's slots and runs varlen causal prefill (against cached prefix + new tokens) or
split-KV decode. It plays the role of the reference's ``FlexAttentionBackend``
(rollouts/inference/attention/flex_backend.py:11-279), whose decode path gathers K/V with a
Python loop per position; here both phases are single kernel launches with GQA handled inside
the kernel (no ``repeat_interleave``).

K and V arrive already rotated (RoPE is applied by the caller, as in the reference backend).
"""

from __future__ import annotations

import math

import torch

from ... import ops
from ..types import InferenceContext
from .config import CacheConfig


class PagedAttentionBackend:
    def __init__(self, config: CacheConfig):
        assert config.block_size == 16, "the kernels use 16-token blocks"
        self.config = config
        dev = torch.device(config.device)
        shape = (config.num_layers, config.num_blocks, config.num_kv_heads, config.block_size, config.head_dim)
        self.k_cache = torch.zeros(shape, dtype=config.dtype, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.scale = 1.0 / math.sqrt(config.head_dim)

    def _store_kv(self, k: torch.Tensor, v: torch.Tensor, layer_idx: int, slots: torch.Tensor) -> None:
        """k, v: ``[tokens, Hkv, D]``; slot = block * block_size + offset; negative slots are skipped."""
        bs = self.config.block_size
        ok = slots >= 0
        s = slots[ok].long()
        self.k_cache[layer_idx][s // bs, :, s % bs] = k[ok]
        self.v_cache[layer_idx][s // bs, :, s % bs] = v[ok]

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layer_idx: int, ctx: InferenceContext) -> torch.Tensor:
        """q ``[tokens, Hq, D]``, k/v ``[tokens, Hkv, D]`` for the NEW tokens of the batch; returns ``[tokens, Hq, D]``."""
        dev = q.device
        slots = torch.tensor(ctx.slot_mapping, dtype=torch.int32, device=dev)
        self._store_kv(k, v, layer_idx, slots)
        B = len(ctx.seq_lens)
        max_blocks = max(len(b) for b in ctx.block_tables)
        bt = torch.zeros(B, max_blocks, dtype=torch.int32, device=dev)
        for i, blocks in enumerate(ctx.block_tables):
            bt[i, :len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
        lens = torch.tensor(ctx.seq_lens, dtype=torch.int32, device=dev)
        if ctx.is_prefill:
            qlens = ctx.query_lens or ctx.seq_lens
            cu = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=dev)
            return ops.paged_prefill(q.contiguous(), self.k_cache[layer_idx], self.v_cache[layer_idx], bt, cu, lens,
                                     max(qlens), self.scale, ctx.sliding_window or self.config.sliding_window)
        splits = ops.decode_num_splits(B, self.config.num_kv_heads, max(ctx.seq_lens), head_dim=self.config.head_dim)
        return ops.paged_decode(q.contiguous(), self.k_cache[layer_idx], self.v_cache[layer_idx], bt, lens, self.scale, splits)
