"""Mask factories: causal, causal + sliding window, packed documents
(rollouts/inference/attention/mask.py:21-191). The reference builds FlexAttention
``BlockMask`` objects; the kernels here take the window size / ``cu_seqlens`` directly, so these
return dense boolean masks (True = attend) for reference computations and tests, plus a
``mask_mod``-style predicate usable with ``torch.nn.attention.flex_attention`` if desired."""

from __future__ import annotations

from typing import Callable

import torch


def causal_mask(q_len: int, kv_len: int | None = None, device=None) -> torch.Tensor:
    kv_len = kv_len or q_len
    q = torch.arange(kv_len - q_len, kv_len, device=device)[:, None]
    k = torch.arange(kv_len, device=device)[None, :]
    return k <= q


def sliding_window_causal_mask(q_len: int, window: int, kv_len: int | None = None, device=None) -> torch.Tensor:
    kv_len = kv_len or q_len
    q = torch.arange(kv_len - q_len, kv_len, device=device)[:, None]
    k = torch.arange(kv_len, device=device)[None, :]
    return (k <= q) & (k > q - window)


def document_causal_mask(cu_seqlens: torch.Tensor, total: int | None = None, device=None) -> torch.Tensor:
    total = total if total is not None else int(cu_seqlens[-1])
    doc = torch.bucketize(torch.arange(total, device=device), cu_seqlens[1:].to(device), right=True)
    same = doc[:, None] == doc[None, :]
    return same & causal_mask(total, device=device)


def causal_mask_mod(b, h, q_idx, kv_idx):
    return kv_idx <= q_idx


def make_sliding_window_mask_mod(window: int) -> Callable:
    def mod(b, h, q_idx, kv_idx):
        return (kv_idx <= q_idx) & (kv_idx > q_idx - window)

    return mod


def make_document_mask_mod(doc_ids: torch.Tensor) -> Callable:
    def mod(b, h, q_idx, kv_idx):
        return (doc_ids[q_idx] == doc_ids[kv_idx]) & (kv_idx <= q_idx)

    return mod
