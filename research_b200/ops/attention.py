"""Paged-KV attention (csrc/attn_sm100.cu) and PyTorch reference twins.

Cache layout per layer: ``[num_blocks, Hkv, block_size(=16), D]`` bf16.
Behaviour replaced: rollouts/inference/attention/flex_backend.py:144-279.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch

from .. import _native
from ._util import check_rc, ptr, status_tensor, stream_handle

c_int, c_ll, c_float, c_vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def _lib() -> ctypes.CDLL:
    lib = _native.load("rb_attn")
    if not getattr(lib, "_rb_typed", False):
        lib.rb_paged_decode.argtypes = [c_vp] * 7 + [c_int] * 8 + [c_float, c_vp, c_vp]
        lib.rb_paged_decode.restype = c_int
        lib.rb_paged_prefill.argtypes = [c_vp] * 8 + [c_int] * 8 + [c_float, c_int, c_vp, c_vp]
        lib.rb_paged_prefill.restype = c_int
        lib.rb_paged_decode_workspace_floats.argtypes = [c_int] * 4
        lib.rb_paged_decode_workspace_floats.restype = c_ll
        lib._rb_typed = True
    return lib


def gather_kv(cache: torch.Tensor, block_table: torch.Tensor, length: int) -> torch.Tensor:
    """Contiguous ``[length, Hkv, D]`` view of one sequence's K or V (reference helper)."""
    bs = cache.shape[2]
    n = (length + bs - 1) // bs
    blocks = cache[block_table[:n].long()]  # [n, Hkv, bs, D]
    return blocks.permute(0, 2, 1, 3).reshape(n * bs, cache.shape[1], cache.shape[3])[:length]


def _sdpa_ref(q, k, v, q_pos, scale, window):
    # q [Tq, Hq, D], k/v [Tk, Hkv, D], q_pos [Tq] absolute positions; causal on absolute positions
    Hq, Hkv = q.shape[1], k.shape[1]
    kf = k.float().repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().repeat_interleave(Hq // Hkv, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    kpos = torch.arange(k.shape[0], device=q.device)
    dead = kpos[None, :] > q_pos[:, None]
    if window > 0:
        dead |= kpos[None, :] <= (q_pos[:, None] - window)
    s = s.masked_fill(dead[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vf)


def paged_decode_reference(q, k_cache, v_cache, block_tables, seq_lens, scale=None):
    B, Hq, D = q.shape
    scale = scale or 1.0 / math.sqrt(D)
    out = torch.zeros_like(q, dtype=torch.float32)
    for b in range(B):
        L = int(seq_lens[b])
        if L == 0:
            continue
        k = gather_kv(k_cache, block_tables[b], L)
        v = gather_kv(v_cache, block_tables[b], L)
        out[b] = _sdpa_ref(q[b : b + 1], k, v, torch.tensor([L - 1], device=q.device), scale, 0)[0]
    return out.to(q.dtype)


def paged_prefill_reference(q, k_cache, v_cache, block_tables, cu_q, seq_lens, scale=None, window=0):
    T, Hq, D = q.shape
    scale = scale or 1.0 / math.sqrt(D)
    out = torch.zeros_like(q, dtype=torch.float32)
    for b in range(len(seq_lens)):
        s, e = int(cu_q[b]), int(cu_q[b + 1])
        L = int(seq_lens[b])
        if e == s:
            continue
        k = gather_kv(k_cache, block_tables[b], L)
        v = gather_kv(v_cache, block_tables[b], L)
        q_pos = torch.arange(L - (e - s), L, device=q.device)
        out[s:e] = _sdpa_ref(q[s:e], k, v, q_pos, scale, window)
    return out.to(q.dtype)


def decode_num_splits(batch: int, hkv: int, max_len: int, sms: int = 148, head_dim: int = 64) -> int:
    """Number of KV splits per (sequence, kv head). One CTA handles one split; the GPU holds
    ``sms x (4 CTAs at head_dim 64, 2 at 128)`` CTAs at once, so the cost of a choice is the number
    of CTA waves divided by the split count, plus a small charge per split for the merge pass."""
    if max_len <= 512:
        return 1
    slots = sms * (4 if head_dim <= 64 else 2)
    ctas = max(batch * hkv, 1)
    max_splits = int(min(32, max(1, max_len // 256)))
    best, best_cost = 1, None
    for s in range(1, max_splits + 1):
        waves = -(-ctas * s // slots)
        cost = waves / s + 0.02 * (s - 1)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def paged_decode(q, k_cache, v_cache, block_tables, seq_lens, scale=None, num_splits: int = 1, out=None,
                 workspace: torch.Tensor | None = None):
    """One query token per sequence against its paged context. ``q``: ``[B, Hq, D]``."""
    if not q.is_cuda:
        res = paged_decode_reference(q, k_cache, v_cache, block_tables, seq_lens, scale)
        if out is not None:
            out.copy_(res)
            return out
        return res
    B, Hq, D = q.shape
    nb, Hkv, bs, _ = k_cache.shape
    scale = scale or 1.0 / math.sqrt(D)
    assert q.is_contiguous() and block_tables.dtype == torch.int32 and seq_lens.dtype == torch.int32
    assert block_tables.is_contiguous()
    if out is None:
        out = torch.empty_like(q)
    if num_splits > 1:
        need = _lib().rb_paged_decode_workspace_floats(B, Hq, D, num_splits)
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.float32, device=q.device)
        assert workspace.numel() >= need
    rc = _lib().rb_paged_decode(ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_tables), ptr(seq_lens), ptr(out),
                                ptr(workspace), B, Hq, Hkv, D, block_tables.shape[1], nb, bs, num_splits, scale,
                                ptr(status_tensor(q.device)), stream_handle(q.device))
    check_rc(rc, "rb_paged_decode", 2 if num_splits > 1 else 1)
    return out


def paged_prefill(q, k_cache, v_cache, block_tables, cu_q, seq_lens, max_new: int, scale=None, window: int = 0,
                  out=None, lse: torch.Tensor | None = None):
    """Causal attention of packed new tokens ``q [T, Hq, D]`` against prefix + themselves."""
    if not q.is_cuda:
        res = paged_prefill_reference(q, k_cache, v_cache, block_tables, cu_q, seq_lens, scale, window)
        if out is not None:
            out.copy_(res)
            return out
        return res
    T, Hq, D = q.shape
    nb, Hkv, bs, _ = k_cache.shape
    scale = scale or 1.0 / math.sqrt(D)
    assert q.is_contiguous() and cu_q.dtype == torch.int32 and seq_lens.dtype == torch.int32
    if out is None:
        out = torch.empty_like(q)
    B = seq_lens.shape[0]
    if D in (64, 128) and bs == 16 and not os.environ.get("RB_PREFILL_MMA_SYNC"):
        from .flash import flash_paged_prefill   # tcgen05 kernel; the mma.sync kernel below is the fallback

        return flash_paged_prefill(q, k_cache, v_cache, block_tables, cu_q, seq_lens, max_new, scale, window, out, lse)
    rc = _lib().rb_paged_prefill(ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_tables), ptr(cu_q), ptr(seq_lens),
                                 ptr(out), ptr(lse), B, max_new, Hq, Hkv, D, block_tables.shape[1], nb, bs, scale,
                                 window, ptr(status_tensor(q.device)), stream_handle(q.device))
    check_rc(rc, "rb_paged_prefill")
    return out
