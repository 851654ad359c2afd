"""Packed variable-length flash attention on the tcgen05 tensor cores (``csrc/flash_sm100.cu``).

``flash_attn_varlen`` is the training / dense-prefill entry point (q, k, v are ``[T, H, D]`` views,
sequence boundaries in ``cu_seqlens``); ``flash_paged_prefill`` reads K/V from the paged cache.
Both return the output and, on request, the per-row log-sum-exp that the backward pass needs.
The PyTorch twins below are the oracles (fp32 softmax over masked scores).

Replaces ``F.scaled_dot_product_attention`` (rollouts/inference/attention/flex_backend.py:180-182)
and the Hopper-only ``flash_attn_varlen_func`` of dev/speedrun/single-file.py:932-943.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch

from .. import _native
from ._util import check_rc, ptr, status_tensor, stream_handle

c_int, c_float, c_vp = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


def _lib() -> ctypes.CDLL:
    lib = _native.load("rb_flash")
    if not getattr(lib, "_rb_typed", False):
        lib.rb_flash_fwd.argtypes = [c_vp] * 9 + [c_int] * 14 + [c_float, c_vp, c_vp]
        lib.rb_flash_fwd.restype = c_int
        lib.rb_flash_bwd.argtypes = [c_vp] * 13 + [c_int] * 13 + [c_float, c_vp, c_vp]
        lib.rb_flash_bwd.restype = c_int
        lib._rb_typed = True
    return lib


def _masked_scores(q, k, scale, q_pos, causal, window):
    Hq, Hkv = q.shape[1], k.shape[1]
    kf = k.float().repeat_interleave(Hq // Hkv, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    kpos = torch.arange(k.shape[0], device=q.device)
    dead = torch.zeros(q.shape[0], k.shape[0], dtype=torch.bool, device=q.device)
    if causal:
        dead |= kpos[None, :] > q_pos[:, None]
    if window > 0:
        dead |= kpos[None, :] <= (q_pos[:, None] - window)
    return s.masked_fill(dead[None], float("-inf"))


def flash_attn_varlen_reference(q, k, v, cu_q, cu_k, causal=True, window=0, scale=None):
    """fp32 oracle. Returns ``(out [Tq,Hq,D] in q.dtype, lse [Hq,Tq] fp32)``; queries of a sequence
    are its LAST positions when it has more keys than queries."""
    Tq, Hq, D = q.shape
    scale = scale or 1.0 / math.sqrt(D)
    out = torch.zeros(Tq, Hq, D, dtype=torch.float32, device=q.device)
    lse = torch.full((Hq, Tq), float("-inf"), dtype=torch.float32, device=q.device)
    g = Hq // k.shape[1]
    for b in range(len(cu_q) - 1):
        qs, qe, ks, ke = int(cu_q[b]), int(cu_q[b + 1]), int(cu_k[b]), int(cu_k[b + 1])
        if qe == qs:
            continue
        q_pos = torch.arange((ke - ks) - (qe - qs), ke - ks, device=q.device)
        s = _masked_scores(q[qs:qe], k[ks:ke], scale, q_pos, causal, window)
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l[..., None]).nan_to_num(0.0)
        out[qs:qe] = torch.einsum("hqk,khd->qhd", p, v[ks:ke].float().repeat_interleave(g, dim=1))
        lse[:, qs:qe] = l
    return out.to(q.dtype), lse


def flash_attn_varlen(q, k, v, cu_q, cu_k, max_seqlen_q: int, causal: bool = True, window: int = 0, scale=None,
                      out=None, return_lse: bool = False):
    """``q [Tq,Hq,D]``, ``k/v [Tk,Hkv,D]`` bf16 with unit stride in D and any row stride (views of a
    fused QKV projection are fine). ``cu_q``/``cu_k``: int32 ``[B+1]`` on the same device."""
    Tq, Hq, D = q.shape
    if not q.is_cuda:
        o, lse = flash_attn_varlen_reference(q, k, v, cu_q, cu_k, causal, window, scale)
        if out is not None:
            out.copy_(o)
            o = out
        return (o, lse) if return_lse else o
    Tk, Hkv, _ = k.shape
    scale = scale or 1.0 / math.sqrt(D)
    for t in (q, k, v):
        assert t.dtype == torch.bfloat16 and t.stride(2) == 1 and t.stride(1) == D, "heads must be packed [T, H, D]"
    assert cu_q.dtype == torch.int32 and cu_k.dtype == torch.int32 and cu_q.is_cuda and cu_k.is_cuda
    if out is None:
        out = torch.empty(Tq, Hq, D, dtype=torch.bfloat16, device=q.device)
    assert out.is_contiguous()
    lse = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device) if return_lse else None
    B = cu_q.shape[0] - 1
    rc = _lib().rb_flash_fwd(ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), ptr(cu_q), ptr(cu_k), None, None, B, Tq, Tk,
                             Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), max_seqlen_q, 0, int(causal),
                             int(window), 0, scale, ptr(status_tensor(q.device)), stream_handle(q.device))
    check_rc(rc, "rb_flash_fwd")
    return (out, lse) if return_lse else out


def flash_paged_prefill(q, k_cache, v_cache, block_tables, cu_q, seq_lens, max_new: int, scale=None, window: int = 0,
                        out=None, lse: torch.Tensor | None = None):
    """Causal attention of packed new tokens against (cached prefix + themselves) in the paged cache.
    Unwritten cache slots must hold finite numbers (the cache is allocated zero-filled)."""
    T, Hq, D = q.shape
    nb, Hkv, bs, _ = k_cache.shape
    assert bs == 16 and q.is_contiguous() and cu_q.dtype == torch.int32 and seq_lens.dtype == torch.int32
    scale = scale or 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty_like(q)
    B = seq_lens.shape[0]
    rc = _lib().rb_flash_fwd(ptr(q), ptr(k_cache), ptr(v_cache), ptr(out), ptr(lse), ptr(cu_q), None, ptr(seq_lens),
                             ptr(block_tables), B, T, nb, Hq, Hkv, D, q.stride(0), 0, 0, max_new,
                             block_tables.shape[1], 1, int(window), 1, scale, ptr(status_tensor(q.device)),
                             stream_handle(q.device))
    check_rc(rc, "rb_flash_fwd(paged)")
    return out


def flash_attn_varlen_backward(q, k, v, out, dout, lse, cu_q, cu_k, max_seqlen_q: int, max_seqlen_k: int,
                               causal: bool = True, window: int = 0, scale=None):
    """Gradients ``(dq, dk, dv)`` of ``flash_attn_varlen`` (bf16, contiguous ``[T, H, D]``)."""
    Tq, Hq, D = q.shape
    Tk, Hkv, _ = k.shape
    scale = scale or 1.0 / math.sqrt(D)
    if not q.is_cuda:
        with torch.enable_grad():
            qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
            o, _ = flash_attn_varlen_reference(qf, kf, vf, cu_q, cu_k, causal, window, scale)
            dq, dk, dv = torch.autograd.grad(o, (qf, kf, vf), dout.float())
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)
    dout = dout.contiguous()
    assert out.is_contiguous() and lse.is_contiguous() and dout.dtype == torch.bfloat16
    dq = torch.empty(Tq, Hq, D, dtype=torch.bfloat16, device=q.device)
    dk = torch.empty(Tk, Hkv, D, dtype=torch.bfloat16, device=q.device)
    dv = torch.empty(Tk, Hkv, D, dtype=torch.bfloat16, device=q.device)
    ws = torch.empty(2 * Hq * Tq, dtype=torch.float32, device=q.device)
    B = cu_q.shape[0] - 1
    part = None
    if head_split_pays(B, max_seqlen_q, max_seqlen_k, Hq, Hkv):
        part = torch.empty(2 * (Hq // Hkv) * Tk * Hkv * D, dtype=torch.float32, device=q.device)
    rc = _lib().rb_flash_bwd(ptr(q), ptr(k), ptr(v), ptr(out), ptr(dout), ptr(lse), ptr(dq), ptr(dk), ptr(dv), ptr(cu_q),
                             ptr(cu_k), ptr(ws), ptr(part) if part is not None else None, B, Tq, Tk, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0),
                             max_seqlen_q, max_seqlen_k, int(causal), int(window), scale,
                             ptr(status_tensor(q.device)), stream_handle(q.device))
    check_rc(rc, "rb_flash_bwd")
    return dq, dk, dv


_HEAD_SPLIT = os.environ.get("RB_FLASH_BWD_HEAD_SPLIT", "auto")     # auto | 0 | 1


def head_split_pays(B: int, max_seqlen_q: int, max_seqlen_k: int, Hq: int, Hkv: int) -> bool:
    """dK/dV as one CTA per (key tile, QUERY head) + a reduction over each group, instead of one CTA per (key tile,
    key/value head) looping over its G query heads. It pays only where the coarse grid has fewer CTAs than the GPU has
    SMs (one long sequence with two kv heads: 64 CTAs). Measured on the Llama-3-8B step (one 4096-token sequence, 8 kv
    heads: 256 CTAs, the longest 256 iterations against 228 per SM on average) the split changes nothing: 255.2 ms per
    step with it, 253.5 without; the kernel is bound by its 3.7 us per iteration, not by balance. The split costs
    2 * G * Tk * Hkv * D floats of workspace and one pass over them."""
    G = Hq // Hkv
    if _HEAD_SPLIT in ("0", "1"):
        return G > 1 and _HEAD_SPLIT == "1"
    ctas = -(-max_seqlen_k // 128) * Hkv * B
    return G > 1 and ctas < 148 and (max_seqlen_q // 64) * G >= 64


class FlashAttnVarlen(torch.autograd.Function):
    """Differentiable packed attention: tcgen05 kernels on CUDA, the fp32 reference on CPU."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, causal, window, scale):
        out, lse = flash_attn_varlen(q, k, v, cu_q, cu_k, max_q, causal=causal, window=window, scale=scale,
                                     return_lse=True)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.cfg = (max_q, max_k, causal, window, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        max_q, max_k, causal, window, scale = ctx.cfg
        dq, dk, dv = flash_attn_varlen_backward(q, k, v, out, dout, lse, cu_q, cu_k, max_q, max_k, causal, window, scale)
        return dq, dk, dv, None, None, None, None, None, None, None


def flash_attention(q, k, v, cu_q, cu_k, max_seqlen_q: int, max_seqlen_k: int, causal: bool = True, window: int = 0,
                    scale=None):
    """Autograd entry point used by the training model."""
    return FlashAttnVarlen.apply(q, k, v, cu_q, cu_k, max_seqlen_q, max_seqlen_k, causal, window, scale)
