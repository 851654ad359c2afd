"""RMSNorm, RoPE + paged KV append, SwiGLU, embedding (csrc/ops_sm100.cu) with reference twins.

The reference twins follow the rounding points of the bf16 Hugging Face modules, which are
also what the functional oracles in the reference implement
(rollouts/tools/functional_extractor/qwen_functional.py:46-150, 251-274).
"""

from __future__ import annotations

import ctypes

import torch

from .. import _native
from ._util import check_rc, ptr, status_tensor, stream_handle

c_int, c_ll, c_float, c_vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def _lib() -> ctypes.CDLL:
    lib = _native.load("rb_ops")
    if not getattr(lib, "_rb_typed", False):
        lib.rb_rmsnorm.argtypes = [c_vp, c_vp, c_vp, c_ll, c_int, c_ll, c_ll, c_float, c_vp]
        lib.rb_rope_kv_append.argtypes = [c_vp] * 9 + [c_float, c_int, c_int, c_int, c_int, c_int, c_ll, c_int, c_vp, c_vp]
        lib.rb_swiglu.argtypes = [c_vp, c_vp, c_ll, c_int, c_vp]
        lib.rb_swiglu_bwd.argtypes = [c_vp, c_vp, c_vp, c_ll, c_int, c_vp]
        lib.rb_swiglu_bounded.argtypes = [c_vp, c_vp, c_ll, c_int, c_vp, c_vp]
        lib.rb_swiglu_bounded.restype = c_int
        lib.rb_embedding.argtypes = [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_vp]
        lib.rb_transpose_bf16.argtypes = [c_vp, c_vp, c_int, c_int, c_vp]
        for f in ("rb_rmsnorm", "rb_rope_kv_append", "rb_swiglu", "rb_swiglu_bwd", "rb_embedding", "rb_transpose_bf16"):
            getattr(lib, f).restype = c_int
        lib._rb_typed = True
    return lib


# ------------------------------------------------------------------------------- RMSNorm
def rmsnorm_reference(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = (xf * torch.rsqrt(var + eps)).to(x.dtype)
    return w * y


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """Row RMSNorm over the last dim; also used per head (QK-norm) with ``x`` reshaped."""
    if not x.is_cuda:
        res = rmsnorm_reference(x, w, eps)
        if out is not None:
            out.copy_(res)
            return out
        return res
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    assert x2.stride(1) == 1 and x.dtype == torch.bfloat16
    if out is None:
        out = torch.empty_like(x2)
    o2 = out.reshape(-1, d)
    rc = _lib().rb_rmsnorm(ptr(x2), ptr(w), ptr(o2), x2.shape[0], d, x2.stride(0), o2.stride(0), eps, stream_handle(x.device))
    check_rc(rc, "rb_rmsnorm")
    return out.reshape(x.shape)


# ------------------------------------------------------------------------------- RoPE tables
def rope_table(max_pos: int, head_dim: int, theta: float, device=None) -> torch.Tensor:
    """``[max_pos, head_dim/2, 2]`` fp32 table of (cos, sin), HF ``inv_freq`` convention."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    pos = torch.arange(max_pos, dtype=torch.float32)
    ang = torch.outer(pos, inv_freq)
    tab = torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()
    return tab.to(device) if device is not None else tab


def _rotate_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x [T, H, D]; cos/sin [T, D/2] fp32 -> HF: cat(freqs,freqs), cast to x.dtype, x*cos + rotate_half(x)*sin
    c = torch.cat([cos, cos], -1).to(x.dtype)[:, None, :]
    s = torch.cat([sin, sin], -1).to(x.dtype)[:, None, :]
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], -1)
    return x * c + rot * s


def rope_kv_append_reference(qkv, positions, slots, table, k_cache, v_cache, Hq, Hkv, D, q_norm_w=None, k_norm_w=None, eps=1e-6):
    T = qkv.shape[0]
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    q = q.reshape(T, Hq, D)
    k = k.reshape(T, Hkv, D)
    v = v.reshape(T, Hkv, D)
    if q_norm_w is not None:
        q = rmsnorm_reference(q, q_norm_w, eps)
        k = rmsnorm_reference(k, k_norm_w, eps)
    cs = table[positions.long().clamp(min=0)]
    q = _rotate_reference(q, cs[..., 0], cs[..., 1])
    k = _rotate_reference(k, cs[..., 0], cs[..., 1])
    bs = k_cache.shape[2]
    ok = slots >= 0
    sl = slots[ok].long()
    k_cache[sl // bs, :, sl % bs] = k[ok]
    v_cache[sl // bs, :, sl % bs] = v[ok]
    return q.reshape(T, Hq * D)


def rope_kv_append(qkv, positions, slots, table, k_cache, v_cache, Hq, Hkv, D, q_norm_w=None, k_norm_w=None,
                   eps: float = 1e-6, q_out: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate q and k, write k/v into the paged cache at ``slots``, return rotated q ``[T, Hq*D]``.

    ``k_cache``/``v_cache``: ``[num_blocks, Hkv, block_size, D]``; ``slots`` < 0 rows are skipped.
    """
    if not qkv.is_cuda:
        res = rope_kv_append_reference(qkv, positions, slots, table, k_cache, v_cache, Hq, Hkv, D, q_norm_w, k_norm_w, eps)
        if q_out is not None:
            q_out.copy_(res)
            return q_out
        return res
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (Hq + 2 * Hkv) * D
    assert positions.dtype == torch.int32 and slots.dtype == torch.int32
    assert table.dtype == torch.float32 and table.is_contiguous()
    if q_out is None:
        q_out = torch.empty(T, Hq * D, dtype=qkv.dtype, device=qkv.device)
    nb, _, bs, _ = k_cache.shape
    rc = _lib().rb_rope_kv_append(
        ptr(qkv), ptr(q_out), ptr(k_cache), ptr(v_cache), ptr(positions), ptr(slots), ptr(table), ptr(q_norm_w),
        ptr(k_norm_w), eps, T, Hq, Hkv, D, bs, nb * bs, table.shape[0], ptr(status_tensor(qkv.device)),
        stream_handle(qkv.device))
    check_rc(rc, "rb_rope_kv_append")
    return q_out


# ------------------------------------------------------------------------------- SwiGLU
def swiglu_reference(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu.chunk(2, dim=-1)
    return torch.nn.functional.silu(g) * u


def swiglu(gu: torch.Tensor, out: torch.Tensor | None = None, rows_dev: torch.Tensor | None = None) -> torch.Tensor:
    """``silu(gate) * up`` for ``gu = [gate | up]`` of shape ``[T, 2F]``. ``rows_dev`` (an int32 element on the
    device) caps the number of rows processed at run time; rows beyond it are left untouched."""
    if not gu.is_cuda:
        res = swiglu_reference(gu)
        if out is not None:
            out.copy_(res)
            return out
        return res
    T, F2 = gu.reshape(-1, gu.shape[-1]).shape
    F = F2 // 2
    assert gu.is_contiguous()
    if out is None:
        out = torch.empty(*gu.shape[:-1], F, dtype=gu.dtype, device=gu.device)
    if rows_dev is not None:
        assert rows_dev.dtype == torch.int32 and rows_dev.is_cuda
        rc = _lib().rb_swiglu_bounded(ptr(gu), ptr(out), T, F, rows_dev.data_ptr(), stream_handle(gu.device))
    else:
        rc = _lib().rb_swiglu(ptr(gu), ptr(out), T, F, stream_handle(gu.device))
    check_rc(rc, "rb_swiglu")
    return out


def swiglu_backward(gu: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    if not gu.is_cuda:
        g, u = gu.float().chunk(2, dim=-1)
        sig = torch.sigmoid(g)
        silu = g * sig
        dy = dout.float()
        return torch.cat([dy * u * (sig + silu * (1 - sig)), dy * silu], -1).to(gu.dtype)
    T, F2 = gu.reshape(-1, gu.shape[-1]).shape
    dgu = torch.empty_like(gu)
    rc = _lib().rb_swiglu_bwd(ptr(gu), ptr(dout.contiguous()), ptr(dgu), T, F2 // 2, stream_handle(gu.device))
    check_rc(rc, "rb_swiglu_bwd")
    return dgu


# ------------------------------------------------------------------------------- embedding
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if not table.is_cuda:
        res = table[ids.long()]
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert ids.dtype == torch.int32 and ids.is_contiguous()
    T = ids.numel()
    d = table.shape[1]
    if out is None:
        out = torch.empty(T, d, dtype=table.dtype, device=table.device)
    rc = _lib().rb_embedding(ptr(ids), ptr(table), ptr(out), T, d, table.shape[0], ptr(status_tensor(table.device)),
                             stream_handle(table.device))
    check_rc(rc, "rb_embedding")
    return out


def transpose(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        return x.t().contiguous()
    assert x.dim() == 2 and x.is_contiguous() and x.dtype == torch.bfloat16
    out = torch.empty(x.shape[1], x.shape[0], dtype=x.dtype, device=x.device)
    rc = _lib().rb_transpose_bf16(ptr(x), ptr(out), x.shape[0], x.shape[1], stream_handle(x.device))
    check_rc(rc, "rb_transpose_bf16")
    return out
