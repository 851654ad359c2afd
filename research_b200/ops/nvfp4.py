"""NVFP4 (e2m1 data, e4m3 scale per 16 elements) block-scaled matrix-vector product.

``nvfp4_gemv`` runs ``csrc/quant_sm100.cu`` on CUDA and the decode-and-dot reference on CPU; the
helpers quantise / dequantise tensors so tests and callers need no special torch dtypes. Semantics
follow dev/kernels-gpumode/nvfp4/reference_kernel.py:29-55 (``c[m,l] = sum_k a*sfa*b*sfb`` in fp16).
"""

from __future__ import annotations

import ctypes

import torch

from .. import _native
from ._util import check_rc, ptr, stream_handle

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def _lib() -> ctypes.CDLL:
    lib = _native.load("rb_quant")
    if not getattr(lib, "_rb_typed", False):
        lib.rb_nvfp4_gemv.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
        lib.rb_nvfp4_gemv.restype = ctypes.c_int
        lib._rb_typed = True
    return lib


def decode_e2m1(packed: torch.Tensor) -> torch.Tensor:
    """uint8 ``[..., K/2]`` (low nibble first) -> fp32 ``[..., K]``."""
    lo, hi = packed & 0xF, packed >> 4
    nib = torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], -1).long()
    mag = E2M1_VALUES.to(packed.device)[nib & 7]
    return torch.where((nib & 8) != 0, -mag, mag)


def decode_e4m3(b: torch.Tensor) -> torch.Tensor:
    """uint8 e4m3 (bias 7, no infinities) -> fp32."""
    x = b.long()
    e, m = (x >> 3) & 0xF, x & 7
    mag = torch.where(e == 0, m.float() / 8 * 2.0 ** -6, (1 + m.float() / 8) * torch.pow(2.0, (e - 7).float()))
    return torch.where((x & 0x80) != 0, -mag, mag)


def encode_e4m3(x: torch.Tensor) -> torch.Tensor:
    """Nearest e4m3 code of non-negative fp32 values (used for scale factors)."""
    codes = torch.arange(0, 127, dtype=torch.uint8, device=x.device)          # 0x7f is NaN
    table = decode_e4m3(codes)
    idx = torch.bucketize(x.clamp(0, table[-1].item()).contiguous(), table).clamp(1, len(table) - 1)
    lower_closer = (x - table[idx - 1]).abs() <= (table[idx] - x).abs()
    return torch.where(lower_closer, idx - 1, idx).to(torch.uint8)


def quantize_nvfp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``[..., K]`` (K % 16 == 0) -> (packed e2m1 ``[..., K/2]`` uint8, e4m3 scales ``[..., K/16]`` uint8)."""
    K = x.shape[-1]
    assert K % 16 == 0
    blocks = x.float().reshape(*x.shape[:-1], K // 16, 16)
    sf = encode_e4m3(blocks.abs().amax(-1) / 6.0)
    scale = decode_e4m3(sf).clamp_min(2.0 ** -9)[..., None]
    y = blocks / scale
    table = E2M1_VALUES.to(x.device)
    code = (y.abs()[..., None] - table).abs().argmin(-1)
    code = code | ((y < 0).long() << 3)
    code = code.reshape(*x.shape[:-1], K)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).to(torch.uint8)
    return packed, sf


def nvfp4_gemv_reference(a, b, sfa, sfb) -> torch.Tensor:
    """``a [L,M,K/2]``, ``b [L,K/2]``, ``sfa [L,M,K/16]``, ``sfb [L,K/16]`` uint8 -> fp16 ``[L,M]``."""
    av = decode_e2m1(a) * decode_e4m3(sfa).repeat_interleave(16, dim=-1)
    bv = decode_e2m1(b) * decode_e4m3(sfb).repeat_interleave(16, dim=-1)
    return torch.einsum("lmk,lk->lm", av.double(), bv.double()).to(torch.float16)


def nvfp4_gemv(a, b, sfa, sfb, out=None) -> torch.Tensor:
    L, M, kb = a.shape
    if not a.is_cuda:
        res = nvfp4_gemv_reference(a, b, sfa, sfb)
        if out is not None:
            out.copy_(res)
            return out
        return res
    for t in (a, b, sfa, sfb):
        assert t.dtype == torch.uint8 and t.is_contiguous()
    assert b.shape == (L, kb) and sfa.shape == (L, M, kb // 8) and sfb.shape == (L, kb // 8)
    if out is None:
        out = torch.empty(L, M, dtype=torch.float16, device=a.device)
    rc = _lib().rb_nvfp4_gemv(ptr(a), ptr(b), ptr(sfa), ptr(sfb), ptr(out), L, M, kb * 2, stream_handle(a.device))
    check_rc(rc, "rb_nvfp4_gemv")
    return out
