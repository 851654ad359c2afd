"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory where they need attention (a serving
loop with a frozen memory pool, a host application whose other runtime owns all GPU memory, a
plugin called where cudaMalloc is forbidden). ``rb_paged_decode_noalloc`` keeps the split-KV
workspace inside the library for them. This test calls the raw symbol with raw pointers, twice
in a row (the internal array keeps the previous call's contents), and compares with the regular
entry point. It lives in a file that pytest collects last so an earlier-stopping run has
already exercised everything else; it also passes when run alone in a fresh process.
"""

import ctypes

import pytest
import torch

from research_b200 import _native, ops

pytestmark = pytest.mark.gpu

MAX_FLOATS = 4 * 1024 * 1024
TOO_LARGE = -40


def _lib():
    lib = ctypes.CDLL(str(_native.lib_path("rb_attn")))
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.rb_paged_decode_noalloc.argtypes = [vp] * 6 + [i] * 8 + [f, vp, vp]
    lib.rb_paged_decode_noalloc.restype = i
    lib.rb_paged_decode_noalloc_required_floats.argtypes = [i] * 4
    lib.rb_paged_decode_noalloc_required_floats.restype = ctypes.c_longlong
    return lib


def _case(device, B, Hq, Hkv, D, lens, seed):
    g = torch.Generator().manual_seed(seed)
    bs = 16
    nblk = [(n + bs - 1) // bs for n in lens]
    total = sum(nblk) + 2
    kc = (torch.randn(total, Hkv, bs, D, generator=g)).bfloat16().to(device)
    vc = (torch.randn(total, Hkv, bs, D, generator=g)).bfloat16().to(device)
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(B, max(nblk), dtype=torch.int32)
    o = 0
    for b in range(B):
        bt[b, :nblk[b]] = perm[o:o + nblk[b]].to(torch.int32)
        o += nblk[b]
    q = torch.randn(B, Hq, D, generator=g).bfloat16().to(device)
    return q, kc, vc, bt.to(device), torch.tensor(lens, dtype=torch.int32, device=device)


def _call(lib, q, kc, vc, bt, sl, splits):
    B, Hq, D = q.shape
    out = torch.empty_like(q)
    status = ops.status_tensor(q.device)
    rc = lib.rb_paged_decode_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(),
                                     out.data_ptr(), B, Hq, kc.shape[1], D, bt.shape[1], kc.shape[0], 16, splits,
                                     1.0 / D ** 0.5, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_noalloc_decode_matches_regular_entry_point_twice(cuda_device):
    lib = _lib()
    # two different problems back to back: the second runs over the first one's leftovers
    for seed, (B, Hq, Hkv, D, lens, splits) in enumerate([(6, 14, 2, 64, [700, 33, 1024, 16, 257, 5], 4),
                                                           (4, 32, 8, 128, [2048, 100, 900, 1], 8)]):
        q, kc, vc, bt, sl = _case(cuda_device, B, Hq, Hkv, D, lens, seed)
        assert lib.rb_paged_decode_noalloc_required_floats(B, Hq, D, splits) <= MAX_FLOATS
        want = ops.paged_decode(q, kc, vc, bt, sl, num_splits=splits)
        rc, got = _call(lib, q, kc, vc, bt, sl, splits)
        assert rc == 0
        torch.cuda.synchronize()
        diff = (got.float() - want.float()).abs()
        assert diff.max().item() < 0.01 and diff.mean().item() < 0.001, (diff.max().item(), diff.mean().item())
        # and against the fp32 reference of the op, within the tolerance the attention tests use
        ref = ops.paged_decode_reference(q, kc, vc, bt, sl)
        d2 = (got.float() - ref.float()).abs()
        assert d2.max().item() < 0.01 and d2.mean().item() < 0.001
    ops.check_status()


def test_noalloc_decode_rejects_oversize(cuda_device):
    lib = _lib()
    B, Hq, D, splits = 256, 32, 128, 32
    assert lib.rb_paged_decode_noalloc_required_floats(B, Hq, D, splits) > MAX_FLOATS
    q, kc, vc, bt, sl = _case(cuda_device, 2, 32, 8, 128, [64, 64], 3)
    # the size check happens before any pointer is used, so small buffers are fine here
    rc = lib.rb_paged_decode_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(),
                                     q.data_ptr(), B, Hq, 8, D, bt.shape[1], kc.shape[0], 16, splits, 0.1,
                                     ops.status_tensor(cuda_device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == TOO_LARGE
    torch.cuda.synchronize()
    ops.check_status()


def test_noalloc_decode_single_split_uses_no_scratch_and_has_no_size_limit(cuda_device):
    """One split writes the output directly: the entry point asks for none of the internal array, so a shape whose
    split form would not fit is still accepted, and the result equals the regular entry point's."""
    lib = _lib()
    assert lib.rb_paged_decode_noalloc_required_floats(4096, 32, 128, 1) == 0
    assert lib.rb_paged_decode_noalloc_required_floats(4096, 32, 128, 2) > MAX_FLOATS
    q, kc, vc, bt, sl = _case(cuda_device, 5, 14, 2, 64, [300, 17, 512, 1, 96], 11)
    want = ops.paged_decode(q, kc, vc, bt, sl, num_splits=1)
    for _ in range(2):
        rc, got = _call(lib, q, kc, vc, bt, sl, 1)
        assert rc == 0
        torch.cuda.synchronize()
        diff = (got.float() - want.float()).abs()
        assert diff.max().item() < 0.01 and diff.mean().item() < 0.001
    ops.check_status()
