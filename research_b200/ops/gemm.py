"""bf16 GEMM on tcgen05 tensor cores (see csrc/gemm_sm100.cu) and its PyTorch reference.

Replaces the cuBLAS ``F.linear`` calls inside the HF modules the reference runs
(rollouts/inference/engine.py:231, training/backends/pytorch.py:186).
"""

from __future__ import annotations

import ctypes
import functools
import os

import torch

from .. import _native
from ._util import check_rc, ptr, status_tensor, stream_handle

RB_MAX_PARTS = 8
EPI_STORE, EPI_REDUCE_SCATTER, EPI_ALL_REDUCE, EPI_ALL_REDUCE_ONESHOT = 0, 1, 2, 3


class RbGemmArgs(ctypes.Structure):
    """Mirror of ``RbGemmArgs`` in csrc/gemm_sm100.h (field order matters)."""

    _fields_ = [
        ("A", ctypes.c_void_p * RB_MAX_PARTS),
        ("B", ctypes.c_void_p * RB_MAX_PARTS),
        ("C", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("residual", ctypes.c_void_p),
        ("lda", ctypes.c_longlong),
        ("ldb", ctypes.c_longlong),
        ("ldc", ctypes.c_longlong),
        ("ldr", ctypes.c_longlong),
        ("M", ctypes.c_int),
        ("N", ctypes.c_int),
        ("K", ctypes.c_int),
        ("a_parts", ctypes.c_int),
        ("b_parts", ctypes.c_int),
        ("a_mn_major", ctypes.c_int),
        ("b_mn_major", ctypes.c_int),
        ("out_f32", ctypes.c_int),
        ("bn", ctypes.c_int),
        ("max_ctas", ctypes.c_int),
        ("epi_mode", ctypes.c_int),
        ("rank", ctypes.c_int),
        ("world", ctypes.c_int),
        ("a_ready", ctypes.c_void_p),
        ("b_ready", ctypes.c_void_p),
        ("ready_epoch", ctypes.c_int),
        ("reduce_epoch", ctypes.c_int),
        ("stage_ptrs", ctypes.c_void_p * RB_MAX_PARTS),
        ("flag_ptrs", ctypes.c_void_p * RB_MAX_PARTS),
        ("out_ptrs", ctypes.c_void_p * RB_MAX_PARTS),
        ("status", ctypes.c_void_p),
        ("epoch_counter", ctypes.c_void_p),
        ("cta_ticket", ctypes.c_void_p),
        ("stage_parity_bytes", ctypes.c_longlong),
        ("flag_parity_bytes", ctypes.c_longlong),
        ("tile_table", ctypes.c_void_p),
        ("num_tiles_ptr", ctypes.c_void_p),
        ("group_n", ctypes.c_int),
        ("max_tiles", ctypes.c_int),
        ("row_dst", ctypes.c_void_p),
        ("swiglu", ctypes.c_int),
        ("split_k", ctypes.c_int),
        ("splitk_ws", ctypes.c_void_p),
        ("splitk_tickets", ctypes.c_void_p),
        ("scaled_epilogue", ctypes.c_int),
        ("alpha", ctypes.c_float),
        ("beta", ctypes.c_float),
        ("mirror", ctypes.c_int),
        ("fp8", ctypes.c_int),
        ("sample_ws", ctypes.c_void_p),
        ("sample_temperature", ctypes.c_void_p),
        ("sample_seeds", ctypes.c_void_p),
        ("sample_step_ptr", ctypes.c_void_p),
        ("sample_step_add", ctypes.c_ulonglong),
        ("cluster_split", ctypes.c_int),
        ("norm_fold", ctypes.c_int),
        ("norm_eps", ctypes.c_float),
        ("gather_src", ctypes.c_void_p * RB_MAX_PARTS),
        ("gather_dst", ctypes.c_void_p),
        ("gather_part_bytes", ctypes.c_longlong),
        ("gather_count", ctypes.c_void_p),
        ("gather_ready", ctypes.c_void_p),
        ("gather_epoch", ctypes.c_int),
        ("gather_parts", ctypes.c_int),
        ("b_part_rot", ctypes.c_int),
        ("ready_epoch_ptr", ctypes.c_void_p),
        ("gather_src_ready", ctypes.c_void_p),
        ("gather_wait_all", ctypes.c_int),
        ("group_mode", ctypes.c_int),
        ("group_b_rows", ctypes.c_int),
    ]


def _lib() -> ctypes.CDLL:
    lib = _native.load("rb_gemm")
    if not getattr(lib, "_rb_typed", False):
        lib.rb_gemm_bf16_ex.argtypes = [ctypes.POINTER(RbGemmArgs), ctypes.c_void_p]
        lib.rb_gemm_bf16_ex.restype = ctypes.c_int
        lib.rb_sample_merge.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.rb_sample_merge.restype = ctypes.c_int
        lib._rb_typed = True
    return lib


def _lib2() -> ctypes.CDLL:
    lib = _native.load("rb_gemm2")
    if not getattr(lib, "_rb_typed", False):
        vp, i, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.rb_gemm2_bf16.argtypes = [vp] * 5 + [i, i, i, ll, ll, ll, ll, i, i, i, i, vp, vp]
        lib.rb_gemm2_bf16.restype = i
        lib.rb_gemm2_pairs.restype = i
        lib.rb_gemm2_bf16_gather.argtypes = ([vp] * 5 + [i, i, i, ll, ll, ll, ll, i, i, i] +
                                             [ctypes.POINTER(vp), vp, ll, vp, vp, i, i, i, i, i, vp, vp])
        lib.rb_gemm2_bf16_gather.restype = i
        lib._rb_typed = True
    return lib


_GEMM2 = os.environ.get("RB_GEMM2", "1") != "0"
_GEMM2_GATHER = os.environ.get("RB_GEMM2_GATHER", "1") != "0"     # gather-carrying launches on the two-CTA kernel too
_GATHER_CHUNKS = int(os.environ.get("RB_GATHER_CHUNKS", "8"))      # pieces a gathered part is published in (tiles start per piece)
_GEMM2_PAIRS = 74      # CTA pairs resident on a B200 (148 SMs)


def _use_pair_kernel(M: int, N: int, K: int, a_mn_major: bool, b_mn_major: bool) -> bool:
    """Large problems go to the two-CTA kernel (csrc/gemm2_sm100.cu): at least one full wave of 256-row tiles and a
    K loop long enough to amortise a tile's prologue. Small or skinny problems stay on the one-CTA kernel, which has
    the narrow tiles and the split-K forms they need."""
    if not _GEMM2 or (a_mn_major and not b_mn_major) or N % 8 or K < 256 or M < 512:
        return False
    if not (a_mn_major and b_mn_major) and K % 8:
        return False
    return -(-M // 256) * -(-N // 128) >= _GEMM2_PAIRS


def gemm2(a: torch.Tensor, b: torch.Tensor, bias=None, residual=None, out=None, *, a_mn_major=False, b_mn_major=False,
          out_f32=False, bn: int = 0) -> torch.Tensor:
    """``C = op(A) @ op(B)^T (+bias) (+residual)`` on the two-CTA (``cta_group::2``) kernel; same operand conventions
    as ``gemm``. ``bn``: 256 or 128 output columns per tile (0 = fewest waves)."""
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    K, M = a.shape if a_mn_major else a.shape[::-1]
    Kb, N = b.shape if b_mn_major else b.shape[::-1]
    assert K == Kb, f"K mismatch: {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    assert out.stride(1) == 1 and (residual is None or residual.stride(1) == 1)
    rc = _lib2().rb_gemm2_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), bias.data_ptr() if bias is not None else None,
                               residual.data_ptr() if residual is not None else None, M, N, K, a.stride(0), b.stride(0),
                               out.stride(0), residual.stride(0) if residual is not None else 0, int(a_mn_major),
                               int(b_mn_major), int(out_f32), bn, status_tensor(a.device).data_ptr(), stream_handle(a.device))
    check_rc(rc, "rb_gemm2_bf16")
    return out


def _gemm2_gather(a, b, bias, residual, out, M, N, K, mn_major: bool, out_f32: bool, gather, consume: bool) -> torch.Tensor:
    """A gather-carrying launch on the two-CTA kernel (``rb_gemm2_bf16_gather``): forward (K-major operands, the
    gathered matrix consumed as B) or weight gradient (both MN-major, the gather only carried)."""
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    W = gather.world
    src = (ctypes.c_void_p * 8)(*[gather.peer_ptrs[r] for r in range(W)])
    rc = _lib2().rb_gemm2_bf16_gather(
        a.data_ptr(), None if consume else b.data_ptr(), out.data_ptr(), bias.data_ptr() if bias is not None else None,
        residual.data_ptr() if residual is not None else None, M, N, K, a.stride(0), K if consume else b.stride(0), out.stride(0),
        residual.stride(0) if residual is not None else 0, int(mn_major), int(mn_major), int(out_f32), src,
        gather.b.stage.data_ptr(), gather.part_bytes, gather.b.gather_count.data_ptr(), gather.b.gather_ready.data_ptr(),
        gather.next_epoch(), W, gather.rank, int(consume), _GATHER_CHUNKS, status_tensor(a.device).data_ptr(), stream_handle(a.device))
    check_rc(rc, "rb_gemm2_bf16_gather")
    return out


def gemm_reference(a, b, bias=None, residual=None, a_mn_major=False, b_mn_major=False, out_dtype=None):
    """fp32 PyTorch reference: ``op(a) @ op(b).T`` (+bias) (+residual)."""
    af = a.float().t() if a_mn_major else a.float()
    bf = b.float().t() if b_mn_major else b.float()
    c = af @ bf.t()
    if bias is not None:
        c = c + bias.float()
    if residual is not None:
        c = c + residual.float()
    return c.to(out_dtype or a.dtype)


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    *,
    a_mn_major: bool = False,
    b_mn_major: bool = False,
    out_f32: bool = False,
    bn: int = 0,
    max_ctas: int = 0,
    swiglu: bool = False,
    split_k: int = 0,
    alpha: float = 1.0,
    beta: float = 1.0,
    cluster_split: bool | None = None,
    norm_eps: float | None = None,
    b_gather=None,
    carry_gather=None,
    wait_flag: tuple[int, int] | None = None,
) -> torch.Tensor:
    """``C[M,N] = alpha * op(A) @ op(B)^T (+bias) (+ beta * residual)``.

    Sharded parameters (``parallel.fsdp.ShardedWeight`` handles): with ``b_gather=w`` (pass ``b=None``) the K-major B
    operand is the row-sharded matrix ``w``; the launch itself gathers the peers' slabs into the local staging matrix
    and its tiles start part by part as the slabs land (all-gather fused into the consuming GEMM). With
    ``carry_gather=w`` the launch computes its own, unrelated product and fetches ``w`` on the side for the launch
    that follows (the weight-gradient GEMM carries the gather for the data-gradient GEMM).

    ``wait_flag=(flag_address, value_address)``: the launch's tile producers wait (bounded) until the int at
    ``flag_address`` has reached the int at ``value_address`` before their first load, and so before anything is stored:
    a launch that overwrites a buffer other GPUs read waits for their acknowledgements this way, inside the launch.

    ``norm_eps`` folds an RMSNorm of A's rows into the launch: ``C = rstd(row) * (A @ B^T) (+bias)`` with
    ``rstd = rsqrt(mean(A[row]^2) + norm_eps)``; together with the norm weight multiplied into B's columns
    beforehand this equals ``rmsnorm(A) @ B^T`` without a separate normalisation pass.

    K-major operands are ``[rows, K]`` row-major (a torch ``Linear`` weight is a K-major B);
    MN-major operands are ``[K, rows]`` row-major. On CUDA this launches the tcgen05 kernel;
    on CPU it evaluates the fp32 reference (used as the oracle in tests).
    """
    if swiglu:
        assert bn >= 64 and not (a_mn_major or b_mn_major), "fused SwiGLU needs an explicit bn and K-major operands"
    if norm_eps is not None:
        assert not a_mn_major and split_k in (0, 1) and alpha == 1.0 and beta == 1.0, "folded RMSNorm: K-major A, no split"
        split_k = 1
    if b_gather is not None:
        assert b is None and not b_mn_major and not a_mn_major, "the gathered operand is a K-major B"
        if not a.is_cuda:
            b = b_gather.b.full_param(b_gather.spec.name)
            b_gather = None
    if not a.is_cuda:
        carry_gather = None
        if norm_eps is not None:
            af = a.float()
            a = (af * torch.rsqrt(af.pow(2).mean(-1, keepdim=True) + norm_eps)).to(a.dtype)
        if alpha != 1.0 or beta != 1.0:
            res = alpha * gemm_reference(a, b, None, None, a_mn_major, b_mn_major, torch.float32)
            if bias is not None:
                res = res + bias.float()
            if residual is not None:
                res = res + beta * residual.float()
            res = res.to(torch.float32 if out_f32 else a.dtype)
        else:
            res = gemm_reference(a, b, bias, residual, a_mn_major, b_mn_major, torch.float32 if out_f32 else None)
        if swiglu:
            res = swiglu_interleaved_reference(res, bn)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if b_gather is not None:
        b = b_gather.staged          # [rows, cols] view of the staging matrix this launch fills
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1, "operands must be contiguous in their last dim"
    if a_mn_major:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn_major:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"K mismatch: {K} vs {Kb}"
    gather = b_gather if b_gather is not None else carry_gather
    if (gather is None and wait_flag is None and not swiglu and norm_eps is None and alpha == 1.0 and beta == 1.0 and bn == 0 and max_ctas == 0 and split_k in (0, 1)
            and not cluster_split and _use_pair_kernel(M, N, K, a_mn_major, b_mn_major)):
        return gemm2(a, b, bias, residual, out, a_mn_major=a_mn_major, b_mn_major=b_mn_major, out_f32=out_f32)
    if (gather is not None and _GEMM2_GATHER and wait_flag is None and not swiglu and norm_eps is None and alpha == 1.0 and beta == 1.0
            and bn == 0 and max_ctas == 0 and split_k in (0, 1) and not cluster_split and a_mn_major == b_mn_major
            and _use_pair_kernel(M, N, K, a_mn_major, b_mn_major)
            and (b_gather is None or (N % gather.world == 0 and (N // gather.world) % 256 == 0))):
        return _gemm2_gather(a, b, bias, residual, out, M, N, K, a_mn_major, out_f32, gather, b_gather is not None)
    if out is None:
        out = torch.empty(M, N // 2 if swiglu else N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    assert out.stride(1) == 1
    args = RbGemmArgs()
    args.A[0] = a.data_ptr()
    args.B[0] = b.data_ptr()
    args.C = out.data_ptr()
    args.bias = bias.data_ptr() if bias is not None else None
    args.residual = residual.data_ptr() if residual is not None else None
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), out.stride(0)
    args.ldr = residual.stride(0) if residual is not None else 0
    args.M, args.N, args.K = M, N, K
    args.a_parts = args.b_parts = 1
    args.a_mn_major, args.b_mn_major = int(a_mn_major), int(b_mn_major)
    args.out_f32 = int(out_f32)
    args.bn = bn
    args.max_ctas = max_ctas
    args.epi_mode = EPI_STORE
    args.rank, args.world = 0, 1
    args.swiglu = int(swiglu)
    if norm_eps is not None:
        args.norm_fold, args.norm_eps = 1, float(norm_eps)
    if gather is not None:
        assert not swiglu and norm_eps is None and alpha == 1.0 and beta == 1.0 and split_k in (0, 1), "gather launches are plain GEMMs"
        split_k = 1
        W = gather.world
        for r in range(W):
            args.gather_src[r] = gather.peer_ptrs[r]
        args.gather_dst = gather.b.stage.data_ptr()
        args.gather_part_bytes = gather.part_bytes
        args.gather_count = gather.b.gather_count.data_ptr()
        args.gather_ready = gather.b.gather_ready.data_ptr()
        args.gather_epoch = gather.next_epoch()
        args.gather_parts = W
        args.rank = gather.rank
        if b_gather is not None:          # consumed by this launch: B is the staging matrix, part by part
            args.b_parts = W
            for r in range(W):
                args.B[r] = args.gather_dst + r * gather.part_bytes
            args.b_ready = args.gather_ready
            args.ready_epoch = args.gather_epoch
            args.b_part_rot = gather.rank
    if alpha != 1.0 or beta != 1.0:
        assert not swiglu, "the scaled epilogue is not combined with the fused SwiGLU"
        args.scaled_epilogue, args.alpha, args.beta = 1, alpha, beta
        split_k = 1
    if split_k == 0:
        split_k, auto_bn = _auto_split_k(M, N, K, swiglu or bn != 0, 64 if b_mn_major else 32)
        if auto_bn:
            args.bn = auto_bn
    if cluster_split is None:
        # slices as one thread-block cluster (partials meet in distributed shared memory) whenever the shape allows
        cluster_split = (split_k in (2, 4, 8) and args.bn in (32, 64, 128, 256) and args.bn // split_k >= 8 and not swiglu
                         and (-(-K // 64)) > (split_k - 1) * (-(-(-(-K // 64)) // split_k)) and _SPLITK_MODE != "l2")
    if split_k > 1 and cluster_split:
        args.split_k, args.cluster_split = split_k, 1
    elif split_k > 1:
        # one [128 x bn] fp32 tile per (output tile, K slice); padded for the widest tile the kernel may pick
        ws, tickets = _splitk_scratch(a.device, split_k * (-(-M // 128) * 128) * (-(-N // 256) * 256), (-(-M // 128)) * (-(-N // 32)))
        args.split_k, args.splitk_ws, args.splitk_tickets = split_k, ws.data_ptr(), tickets.data_ptr()
    if wait_flag is not None:
        assert gather is None, "a launch waits either for a gather's parts or for a flag"
        args.a_ready, args.ready_epoch_ptr = wait_flag
    args.status = status_tensor(a.device).data_ptr()
    rc = _lib().rb_gemm_bf16_ex(ctypes.byref(args), stream_handle(a.device))
    check_rc(rc, "rb_gemm_bf16_ex")
    return out


_SPLITK: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
_SPLITK_MODE = os.environ.get("RB_SPLITK_MODE", "cluster")   # "l2" keeps the workspace + ticket reduction


def _auto_split_k(M: int, N: int, K: int, excluded: bool, min_bn: int = 32) -> tuple[int, int]:
    """Tile width and K split for problems with few output tiles and a long K (decode-sized GEMMs, weight gradients
    of narrow projections): returns ``(split, bn)``, ``(1, 0)`` = leave it to the kernel.

    These launches are bound by what one SM can pull from L2 (about 80 GB/s measured): a CTA streams
    ``(128 + bn) * 128`` bytes per k-block, and with narrow tiles or few tiles most of the 148 SMs idle. Splitting
    K inside a thread-block cluster (the slices exchange partial tiles through distributed shared memory) fills
    the machine without a workspace round trip. The choice minimises a small cost model fitted to B200
    timings with weights streamed from HBM (M=256): N=896,K=4864 29.1 us unsplit -> 18.7 (bn 64, 4 slices);
    N=4096,K=14336 74.6 -> 54.5 (bn 128, 2 slices); K <= 896 is never split (12.2 us either way)."""
    if excluded or N % 8 or os.environ.get("RB_NO_SPLITK") or -(-M // 128) * -(-N // 256) > 74:
        return 1, 0       # more than half a wave of the widest tiles: nothing to gain from a split
    if _SPLITK_MODE == "l2":
        return _auto_split_k_workspace(M, N, K) if M <= 256 and min_bn == 32 else (1, 0)
    return _cluster_split_choice(M, N, K, min_bn)


_STREAM_GBS = {32: 80e3, 64: 85e3, 128: 98e3, 256: 114e3}     # bytes per microsecond one SM pulls from L2, by tile width


@functools.lru_cache(maxsize=4096)
def _cluster_split_choice(M: int, N: int, K: int, min_bn: int = 32) -> tuple[int, int]:
    """Cheapest (split, bn) under a model fitted to 100 timed B200 launches (mean error 10 %): per k-block a CTA
    streams ``(128 + bn) * 128`` bytes at the per-SM rate above; a cluster reduction costs 1 + 0.045 bn (2 slices),
    1.5 + 0.025 bn (4) or 3 + 0.03 bn microseconds (8); split launches must fit one wave."""
    m_tiles = -(-M // 128)
    num_kb = -(-K // 64)
    best = None
    for bn in (256, 128, 64, 32):
        if (bn > 32 and N < bn) or bn < min_bn:
            continue
        n_tiles = -(-N // bn)
        stage_us = (128 + bn) * 128 / _STREAM_GBS[bn]
        mma_us = 128 * bn * 64 * 2 / 8.0e6
        for s in (1, 2, 4, 8):
            per = -(-num_kb // s)
            if s > 1 and (bn // s < 8 or per < 4 or (s - 1) * per >= num_kb):
                continue
            units = m_tiles * n_tiles * s
            grid = min(units, 148 - 148 % s)
            if s > 1 and units > grid:
                continue
            waves = -(-units // grid)
            red = {1: 0.0, 2: 1 + 0.045 * bn, 4: 1.5 + 0.025 * bn, 8: 3 + 0.03 * bn}[s]
            cost = waves * (per * max(stage_us, mma_us) + 1.0 + red)
            if best is None or cost < best[0] - 0.5:
                best = (cost, s, bn)
    if best is None or best[1] == 1:
        return 1, 0
    return best[1], best[2]


def _auto_split_k_workspace(M: int, N: int, K: int) -> tuple[int, int]:
    """Choice for the workspace + ticket reduction (RB_SPLITK_MODE=l2): most CTAs within one wave, at least 1024 of
    K per slice, N < 2048 only (wider outputs measured slower inside the decode graph)."""
    if K < 3072 or N >= 2048:
        return 1, 0
    m_tiles = -(-M // 128)
    best = None
    for bn in (256, 128, 64, 32):
        if bn > 32 and N < bn:
            continue
        tiles = m_tiles * (-(-N // bn))
        for s in (1, 2, 4, 8):
            if tiles * s > 148 or (s > 1 and K // s < 1024):
                continue
            key = (tiles * s, bn)
            if best is None or key > best[0]:
                best = (key, bn, s)
    if best is None:
        return 1, 0
    return best[2], best[1]


def _splitk_scratch(device: torch.device, floats: int, tiles: int) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 partial-tile workspace and per-tile ticket counters, one growing pair per device.
    Kernels on one stream run in order, so the pair is shared by all split-K launches of that stream."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    cur = _SPLITK.get(idx)
    if cur is None or cur[0].numel() < floats or cur[1].numel() < tiles:
        ws = torch.empty(max(floats, cur[0].numel() if cur else 0, 1 << 22), dtype=torch.float32, device=device)
        tk = torch.zeros(max(tiles, cur[1].numel() if cur else 0, 4096), dtype=torch.int32, device=device)
        _SPLITK[idx] = (ws, tk)
    return _SPLITK[idx]


def gemm_fp8(a: torch.Tensor, b: torch.Tensor, scale: float = 1.0, bias=None, out: torch.Tensor | None = None,
             out_f32: bool = False, bn: int = 0) -> torch.Tensor:
    """``C = scale * A @ B^T`` for ``float8_e4m3fn`` / ``float8_e5m2`` operands ``A [M,K]``, ``B [N,K]``
    (fp32 accumulation on the tcgen05 ``kind::f8f6f4`` path, bf16 or fp32 output). ``scale`` is the
    product of the per-tensor scales, as with ``torch._scaled_mm`` (dev/speedrun/single-file.py:35-96)."""
    f8 = (torch.float8_e4m3fn, torch.float8_e5m2)
    assert a.dtype in f8 and b.dtype in f8 and a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1]
    M, K = a.shape
    N = b.shape[0]
    if not a.is_cuda:
        res = scale * (a.float() @ b.float().T)
        if bias is not None:
            res = res + bias.float()
        res = res.to(torch.float32 if out_f32 else torch.bfloat16)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert K % 16 == 0 and a.stride(1) == 1 and b.stride(1) == 1 and a.stride(0) % 16 == 0 and b.stride(0) % 16 == 0
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    args = RbGemmArgs()
    args.A[0], args.B[0], args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.bias = bias.data_ptr() if bias is not None else None
    # described as bf16 matrices with half as many columns: same bytes, see RbGemmArgs.fp8
    args.lda, args.ldb, args.ldc = a.stride(0) // 2, b.stride(0) // 2, out.stride(0)
    args.M, args.N, args.K = M, N, K // 2
    args.a_parts = args.b_parts = 1
    args.out_f32 = int(out_f32)
    args.bn = bn
    args.epi_mode = EPI_STORE
    args.rank, args.world = 0, 1
    args.fp8 = 1 | (2 if a.dtype == torch.float8_e5m2 else 0) | (4 if b.dtype == torch.float8_e5m2 else 0)
    if scale != 1.0:
        args.scaled_epilogue, args.alpha, args.beta = 1, scale, 1.0
    args.status = status_tensor(a.device).data_ptr()
    rc = _lib().rb_gemm_bf16_ex(ctypes.byref(args), stream_handle(a.device))
    check_rc(rc, "rb_gemm_bf16_ex(fp8)")
    return out


def quantize_fp8(x: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn) -> tuple[torch.Tensor, float]:
    """Per-tensor scaled cast: returns ``(x / s as fp8, s)`` with ``s = amax / fp8_max``."""
    fmax = torch.finfo(dtype).max
    s = max(x.abs().max().item() / fmax, 1e-12)
    return (x.float() / s).clamp(-fmax, fmax).to(dtype), s


SAMPLE_BN = 256     # tile width of the fused lm_head + sampling launch


def lm_head_sample_workspace(M: int, V: int, device) -> torch.Tensor:
    return torch.empty(M * (-(-V // SAMPLE_BN)) * 8, dtype=torch.float32, device=device)


def lm_head_sample(h: torch.Tensor, w: torch.Tensor, temperatures: torch.Tensor, seeds: torch.Tensor, step: int = 0,
                   step_tensor: torch.Tensor | None = None, out_tokens=None, out_logprobs=None, workspace=None):
    """Sample one token per row of ``h [M, K]`` from ``softmax(h @ w.T / T)`` and return its log-probability
    under the unscaled logits, without materialising the ``[M, V]`` logits: the GEMM epilogue reduces every
    tile to a small record and a merge kernel finishes. Same random stream as ``sample_with_logprobs``."""
    M, K = h.shape
    V = w.shape[0]
    if not h.is_cuda:
        from .sampling import sample_with_logprobs

        return sample_with_logprobs(gemm_reference(h, w, None, None, False, False, torch.float32), temperatures, seeds, step)
    assert h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and temperatures.dtype == torch.float32
    if out_tokens is None:
        out_tokens = torch.empty(M, dtype=torch.int32, device=h.device)
    if out_logprobs is None:
        out_logprobs = torch.empty(M, dtype=torch.float32, device=h.device)
    if workspace is None:
        workspace = lm_head_sample_workspace(M, V, h.device)
    n_tiles = -(-V // SAMPLE_BN)
    assert workspace.numel() >= M * n_tiles * 8
    args = RbGemmArgs()
    args.A[0], args.B[0] = h.data_ptr(), w.data_ptr()
    args.C = workspace.data_ptr()          # unused by the sampling epilogue, must be a valid pointer
    args.lda, args.ldb, args.ldc = h.stride(0), w.stride(0), V
    args.M, args.N, args.K = M, V, K
    args.a_parts = args.b_parts = 1
    args.out_f32 = 1
    args.bn = SAMPLE_BN
    args.epi_mode = EPI_STORE
    args.rank, args.world = 0, 1
    args.sample_ws = workspace.data_ptr()
    args.sample_temperature = temperatures.data_ptr()
    args.sample_seeds = seeds.data_ptr()
    args.sample_step_ptr = step_tensor.data_ptr() if step_tensor is not None else None
    args.sample_step_add = step
    args.status = status_tensor(h.device).data_ptr()
    check_rc(_lib().rb_gemm_bf16_ex(ctypes.byref(args), stream_handle(h.device)), "rb_gemm_bf16_ex(sample)")
    check_rc(_lib().rb_sample_merge(workspace.data_ptr(), M, n_tiles, out_tokens.data_ptr(), out_logprobs.data_ptr(),
                                    stream_handle(h.device)), "rb_sample_merge")
    return out_tokens, out_logprobs


_SYM_TABLES: dict[tuple, tuple[torch.Tensor, torch.Tensor, int]] = {}


def _symmetric_tiles(M: int, bn: int, device: torch.device) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Tile table (first A row, valid rows, first B row, first output column) of the tiles that touch
    the lower triangle of an M x M output."""
    key = (M, bn, device.index)
    if key not in _SYM_TABLES:
        rows = [(mt * 128, min(128, M - mt * 128), nt * bn, nt * bn)
                for mt in range(-(-M // 128)) for nt in range(-(-M // bn)) if nt * bn < min((mt + 1) * 128, M)]
        # longest rows of tiles first: the persistent CTAs then finish together
        table = torch.tensor(rows, dtype=torch.int32, device=device)
        count = torch.tensor([len(rows)], dtype=torch.int32, device=device)
        _SYM_TABLES[key] = (table, count, len(rows))
    return _SYM_TABLES[key]


def gemm_symmetric(a: torch.Tensor, alpha: float = 1.0, beta: float = 0.0, residual: torch.Tensor | None = None,
                   out: torch.Tensor | None = None, bn: int = 128) -> torch.Tensor:
    """``C = alpha * A @ A^T + beta * residual`` for ``A [M, K]``; ``residual`` must be symmetric.

    Only the output tiles that touch the lower triangle are computed (a device tile table drives the
    grouped mode of the GEMM kernel); the epilogue writes every element below the diagonal to its
    transposed position as well. Covers the ``A A^T`` and ``b A + c A A`` products of the Muon /
    Polar Express orthogonalisation (dev/speedrun/single-file.py:172-383)."""
    M, K = a.shape
    if not a.is_cuda:
        res = alpha * (a.float() @ a.float().T)
        if residual is not None:
            res = res + beta * residual.float()
        res = res.to(a.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert a.dtype == torch.bfloat16 and a.stride(1) == 1 and M % 8 == 0 and K % 8 == 0
    if out is None:
        out = torch.empty(M, M, dtype=torch.bfloat16, device=a.device)
    table, count, n_tiles = _symmetric_tiles(M, bn, a.device)
    args = RbGemmArgs()
    args.A[0] = args.B[0] = a.data_ptr()
    args.C = out.data_ptr()
    args.residual = residual.data_ptr() if residual is not None else None
    args.lda = args.ldb = a.stride(0)
    args.ldc = out.stride(0)
    args.ldr = residual.stride(0) if residual is not None else 0
    args.M, args.N, args.K = M, M, K
    args.a_parts = args.b_parts = 1
    args.bn = bn
    args.epi_mode = EPI_STORE
    args.rank, args.world = 0, 1
    args.tile_table, args.num_tiles_ptr = table.data_ptr(), count.data_ptr()
    args.group_n, args.max_tiles = M, n_tiles
    args.scaled_epilogue, args.alpha, args.beta = 1, alpha, beta
    args.mirror = 1
    args.status = status_tensor(a.device).data_ptr()
    rc = _lib().rb_gemm_bf16_ex(ctypes.byref(args), stream_handle(a.device))
    check_rc(rc, "rb_gemm_bf16_ex(symmetric)")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, bn: int) -> torch.Tensor:
    """Pack ``gate`` and ``up`` ``[F, K]`` for the fused SwiGLU epilogue: blocks of ``bn/2`` gate rows
    followed by the matching ``bn/2`` up rows."""
    F, K = gate.shape
    h = bn // 2
    assert F % h == 0, f"F={F} must be a multiple of {h}"
    return torch.stack([gate.view(F // h, h, K), up.view(F // h, h, K)], dim=1).reshape(2 * F, K).contiguous()


def swiglu_interleaved_reference(y: torch.Tensor, bn: int) -> torch.Tensor:
    """``silu(gate) * up`` for GEMM output whose columns are interleaved as ``interleave_gate_up`` packs them."""
    M, N2 = y.shape
    h = bn // 2
    yv = y.view(M, N2 // bn, 2, h)
    return (torch.nn.functional.silu(yv[:, :, 0]) * yv[:, :, 1]).reshape(M, N2 // 2)


def linear(x: torch.Tensor, weight: torch.Tensor, bias=None, residual=None, out=None, out_f32=False):
    """``x @ weight.T`` for ``x`` of shape ``[..., K]`` and ``weight`` ``[N, K]``."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    r2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
    y = gemm(x2, weight, bias, r2, out, out_f32=out_f32)
    return y.reshape(*lead, weight.shape[0])


__all__ = ["gemm", "gemm2", "lm_head_sample", "lm_head_sample_workspace", "gemm_fp8", "quantize_fp8", "gemm_symmetric", "gemm_reference", "linear", "interleave_gate_up", "swiglu_interleaved_reference", "RbGemmArgs", "EPI_STORE", "EPI_REDUCE_SCATTER", "EPI_ALL_REDUCE", "EPI_ALL_REDUCE_ONESHOT"]
_ = ptr  # re-exported helper kept for wrappers that build RbGemmArgs themselves
