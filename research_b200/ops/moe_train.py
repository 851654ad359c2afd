"""Mixture-of-experts MLP for training as grouped tcgen05 GEMMs: forward, data gradients and weight gradients of ALL
experts of a layer run as six grouped launches over expert-sorted rows, with no host synchronisation.

The (token, slot) pairs are sorted by expert on the device; every expert's row range is padded with zero rows to a
multiple of 64, so the weight gradient ``dW_e = dY_e^T X_e`` is one grouped launch whose contraction runs over the
expert's row range (a 64-row k-block never straddles two experts). Rows keep the token order inside an expert, so the
result does not depend on scheduling.

Math of the per-expert loop in the reference's functional models
(rollouts/tools/functional_extractor/glm4_moe_functional.py:230-369: route, loop over experts, ``index_add_``);
``grouped_experts_reference`` below is that loop in fp32 and serves as the oracle and the CPU path.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _native
from . import elementwise as _ew
from ._util import check_rc, status_tensor, stream_handle
from .gemm import EPI_STORE, RbGemmArgs, _lib as _gemm_lib

_LIB = None
_I, _VP = ctypes.c_int, ctypes.c_void_p


def _lib():
    global _LIB
    if _LIB is None:
        lib = _native.load("rb_moe")
        lib.rb_moe_count.argtypes = [_VP, _I, _I, _VP, _VP]
        lib.rb_moe_train_plan.argtypes = [_VP, _I, _VP, ctypes.POINTER(_I), ctypes.POINTER(_VP), ctypes.POINTER(_VP), _I, _I, _I, _VP, _VP]
        lib.rb_moe_train_rows.argtypes = [_VP, _I, _I, _VP, _VP, _VP, _VP]
        lib.rb_moe_train_gather.argtypes = [_VP, _VP, _VP, _VP, _I, _I, _I, _VP, _VP]
        lib.rb_moe_train_combine.argtypes = [_VP, _VP, _VP, _I, _I, _I, _VP, _VP]
        lib.rb_moe_train_dot.argtypes = [_VP, _VP, _VP, _I, _I, _I, _VP, _VP]
        for f in ("rb_moe_count", "rb_moe_train_plan", "rb_moe_train_rows", "rb_moe_train_gather", "rb_moe_train_combine", "rb_moe_train_dot"):
            getattr(lib, f).restype = _I
        _LIB = lib
    return _LIB


MAX_EXPERTS = 256
FWD_GU, FWD_DN, DGRAD_DN, DGRAD_GU, WGRAD_DN, WGRAD_GU = range(6)


def _tile_width(n: int) -> int:
    return 256 if n >= 256 else 128 if n >= 128 else 64


class GroupedPlan:
    """Row layout and tile tables of one MoE layer call, all on the device.

    ``idx`` ``[T, k]`` (int32) are the chosen experts. ``row_of[t * k + j]`` is the row of pair ``(t, j)`` in the
    expert-sorted matrices, ``src_of[row]`` its inverse (-1 for padding rows), ``offsets[e]`` the first row of expert
    ``e`` and ``offsets[E]`` the rows in use. ``cap`` is the fixed row capacity ``ceil64(T k) + 64 E`` the buffers
    are allocated with (the row count in use is only known on the device)."""

    def __init__(self, idx: torch.Tensor, E: int, d: int, F: int):
        assert idx.dtype == torch.int32 and idx.is_cuda and idx.is_contiguous() and E <= MAX_EXPERTS
        assert d % 64 == 0 and F % 32 == 0
        dev = idx.device
        self.T, self.k = idx.shape
        self.E, self.d, self.F, self.device = E, d, F, dev
        n = self.T * self.k
        self.n_pairs = n
        self.cap = -(-n // 64) * 64 + 64 * E
        lib, s = _lib(), stream_handle(dev)
        st = status_tensor(dev).data_ptr()
        self.counts = torch.zeros(E, dtype=torch.int32, device=dev)
        check_rc(lib.rb_moe_count(idx.data_ptr(), n, E, self.counts.data_ptr(), s), "rb_moe_count")
        # (mode, output columns per expert, tile width, rows of the stacked B per expert | output rows per expert)
        self.desc = [(0, 2 * F, _tile_width(2 * F), 2 * F), (0, d, _tile_width(d), d),
                     (1, F, _tile_width(F), d), (1, d, _tile_width(d), 2 * F),
                     (2, F, _tile_width(F), d), (2, d, _tile_width(d), 2 * F)]
        m_tiles = self.cap // 128 + E
        sizes = []
        for mode, n_total, bn, bs in self.desc:
            nt = -(-n_total // bn)
            sizes.append((E * -(-bs // 128) if mode == 2 else m_tiles) * nt)
        self.max_tiles = max(sizes)
        self.tiles = torch.empty(6, self.max_tiles, 4, dtype=torch.int32, device=dev)
        self.ntiles = torch.zeros(6, dtype=torch.int32, device=dev)
        self.offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        flat = (_I * 24)(*[v for dsc in self.desc for v in dsc])
        tptr = (_VP * 6)(*[self.tiles[i].data_ptr() for i in range(6)])
        nptr = (_VP * 6)(*[self.ntiles.data_ptr() + 4 * i for i in range(6)])
        check_rc(lib.rb_moe_train_plan(self.counts.data_ptr(), E, self.offsets.data_ptr(), flat, tptr, nptr, 6, self.max_tiles,
                                       self.cap, st, s), "rb_moe_train_plan")
        self.row_of = torch.empty(n, dtype=torch.int32, device=dev)
        self.src_of = torch.empty(self.cap, dtype=torch.int32, device=dev)
        check_rc(lib.rb_moe_train_rows(idx.data_ptr(), n, E, self.offsets.data_ptr(), self.row_of.data_ptr(),
                                       self.src_of.data_ptr(), s), "rb_moe_train_rows")

    # ---------------------------------------------------------------- token movement
    def gather(self, src: torch.Tensor, w: torch.Tensor | None = None) -> torch.Tensor:
        """``out[row] = (w[pair] if w else 1) * src[token of row]`` for the rows in use, zeros in the padding rows."""
        assert src.dtype == torch.bfloat16 and src.is_contiguous() and src.shape == (self.T, src.shape[1])
        cols = src.shape[1]
        out = torch.empty(self.cap, cols, dtype=torch.bfloat16, device=self.device)
        wp = None
        if w is not None:
            assert w.dtype == torch.float32 and w.is_contiguous() and w.numel() == self.n_pairs
            wp = w.data_ptr()
        check_rc(_lib().rb_moe_train_gather(src.data_ptr(), wp, self.src_of.data_ptr(), self.offsets.data_ptr() + 4 * self.E, self.cap,
                                            self.k, cols, out.data_ptr(), stream_handle(self.device)), "rb_moe_train_gather")
        return out

    def combine(self, y: torch.Tensor, w: torch.Tensor | None = None) -> torch.Tensor:
        """``out[t] = sum_j (w[t, j] if w else 1) * y[row_of[t, j]]``."""
        assert y.dtype == torch.bfloat16 and y.is_contiguous() and y.shape[0] == self.cap
        cols = y.shape[1]
        out = torch.empty(self.T, cols, dtype=torch.bfloat16, device=self.device)
        wp = None
        if w is not None:
            assert w.dtype == torch.float32 and w.is_contiguous() and w.numel() == self.n_pairs
            wp = w.data_ptr()
        check_rc(_lib().rb_moe_train_combine(y.data_ptr(), wp, self.row_of.data_ptr(), self.T, self.k, cols, out.data_ptr(),
                                             stream_handle(self.device)), "rb_moe_train_combine")
        return out

    def dot(self, g: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """``dw[t, j] = <g[t], y[row_of[t, j]]>`` (fp32): the gradient of the combine weights."""
        assert g.is_contiguous() and y.is_contiguous() and g.shape[1] == y.shape[1]
        dw = torch.empty(self.T, self.k, dtype=torch.float32, device=self.device)
        check_rc(_lib().rb_moe_train_dot(g.data_ptr(), y.data_ptr(), self.row_of.data_ptr(), self.n_pairs, self.k, g.shape[1],
                                         dw.data_ptr(), stream_handle(self.device)), "rb_moe_train_dot")
        return dw

    # ---------------------------------------------------------------- grouped GEMMs
    def _launch(self, which: int, a, b, c, *, M, N, K, group_n, a_mn, b_mn, group_mode, group_b_rows=0, residual=None) -> None:
        args = RbGemmArgs()
        args.A[0], args.B[0], args.C = a.data_ptr(), b.data_ptr(), c.data_ptr()
        args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), c.stride(0)
        args.M, args.N, args.K = M, N, K
        args.a_parts = args.b_parts = 1
        args.a_mn_major, args.b_mn_major = int(a_mn), int(b_mn)
        args.bn = self.desc[which][2]
        args.epi_mode = EPI_STORE
        args.rank, args.world = 0, 1
        args.status = status_tensor(self.device).data_ptr()
        args.tile_table, args.num_tiles_ptr = self.tiles[which].data_ptr(), self.ntiles.data_ptr() + 4 * which
        args.group_n, args.max_tiles = group_n, self.max_tiles
        args.group_mode, args.group_b_rows = group_mode, group_b_rows
        if residual is not None:
            args.residual, args.ldr = residual.data_ptr(), residual.stride(0)
        check_rc(_gemm_lib().rb_gemm_bf16_ex(ctypes.byref(args), stream_handle(self.device)), "rb_gemm_bf16_ex(grouped training)")

    def forward(self, which: int, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``out[rows of e] = x[rows of e] @ w_e^T`` with ``w`` the experts' ``[n, K]`` matrices stacked along the rows."""
        n = self.desc[which][1]
        out = torch.empty(self.cap, n, dtype=torch.bfloat16, device=self.device)
        self._launch(which, x, w, out, M=self.cap, N=w.shape[0], K=x.shape[1], group_n=n, a_mn=False, b_mn=False, group_mode=0)
        return out

    def dgrad(self, which: int, dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``out[rows of e] = dy[rows of e] @ w_e`` (``w_e`` is ``[K, n]``: the forward weight read MN-major)."""
        n = self.desc[which][1]
        kd = self.desc[which][3]
        assert dy.shape[1] == kd and w.shape == (self.E * kd, n)
        out = torch.empty(self.cap, n, dtype=torch.bfloat16, device=self.device)
        self._launch(which, dy, w, out, M=self.cap, N=n, K=kd, group_n=n, a_mn=False, b_mn=True, group_mode=1, group_b_rows=self.E * kd)
        return out

    def wgrad(self, which: int, dy: torch.Tensor, x: torch.Tensor, gw: torch.Tensor, accumulate: bool) -> None:
        """``gw_e (+)= dy[rows of e]^T @ x[rows of e]`` for every expert; ``gw`` is ``[E * m, n]``."""
        n, m = self.desc[which][1], self.desc[which][3]
        assert dy.shape == (self.cap, m) and x.shape == (self.cap, n) and gw.shape == (self.E * m, n)
        self._launch(which, dy, x, gw, M=m, N=n, K=self.cap, group_n=n, a_mn=True, b_mn=True, group_mode=2,
                     residual=gw if accumulate else None)


class GroupedExperts(torch.autograd.Function):
    """``out[t] = sum_j wt[t, j] * down_e(silu(gate_e x_t) * up_e x_t)``, ``e = idx[t, j]``.

    ``wgu`` ``[E * 2F, d]``: per expert the gate rows then the up rows; ``wd`` ``[E * d, F]``. ``ggu`` / ``gd`` are
    the gradient views the weight gradients are written into; ``sink.accumulate_into(view)`` says whether a view
    already holds gradients of this window (add) or is written for the first time (store)."""

    @staticmethod
    def forward(ctx, h, wt, wgu, ggu, wd, gd, plan: GroupedPlan, sink):
        xs = plan.gather(h)
        gu = plan.forward(FWD_GU, xs, wgu)
        act = _ew.swiglu(gu)
        y = plan.forward(FWD_DN, act, wd)
        wt = wt.contiguous()
        ctx.save_for_backward(xs, gu, y, wt, wgu, wd)
        ctx.plan, ctx.ggu, ctx.gd, ctx.sink = plan, ggu, gd, sink
        return plan.combine(y, wt)

    @staticmethod
    def backward(ctx, dout):
        xs, gu, y, wt, wgu, wd = ctx.saved_tensors
        plan: GroupedPlan = ctx.plan
        dout = dout.contiguous()
        dwt = plan.dot(dout, y) if ctx.needs_input_grad[1] else None
        dy = plan.gather(dout, wt)
        act = _ew.swiglu(gu)                                  # recomputed: cheaper than keeping [rows, F] alive
        plan.wgrad(WGRAD_DN, dy, act, ctx.gd, ctx.sink.accumulate_into(ctx.gd))
        dact = plan.dgrad(DGRAD_DN, dy, wd)
        del act, dy
        dgu = _ew.swiglu_backward(gu, dact)
        plan.wgrad(WGRAD_GU, dgu, xs, ctx.ggu, ctx.sink.accumulate_into(ctx.ggu))
        dh = None
        if ctx.needs_input_grad[0]:
            dh = plan.combine(plan.dgrad(DGRAD_GU, dgu, wgu))
        return dh, dwt, None, None, None, None, None, None


def grouped_experts_reference(h: torch.Tensor, idx: torch.Tensor, wt: torch.Tensor, wgu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """The per-expert loop in fp32 (differentiable): the oracle of ``GroupedExperts`` and the path without a GPU."""
    T, d = h.shape
    E = wd.shape[0] // d
    F2 = wgu.shape[0] // E
    hf = h.float()
    out = torch.zeros(T, d, dtype=torch.float32, device=h.device)
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        gu = hf[tok] @ wgu[e * F2:(e + 1) * F2].float().t()
        g, u = gu[:, :F2 // 2], gu[:, F2 // 2:]
        y = (torch.nn.functional.silu(g) * u) @ wd[e * d:(e + 1) * d].float().t()
        out = out.index_add(0, tok, y * wt[tok, slot].float()[:, None])
    return out
