"""Mixture-of-experts layer: router, dispatch, grouped expert GEMMs on tcgen05, fused combine.

Single GPU: tokens are permuted into expert-contiguous order, the gate|up and down projections
run as two grouped GEMMs driven by a tile table built on the device, and the down projection's
epilogue writes each result row straight back to its ``(token, k)`` slot.

Expert parallel (one rank per GPU): experts are split evenly over the ranks. Dispatch PUSHES
each routed row into the receive buffer of the expert's owner over NVLink (peer stores, slot
positions derived from an exchanged ``[world, E]`` count matrix, so no atomics cross the
link). The owner runs the grouped GEMMs on what it received; the down-projection epilogue
stores every result row into the SOURCE rank's result buffer (peer stores from inside the GEMM
kernel), which is the combine half of the all-to-all. Device barriers separate the phases.

The reference has no MoE/EP code (design notes only, pretrain/docs/design/nano_megatron.md);
the routing math follows its functional oracles (qwen3_next_functional.py:409-490,
glm4_moe_functional.py:230-369), reproduced in ``models/functional.py``.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _native, ops
from ..models.config import ModelConfig
from ..ops._util import check_rc, status_tensor, stream_handle
from ..ops.gemm import EPI_STORE, RbGemmArgs, _lib as _gemm_lib
from .symm import ptr_array

_VP, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _lib():
    lib = _native.load("rb_moe")
    if not getattr(lib, "_rb_typed", False):
        PP = ctypes.POINTER(_VP)
        lib.rb_moe_route.argtypes = [_VP, _VP, _I, _I, _I, _I, _I, _F, _VP, _VP, _VP]
        lib.rb_moe_count.argtypes = [_VP, _I, _I, _VP, _VP]
        lib.rb_moe_plan.argtypes = [_VP, _I, _I, _I, _I, _VP, _I, _I, _VP, _VP, _I, _I, _VP, _VP, _I, _VP, _VP]
        lib.rb_moe_permute.argtypes = [_VP, _VP, _I, _I, _I, _I, _I, _I, _VP, _VP, PP, PP, _I, _VP, _VP]
        lib.rb_moe_translate.argtypes = [_VP, _I, PP, _I, _I, _VP]
        lib.rb_moe_combine.argtypes = [_VP, _VP, _I, _I, _I, _VP, _I, _VP]
        lib.rb_moe_publish_counts.argtypes = [_VP, PP, _I, _I, _I, _VP]
        lib.rb_moe_route_count.argtypes = [_VP, _VP, _I, _I, _I, _I, _I, _F, _VP, _VP, _VP, _VP]
        lib.rb_moe_route_groups.argtypes = [_VP, _VP, _I, _I, _I, _I, _F, _I, _I, _VP, _VP, _VP, _VP]
        lib.rb_moe_plan_dispatch.argtypes = [_VP, _I, _I, _I, _I, _VP, _I, _I, _VP, _VP, _I, _I, _VP, _VP, _I, _VP, _I, _VP, _VP]
        lib.rb_moe_permute_planned.argtypes = lib.rb_moe_permute.argtypes
        for f in ("rb_moe_publish_counts", "rb_moe_route_groups", "rb_moe_route_count", "rb_moe_plan_dispatch", "rb_moe_permute_planned", "rb_moe_route", "rb_moe_count", "rb_moe_plan", "rb_moe_permute", "rb_moe_translate", "rb_moe_combine"):
            getattr(lib, f).restype = _I
        lib._rb_typed = True
    return lib


def route_reference(logits: torch.Tensor, k: int, sigmoid: bool, bias, norm_topk: bool, scaling: float, n_group: int = 1,
                    topk_group: int = 1):
    lg = logits.float()
    if sigmoid:
        from ..models.functional import group_limited_choice

        scores = lg.sigmoid()
        choice = group_limited_choice(scores + (bias.float() if bias is not None else 0), n_group, topk_group)
        idx = choice.topk(k, -1).indices
        w = scores.gather(-1, idx)
        if norm_topk:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
    else:
        probs = lg.softmax(-1)
        w, idx = probs.topk(k, -1)
        if norm_topk:
            w = w / w.sum(-1, keepdim=True)
    return idx.to(torch.int32), (w * scaling).float()


class MoEScratch:
    """Routing tables, dispatch / receive buffers and tile tables of the MoE forward. One object can serve every MoE
    layer of a model (the three device barriers of a layer order its reuse by the next one). With ``fixed=True`` it is
    sized once for ``capacity`` tokens and never reallocated, which CUDA graphs (captured pointers) and expert
    parallelism (allocation is a collective) both need."""

    BN_GU, BN_DN = 128, 128

    def __init__(self, cfg: ModelConfig, device: torch.device, ep=None, capacity: int = 0, fixed: bool = True):
        self.cfg, self.device, self.ep = cfg, device, ep
        self.world = ep.world if ep is not None else 1
        self.fixed = fixed
        self._scratch_for = 0
        if fixed:
            self._alloc(max(capacity, 256))

    def ensure(self, T: int) -> None:
        if T <= self._scratch_for:
            return
        assert not self.fixed, f"MoE scratch sized for {self._scratch_for} tokens, got {T}"
        self._alloc(max(T, 256))

    def _alloc(self, Tcap: int) -> None:
        cfg = self.cfg
        dev, k, d, F, E = self.device, cfg.num_experts_per_tok, cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts
        EL = E // self.world
        cap = Tcap * k * (1 if self.world == 1 else min(self.world, 4))
        self.cap = cap
        self.logits = torch.empty(Tcap, E, dtype=torch.float32, device=dev)
        self.idx = torch.empty(Tcap, k, dtype=torch.int32, device=dev)
        self.w = torch.empty(Tcap, k, dtype=torch.float32, device=dev)
        # one buffer, one memset per forward: histogram of this rank's choices | running index | dispatch base
        self.zbuf = torch.zeros(3 * E, dtype=torch.int32, device=dev)
        self.local_counts, self.cursor = self.zbuf[:E], self.zbuf[E:]
        alloc = (lambda shape, dt: self.ep.comm.alloc(shape, dt, zero=True)) if self.ep is not None else None
        if alloc is None:
            self.counts_all = torch.zeros(1, E, dtype=torch.int32, device=dev)
            self.xp = torch.empty(cap, d, dtype=torch.bfloat16, device=dev)
            self.ret = torch.zeros(cap, dtype=torch.int64, device=dev)
            self.y = torch.empty(Tcap * k, d, dtype=torch.bfloat16, device=dev)
            self.xp_ptrs, self.ret_ptrs, self.y_ptrs = [self.xp.data_ptr()], [self.ret.data_ptr()], [self.y.data_ptr()]
            self.counts_ptrs = None
        else:
            c = alloc((self.world, E), torch.int32)
            xp, ret, y = alloc((cap, d), torch.bfloat16), alloc((cap,), torch.int64), alloc((Tcap * k, d), torch.bfloat16)
            self.counts_all, self.xp, self.ret, self.y = c.local, xp.local, ret.local, y.local
            self.xp_ptrs, self.ret_ptrs, self.y_ptrs = xp.peer_ptrs, ret.peer_ptrs, y.peer_ptrs
            self.counts_ptrs = c.peer_ptrs
            self._symm = (c, xp, ret, y)         # keeps the rendezvous handles alive
            if not hasattr(self, "_barrier_slot"):
                self._barrier_slot = self.ep.comm.new_slot()
            self.ep.comm.barrier_host()
        self.gu = torch.empty(cap, 2 * F, dtype=torch.bfloat16, device=dev)
        self.act = torch.empty(cap, F, dtype=torch.bfloat16, device=dev)
        self.max_tiles = (cap // 128 + EL + 1) * max(-(-2 * F // self.BN_GU), -(-d // self.BN_DN))
        self.tiles_gu = torch.zeros(self.max_tiles, 4, dtype=torch.int32, device=dev)
        self.tiles_dn = torch.zeros(self.max_tiles, 4, dtype=torch.int32, device=dev)
        self.ntiles = torch.zeros(2, dtype=torch.int32, device=dev)
        self.expert_offset = torch.zeros(EL + 1, dtype=torch.int32, device=dev)
        self._scratch_for = Tcap


class MoELayerWeights:
    """Weights and scratch of one MoE layer; ``forward(h, x)`` does ``x += MoE(h)`` in place."""

    BN_GU, BN_DN = 128, 128

    def __init__(self, cfg: ModelConfig, device: torch.device, ep=None, scratch: "MoEScratch | None" = None):
        self.scratch = scratch if device.type == "cuda" else None
        self.cfg = cfg
        self.device = device
        self.ep = ep                      # TensorParallel context used as the expert-parallel group, or None
        self.world = ep.world if ep is not None else 1
        self.rank = ep.rank if ep is not None else 0
        E, d, F, k = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts_per_tok
        assert E % self.world == 0 and E <= 256
        self.E, self.EL, self.d, self.F, self.k = E, E // self.world, d, F, k
        self.e_lo = self.rank * self.EL
        on_gpu = device.type == "cuda"
        dt = torch.bfloat16 if on_gpu else torch.float32
        self.gate = torch.empty(E, d, dtype=dt, device=device)
        self.gate_bias = torch.empty(E, dtype=torch.float32, device=device) if cfg.router_type == "sigmoid" else None
        self.wgu = torch.empty(self.EL * 2 * F, d, dtype=dt, device=device)   # per expert: gate rows then up rows
        self.wd = torch.empty(self.EL * d, F, dtype=dt, device=device)
        self.shared = None
        if cfg.n_shared_experts > 0:
            Fs = F * cfg.n_shared_experts
            self.shared = (torch.empty(2 * Fs, d, dtype=dt, device=device), torch.empty(d, Fs, dtype=dt, device=device))
        self._on_gpu = on_gpu

    # ---------------------------------------------------------------- weights
    def load(self, weights: dict[str, torch.Tensor], prefix: str) -> None:
        F, d = self.F, self.d

        def put(dst, src):
            dst.copy_(src.to(device=self.device, dtype=dst.dtype))

        put(self.gate, weights[prefix + "gate.weight"])
        if self.gate_bias is not None:
            put(self.gate_bias, weights[prefix + "gate.e_score_correction_bias"])
        for i in range(self.EL):
            e = self.e_lo + i
            put(self.wgu[i * 2 * F:i * 2 * F + F], weights[f"{prefix}experts.{e}.gate_proj.weight"])
            put(self.wgu[i * 2 * F + F:(i + 1) * 2 * F], weights[f"{prefix}experts.{e}.up_proj.weight"])
            put(self.wd[i * d:(i + 1) * d], weights[f"{prefix}experts.{e}.down_proj.weight"])
        if self.shared is not None:
            Fs = self.shared[1].shape[1]
            put(self.shared[0][:Fs], weights[prefix + "shared_experts.gate_proj.weight"])
            put(self.shared[0][Fs:], weights[prefix + "shared_experts.up_proj.weight"])
            put(self.shared[1], weights[prefix + "shared_experts.down_proj.weight"])

    def sync_segments(self, prefix: str):
        """(name, dst, rows, cols, row0, col0) tuples for the weight-sync plan."""
        F, d = self.F, self.d
        out = [(prefix + "gate.weight", self.gate, self.E, d, 0, 0)]
        for i in range(self.EL):
            e = self.e_lo + i
            out.append((f"{prefix}experts.{e}.gate_proj.weight", self.wgu[i * 2 * F:i * 2 * F + F], F, d, 0, 0))
            out.append((f"{prefix}experts.{e}.up_proj.weight", self.wgu[i * 2 * F + F:(i + 1) * 2 * F], F, d, 0, 0))
            out.append((f"{prefix}experts.{e}.down_proj.weight", self.wd[i * d:(i + 1) * d], d, F, 0, 0))
        if self.shared is not None:
            Fs = self.shared[1].shape[1]
            out.append((prefix + "shared_experts.gate_proj.weight", self.shared[0][:Fs], Fs, d, 0, 0))
            out.append((prefix + "shared_experts.up_proj.weight", self.shared[0][Fs:], Fs, d, 0, 0))
            out.append((prefix + "shared_experts.down_proj.weight", self.shared[1], d, Fs, 0, 0))
        return out

    # ---------------------------------------------------------------- scratch
    def _ensure_scratch(self, T: int) -> None:
        if self.scratch is None:
            self.scratch = MoEScratch(self.cfg, self.device, self.ep, fixed=False)
        self.scratch.ensure(T)

    def __getattr__(self, name):
        # routing tables, receive buffers and tile tables live in the (possibly shared) scratch object
        sc = self.__dict__.get("scratch")
        if sc is not None and name in sc.__dict__:
            return sc.__dict__[name]
        raise AttributeError(name)

    # ---------------------------------------------------------------- forward
    def forward(self, h: torch.Tensor, x: torch.Tensor) -> None:
        """``x += MoE(h)`` for ``h, x`` of shape ``[T, d]``."""
        if not self._on_gpu:
            self._forward_reference(h, x)
            return
        T = h.shape[0]
        self._ensure_scratch(T)
        cfg, k, d, F, E = self.cfg, self.k, self.d, self.F, self.E
        dev = self.device
        st = status_tensor(dev).data_ptr()
        s = stream_handle(dev)
        lib = _lib()
        logits = ops.gemm(h, self.gate, out=self.logits[:T], out_f32=True)
        self.zbuf.zero_()
        bias = self.gate_bias.data_ptr() if self.gate_bias is not None else None
        if cfg.router_type == "sigmoid" and cfg.n_group > 1 and cfg.topk_group < cfg.n_group:
            check_rc(lib.rb_moe_route_groups(logits.data_ptr(), bias, T, E, k, int(cfg.norm_topk_prob), float(cfg.routed_scaling_factor),
                                             cfg.n_group, cfg.topk_group, self.idx.data_ptr(), self.w.data_ptr(),
                                             self.local_counts.data_ptr(), s), "rb_moe_route_groups")
        else:
            check_rc(lib.rb_moe_route_count(logits.data_ptr(), bias, T, E, k, int(cfg.router_type == "sigmoid"), int(cfg.norm_topk_prob),
                                            float(cfg.routed_scaling_factor), self.idx.data_ptr(), self.w.data_ptr(),
                                            self.local_counts.data_ptr(), s), "rb_moe_route_count")
        if self.counts_ptrs is None:
            self.counts_all[0].copy_(self.local_counts)
        else:                                     # one kernel stores my counts row on every rank
            check_rc(lib.rb_moe_publish_counts(self.local_counts.data_ptr(), ptr_array(self.counts_ptrs), self.rank,
                                               self.world, E, s), "rb_moe_publish_counts")
            self.ep.comm.barrier(self._barrier_slot)
        check_rc(lib.rb_moe_plan_dispatch(self.counts_all.data_ptr(), self.world, E, self.e_lo, self.e_lo + self.EL,
                                          self.expert_offset.data_ptr(), 2 * F, self.BN_GU, self.tiles_gu.data_ptr(),
                                          self.ntiles.data_ptr(), d, self.BN_DN, self.tiles_dn.data_ptr(),
                                          self.ntiles.data_ptr() + 4, self.max_tiles, st, self.rank, self.cursor.data_ptr(), s),
                 "rb_moe_plan_dispatch")
        check_rc(lib.rb_moe_permute_planned(h.data_ptr(), self.idx.data_ptr(), T, k, d, E, self.world, self.rank,
                                    self.counts_all.data_ptr(), self.cursor.data_ptr(), ptr_array(self.xp_ptrs),
                                    ptr_array(self.ret_ptrs), self.cap, st, s), "rb_moe_permute_planned")
        if self.counts_ptrs is not None:
            self.ep.comm.barrier(self._barrier_slot)   # every routed row has landed on its owner
        check_rc(lib.rb_moe_translate(self.ret.data_ptr(), self.cap, ptr_array(self.y_ptrs), self.world, d, s), "rb_moe_translate")
        self._grouped(self.xp, self.wgu, self.gu, 2 * F, d, self.BN_GU, self.tiles_gu, self.ntiles.data_ptr(), None)
        if self.world > 1:   # only the device knows how many rows arrived: expert_offset[EL] bounds the pass
            ops.swiglu(self.gu, out=self.act, rows_dev=self.expert_offset[self.EL:])
        else:
            ops.swiglu(self.gu[:T * k], out=self.act[:T * k])
        self._grouped(self.act, self.wd, None, d, F, self.BN_DN, self.tiles_dn, self.ntiles.data_ptr() + 4, self.ret)
        if self.counts_ptrs is not None:
            self.ep.comm.barrier(self._barrier_slot)   # every result row is home
        check_rc(lib.rb_moe_combine(self.y.data_ptr(), self.w.data_ptr(), T, k, d, x.data_ptr(), 1, s), "rb_moe_combine")
        if self.shared is not None:
            wgu, wd = self.shared
            act = ops.swiglu(ops.gemm(h, wgu))
            ops.gemm(act, wd, residual=x, out=x)

    def _grouped(self, a, b, c, group_n, K, bn, tiles, ntiles_ptr, row_dst) -> None:
        args = RbGemmArgs()
        args.A[0], args.B[0] = a.data_ptr(), b.data_ptr()
        args.C = c.data_ptr() if c is not None else a.data_ptr()
        args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), (c.stride(0) if c is not None else group_n)
        args.M, args.N, args.K = a.shape[0], b.shape[0], K
        args.a_parts = args.b_parts = 1
        args.bn = bn
        args.epi_mode = EPI_STORE
        args.rank, args.world = 0, 1
        args.status = status_tensor(self.device).data_ptr()
        args.tile_table, args.num_tiles_ptr = tiles.data_ptr(), ntiles_ptr
        args.group_n, args.max_tiles = group_n, self.max_tiles
        args.row_dst = row_dst.data_ptr() if row_dst is not None else None
        rc = _gemm_lib().rb_gemm_bf16_ex(ctypes.byref(args), stream_handle(self.device))
        check_rc(rc, "rb_gemm_bf16_ex(grouped)")

    # ---------------------------------------------------------------- CPU / oracle path
    def _forward_reference(self, h: torch.Tensor, x: torch.Tensor) -> None:
        cfg, F, d = self.cfg, self.F, self.d
        hf = h.float()
        idx, w = route_reference(hf @ self.gate.float().t(), self.k, cfg.router_type == "sigmoid", self.gate_bias,
                                 cfg.norm_topk_prob, cfg.routed_scaling_factor, cfg.n_group, cfg.topk_group)
        if self.world > 1:
            # every rank evaluates its own experts for everyone's tokens, then the sums are exchanged
            g = self.ep.comm.group
            n_all = [torch.zeros(1, dtype=torch.int64) for _ in range(self.world)]
            dist.all_gather(n_all, torch.tensor([hf.shape[0]]), group=g)
            Tm = int(max(int(n) for n in n_all))            # ranks may hold different token counts: pad to the largest

            def padded(t, fill):
                out = torch.full((Tm,) + tuple(t.shape[1:]), fill, dtype=t.dtype)
                out[:t.shape[0]] = t
                return out

            hp, ip, wp = padded(hf, 0.0), padded(idx, -1), padded(w, 0.0)
            hs = [torch.empty_like(hp) for _ in range(self.world)]
            ids = [torch.empty_like(ip) for _ in range(self.world)]
            ws = [torch.empty_like(wp) for _ in range(self.world)]
            dist.all_gather(hs, hp, group=g)
            dist.all_gather(ids, ip, group=g)
            dist.all_gather(ws, wp, group=g)
            outs = [self._experts_reference(a, b, c) for a, b, c in zip(hs, ids, ws)]
            tot = torch.stack(outs)
            dist.all_reduce(tot, group=g)
            out = tot[self.rank][:hf.shape[0]]
        else:
            out = self._experts_reference(hf, idx, w)
        if self.shared is not None:
            wgu, wd = self.shared
            g, u = (hf @ wgu.float().t()).chunk(2, -1)
            out = out + (torch.nn.functional.silu(g) * u) @ wd.float().t()
        x.add_(out.to(x.dtype))
        _ = (F, d)

    def _experts_reference(self, hf, idx, w) -> torch.Tensor:
        F, d = self.F, self.d
        out = torch.zeros_like(hf)
        for i in range(self.EL):
            e = self.e_lo + i
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            wg = self.wgu[i * 2 * F:(i + 1) * 2 * F].float()
            g, u = (hf[tok] @ wg.t()).chunk(2, -1)
            y = (torch.nn.functional.silu(g) * u) @ self.wd[i * d:(i + 1) * d].float().t()
            out.index_add_(0, tok, y * w[tok, slot][:, None])
        return out
