"""Tensor-parallel linear layers whose collective runs inside the tcgen05 GEMM kernel.

* ``all_gather_gemm``  (column-parallel; activations sharded by rows across ranks): two gather
  warps in every CTA of the GEMM launch copy the peers' row slabs from their symmetric buffers
  into a local staging matrix (each remote row crosses NVLink once), the tile producers wait
  for the parts and the tiles run over the staged matrix.
* ``fsdp_gemm`` (FSDP parameter shards): same mechanism on the B operand - the weight rows a
  rank does not own are read from the owning peer inside the first GEMM that consumes them.
* ``gemm_reduce_scatter`` / ``gemm_all_reduce`` (row-parallel): finished tiles are pushed with
  peer stores into the owner's staging slab and published with a flag; the owner's epilogue
  warps sum the partials and write the result (all-reduce: to every peer).

Staging slabs are double buffered: a rank can only enter call i+2 after every peer finished
call i (its reduce phase waits for all peers' call-(i+1) tiles, which they push only after
finishing call i), so no barrier is needed between reduce-scatters. After a two-hop all-reduce the
outputs live in peer memory written by other GPUs, so a device-side barrier follows. Decode-sized
all-reduces take the one-shot form instead (every rank pushes its partial to every rank and sums
locally): one hop, one kernel, no barrier.

The reference has no tensor parallelism in-tree (``EngineConfig.tensor_parallel_size`` is
unused, rollouts/inference/types.py:25; only ``--tp`` forwarded to an external SGLang).
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops._util import check_rc, status_tensor, stream_handle
from ..ops.gemm import EPI_ALL_REDUCE, EPI_ALL_REDUCE_ONESHOT, EPI_REDUCE_SCATTER, EPI_STORE, RbGemmArgs, _lib as _gemm_lib
from .symm import PeerComm, SymmBuffer


class TensorParallel:
    def __init__(self, comm: PeerComm, max_rows: int, max_cols: int, expert_parallel: bool = False):
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        self.expert_parallel = expert_parallel
        self.row_align = 8 * self.world
        self.max_rows = -(-max_rows // self.row_align) * self.row_align
        self.max_cols = max_cols
        self._registry: dict[int, SymmBuffer] = {}
        self._call = 0
        self._ag_epoch = 0
        self._ar_sync = self._ar_ack = None
        self.ag_stage = self.ag_flags = None
        self._ready_slot = comm.new_slot()
        if comm.on_gpu:
            rpr = self.max_rows // self.world
            self.stage = comm.alloc((2, self.world, rpr, max_cols), torch.bfloat16)
            self.max_tiles = (-(-rpr // 128)) * (-(-max_cols // 32))
            self.tile_flags = comm.alloc((2, self.world, self.max_tiles), torch.int32, zero=True)
            # [0] epoch counter of the reduce calls, [1] CTA ticket (device side, graph safe)
            self.reduce_state = torch.zeros(2, dtype=torch.int32, device=comm.device)
            # epoch of the "my shard is ready" signal, counted on the device (see publish_device)
            self.ready_counter = torch.zeros(1, dtype=torch.int32, device=comm.device)
            self._barrier_slot = comm.new_slot()
            # decode-sized row-parallel GEMMs with a long K: partial tile of this rank for the split path below
            self.SPLIT_AR_ROWS = 256
            self.ar_slab = comm.alloc((self.SPLIT_AR_ROWS * max_cols,), torch.bfloat16, zero=True)
            self._ar_slot = comm.new_slot()
            # two-launch form of that path: [0] epoch, [1] block ticket, [2] acknowledgements this rank's next slab
            # write waits for; the peers count their reads of this rank's slab in _ar_ack
            self._ar_sync = torch.zeros(3, dtype=torch.int32, device=comm.device)
            self._ar_ack = comm.alloc((1,), torch.int32, zero=True)
            self._ar_flag_slot = comm.new_slot()
            comm.barrier_host()

    # ---------------------------------------------------------------- buffers
    def alloc(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        """Symmetric tensor (same address layout on every rank); remembered by base pointer."""
        buf = self.comm.alloc(tuple(shape), dtype, zero=True)
        self._registry[buf.local.data_ptr()] = buf
        return buf.local

    def symm_of(self, t: torch.Tensor) -> SymmBuffer:
        buf = self._registry.get(t.data_ptr())
        assert buf is not None, "tensor was not allocated with TensorParallel.alloc (or is not a row-0 view)"
        return buf

    # ---------------------------------------------------------------- helpers
    def _base_args(self, M, N, K, a, w, bn) -> RbGemmArgs:
        args = RbGemmArgs()
        args.M, args.N, args.K = M, N, K
        args.lda, args.ldb = a.stride(0), w.stride(0)
        args.a_parts = args.b_parts = 1
        args.bn = bn
        args.rank, args.world = self.rank, self.world
        args.status = status_tensor(a.device).data_ptr()
        return args

    def _launch(self, args: RbGemmArgs, device) -> None:
        rc = _gemm_lib().rb_gemm_bf16_ex(ctypes.byref(args), stream_handle(device))
        check_rc(rc, "rb_gemm_bf16_ex(tp)")

    @staticmethod
    def _pick_bn(rows_per_rank: int, N: int) -> int:
        """0 = let the kernel's cost model choose (it weighs tile count against the 148 SMs: decode-sized
        problems get narrow tiles so that every SM streams weights). The flag arrays are sized for the
        narrowest tile (32 columns), so any choice fits."""
        return 0

    # ---------------------------------------------------------------- row-parallel
    def _reduce(self, a: torch.Tensor, w: torch.Tensor, mode: int, out_ptrs, ldc: int, residual, ldr: int) -> None:
        M, K = a.shape
        N = w.shape[0]
        assert M % self.row_align == 0, f"rows ({M}) must be a multiple of {self.row_align}"
        assert M <= self.max_rows and N <= self.max_cols
        rpr = M // self.world
        bn = self._pick_bn(rpr, N)
        self._call += 1
        args = self._base_args(M, N, K, a, w, bn)
        args.a_parts = self.world
        for i in range(self.world):
            args.A[i] = a.data_ptr() + i * rpr * a.stride(0) * 2
        args.B[0] = w.data_ptr()
        args.epi_mode = mode
        args.ldc, args.ldr = ldc, ldr
        args.residual = residual
        # the epoch and the staging parity come from the device counter (see gemm_sm100.h)
        args.epoch_counter = self.reduce_state.data_ptr()
        args.cta_ticket = self.reduce_state.data_ptr() + 4
        args.stage_parity_bytes = self.world * (self.max_rows // self.world) * self.max_cols * 2
        args.flag_parity_bytes = self.world * self.max_tiles * 4
        # staging is addressed as [src_rank][rows_per_rank][N] inside one parity slab
        for r in range(self.world):
            args.stage_ptrs[r] = self.stage.peer_ptrs[r]
            args.flag_ptrs[r] = self.tile_flags.peer_ptrs[r]
            args.out_ptrs[r] = out_ptrs[r]
        args.C = out_ptrs[self.rank]
        self._launch(args, a.device)

    def gemm_all_reduce(self, a: torch.Tensor, w: torch.Tensor, x: torch.Tensor) -> None:
        """``x += sum_ranks(a_r @ w_r.T)`` in place on every rank; ``x`` is a symmetric tensor."""
        if not self.comm.on_gpu:
            part = a.float() @ w.float().t()
            dist.all_reduce(part, group=self.comm.group)
            x.add_(part.to(x.dtype))
            return
        M, N = a.shape[0], w.shape[0]
        if (self.SPLIT_AR and M <= self.SPLIT_AR_ROWS and a.shape[1] >= 2048 and N <= self.max_cols and x.stride(0) == N
                and (M * N) % 8 == 0):
            self._reduce_split(a, w, x)
            return
        if M <= self.max_rows // self.world and M * N * 2 * (self.world - 1) <= self.ONESHOT_MAX_BYTES:
            # decode-sized output: push the partial to every rank, each rank sums locally. One hop, one kernel,
            # and no barrier afterwards: staging alternates between two parity slabs and a rank cannot run two
            # calls ahead of a peer, because finishing a call needs the peer's partial of that call.
            self._reduce_oneshot(a, w, x)
            return
        buf = self.symm_of(x)
        self._reduce(a, w, EPI_ALL_REDUCE, buf.peer_ptrs, x.stride(0), x.data_ptr(), x.stride(0))
        self.comm.barrier(self._barrier_slot)

    # Bytes a rank may push to its peers in a one-shot call (output bytes x (ranks - 1)). One shot saves a hop and a
    # barrier but moves (W - 1) copies of the output per rank where the two-hop path moves 2 (W - 1) / W: measured on
    # the 8B decode step (M = 256, N = 4096) one shot wins at 2 ranks (2 MB pushed) and loses at 8 (14 MB pushed:
    # 7.20 vs 6.59 ms per step). RB_TP_ONESHOT_MAX_BYTES overrides (0 = always two hops).
    ONESHOT_MAX_BYTES = int(os.environ.get("RB_TP_ONESHOT_MAX_BYTES", 4 << 20))

    # The fused reduce epilogues cannot split K (their epilogue is the reduction), so with few rows and a long K the
    # per-rank GEMM runs on few CTAs at the rate one SM streams operands and does not shrink with the rank count.
    # This path is two launches instead: the plain GEMM (which splits K over thread-block clusters) into this rank's
    # slab, and a pull-sum over all ranks' slabs (peer loads, rank order, so every rank gets the same bits) that
    # carries its own synchronisation: it publishes "my slab is complete", waits for the peers' flags, sums, and
    # acknowledges the peers' slabs; the NEXT call's GEMM waits inside its launch for the acknowledgements of this
    # call before it overwrites the slab. No barrier launches; epochs live on the device (graph replay).
    # RB_TP_SPLIT_AR=0 switches the path off, RB_TP_SPLIT_AR=barriers keeps the earlier four-launch form.
    SPLIT_AR = os.environ.get("RB_TP_SPLIT_AR", "1") != "0"
    SPLIT_AR_BARRIERS = os.environ.get("RB_TP_SPLIT_AR", "1") == "barriers"

    def _reduce_split(self, a: torch.Tensor, w: torch.Tensor, x: torch.Tensor) -> None:
        from .symm import _lib as _comm_lib, ptr_array
        from .. import ops

        M, N = a.shape[0], w.shape[0]
        part = self.ar_slab.local[: M * N].view(M, N)
        dev = a.device
        if self.SPLIT_AR_BARRIERS:
            ops.gemm(a, w, out=part)
            self.comm.barrier(self._ar_slot)                  # every rank's partial is complete
            rc = _comm_lib().rb_pull_sum(ptr_array(self.ar_slab.peer_ptrs), x.data_ptr(), x.data_ptr(), M * N, self.world,
                                         stream_handle(dev))
            check_rc(rc, "rb_pull_sum")
            self.comm.barrier(self._ar_slot)                  # every rank has read every slab: the next call may write
            return
        sync = self._ar_sync.data_ptr()
        ops.gemm(a, w, out=part, wait_flag=(self._ar_ack.local.data_ptr(), sync + 8))
        rc = _comm_lib().rb_pull_sum_sync(ptr_array(self.ar_slab.peer_ptrs), x.data_ptr(), x.data_ptr(), M * N, self.world, self.rank,
                                          self.comm.flags.ptrs(), self._ar_flag_slot, sync, self._ar_ack.ptrs(), sync + 8,
                                          status_tensor(dev).data_ptr(), stream_handle(dev))
        check_rc(rc, "rb_pull_sum_sync")

    def _reduce_oneshot(self, a: torch.Tensor, w: torch.Tensor, x: torch.Tensor) -> None:
        M, K = a.shape
        N = w.shape[0]
        assert M % 8 == 0 and N <= self.max_cols
        bn = self._pick_bn(M, N)
        self._call += 1
        args = self._base_args(M, N, K, a, w, bn)
        args.A[0], args.B[0] = a.data_ptr(), w.data_ptr()
        args.epi_mode = EPI_ALL_REDUCE_ONESHOT
        args.C, args.ldc = x.data_ptr(), x.stride(0)
        args.residual, args.ldr = x.data_ptr(), x.stride(0)
        args.epoch_counter = self.reduce_state.data_ptr()
        args.cta_ticket = self.reduce_state.data_ptr() + 4
        args.stage_parity_bytes = self.world * (self.max_rows // self.world) * self.max_cols * 2
        args.flag_parity_bytes = self.world * self.max_tiles * 4
        for r in range(self.world):
            args.stage_ptrs[r] = self.stage.peer_ptrs[r]
            args.flag_ptrs[r] = self.tile_flags.peer_ptrs[r]
        self._launch(args, a.device)

    def gemm_reduce_scatter(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                            residual: torch.Tensor | None = None) -> torch.Tensor:
        """``out[M/P, N] = (sum_ranks a_r @ w_r.T)[rank's row slab] (+ residual)``; ``out`` is local."""
        if not self.comm.on_gpu:
            part = a.float() @ w.float().t()
            dist.all_reduce(part, group=self.comm.group)
            rpr = a.shape[0] // self.world
            res = part[self.rank * rpr:(self.rank + 1) * rpr]
            if residual is not None:
                res = res + residual.float()
            out.copy_(res.to(out.dtype))
            return out
        ptrs = [0] * self.world
        ptrs[self.rank] = out.data_ptr()
        self._reduce(a, w, EPI_REDUCE_SCATTER, ptrs, out.stride(0), residual.data_ptr() if residual is not None else None,
                     residual.stride(0) if residual is not None else 0)
        return out

    # ---------------------------------------------------------------- column-parallel / FSDP
    def publish(self) -> int:
        """Signal that this rank's symmetric operand (activation or weight shard) is complete."""
        return self.comm.signal(self._ready_slot)

    def publish_device(self) -> None:
        """``publish`` with the epoch counted on the device: safe inside a captured CUDA graph. Pair it with
        ``all_gather_gemm(..., ready_epoch="device")``."""
        if not self.comm.on_gpu:
            return
        from .symm import _lib as _comm_lib

        rc = _comm_lib().rb_symm_signal_counter(self.comm.flags.ptrs(), self.rank, self.world, self._ready_slot,
                                                self.ready_counter.data_ptr(), stream_handle(self.comm.device))
        check_rc(rc, "rb_symm_signal_counter")

    def all_gather_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias=None,
                        ready_epoch: int | str | None = None, out_f32: bool = False) -> torch.Tensor:
        """``out[M, N] = concat_ranks(x_shard_r) @ w.T``; ``x_shard`` is a symmetric ``[M/P, K]`` tensor.

        ``ready_epoch`` is the value returned by ``publish()`` on every rank after the shard was
        written (or ``"device"`` after ``publish_device()``); the kernel's producer warp waits for each peer's
        flag before its first load from that peer.
        """
        rows, K = x_shard.shape
        N = w.shape[0]
        if not self.comm.on_gpu:
            parts = [torch.empty_like(x_shard) for _ in range(self.world)]
            dist.all_gather(parts, x_shard.contiguous(), group=self.comm.group)
            res = torch.cat(parts).float() @ w.float().t()
            if bias is not None:
                res = res + bias.float()
            out.copy_(res.to(out.dtype))
            return out
        assert out.dtype == (torch.float32 if out_f32 else torch.bfloat16)
        assert x_shard.is_contiguous() and rows * self.world <= self.max_rows and K <= self.max_cols
        buf = self.symm_of(x_shard)
        # Every CTA of the launch copies a share of the peers' slabs into the local staging matrix with its two gather
        # warps (each remote row crosses NVLink once, whatever the number of column tiles), the tile producers wait for
        # the parts, and the tiles then run over the staged [M, K] matrix as one A operand.
        if self.ag_stage is None:
            self.ag_stage = torch.empty(self.max_rows * self.max_cols, dtype=torch.bfloat16, device=x_shard.device)
            self.ag_flags = torch.zeros(4, 8, dtype=torch.int32, device=x_shard.device)   # count / ready: host epochs, device epochs
        args = self._base_args(rows * self.world, N, K, x_shard, w, 0)
        args.out_f32 = int(out_f32)
        args.A[0] = self.ag_stage.data_ptr()
        args.lda = K
        args.B[0] = w.data_ptr()
        args.C, args.ldc = out.data_ptr(), out.stride(0)
        args.bias = bias.data_ptr() if bias is not None else None
        args.epi_mode = EPI_STORE
        args.world = 1                      # plain store epilogue; `rank` names this rank's part of the gather
        for r in range(self.world):
            args.gather_src[r] = buf.peer_ptrs[r]
        args.gather_dst = self.ag_stage.data_ptr()
        args.gather_part_bytes = rows * K * 2
        args.gather_parts = self.world
        args.gather_wait_all = 1
        device_epoch = ready_epoch == "device"
        flags = self.ag_flags[2:] if device_epoch else self.ag_flags[:2]
        args.gather_count, args.gather_ready = flags[0].data_ptr(), flags[1].data_ptr()
        if device_epoch:
            args.gather_src_ready = self.comm.flag_ptr(self._ready_slot)
            args.ready_epoch_ptr = self.ready_counter.data_ptr()
        else:
            self._ag_epoch += 1
            args.gather_epoch = self._ag_epoch
            if ready_epoch is not None:
                args.gather_src_ready = self.comm.flag_ptr(self._ready_slot)
                args.ready_epoch = ready_epoch
        self._launch(args, x_shard.device)
        return out

    def fsdp_gemm(self, x: torch.Tensor, w_shard: torch.Tensor, out: torch.Tensor,
                  ready_epoch: int | None = None) -> torch.Tensor:
        """``out[M, N] = x @ concat_ranks(w_shard_r).T``; ``w_shard`` is a symmetric ``[N/P, K]`` tensor."""
        M, K = x.shape
        rows = w_shard.shape[0]
        if not self.comm.on_gpu:
            parts = [torch.empty_like(w_shard) for _ in range(self.world)]
            dist.all_gather(parts, w_shard.contiguous(), group=self.comm.group)
            out.copy_((x.float() @ torch.cat(parts).float().t()).to(out.dtype))
            return out
        buf = self.symm_of(w_shard)
        args = self._base_args(M, rows * self.world, K, x, w_shard, 0)
        args.b_parts = self.world
        args.A[0] = x.data_ptr()
        for r in range(self.world):
            args.B[r] = buf.peer_ptrs[r]
        args.C, args.ldc = out.data_ptr(), out.stride(0)
        args.epi_mode = EPI_STORE
        if ready_epoch is not None:
            args.b_ready = self.comm.flag_ptr(self._ready_slot)
            args.ready_epoch = ready_epoch
        self._launch(args, x.device)
        return out
