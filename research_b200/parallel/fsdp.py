"""Sharded data-parallel training state: flat parameter / gradient buckets in symmetric memory
and a sharded AdamW whose collectives run inside the optimizer kernels.

Layout (B200-first: 180 GB of HBM per GPU makes replicated bf16 parameters cheap, so only what
is large - fp32 master weights, both moments and the reduced gradients - is sharded):

* ``params``  one flat bf16 tensor, complete on every rank, in symmetric memory;
* ``grads``   one flat bf16 tensor per rank (local accumulation target of backward), symmetric;
* chunk c (a layer) of both tensors is split evenly over the ranks; rank r keeps the fp32
  master copy, ``exp_avg`` and ``exp_avg_sq`` of its slice only.

One optimizer step:
  1. per chunk, as soon as its backward finished: ``rs_reduce`` - the owner PULLS its slice of
     every peer's gradient chunk over NVLink, sums in fp32, applies 1/(world*accum) and
     accumulates the squared norm, in one pass (reduce-scatter + cast + scale + norm partials);
  2. ``clip_coef`` - ranks exchange their partial norms through peer memory; the clip
     coefficient stays on the device;
  3. per chunk: ``adamw_allgather`` - AdamW on the slice, the new bf16 values PUSHED into every
     rank's ``params`` from the same kernel (optimizer + all-gather fused);
  4. one device barrier: parameters are complete everywhere, gradients may be reused.

Replaces FSDP2's NCCL all-gather/reduce-scatter, ``clip_grad_norm_`` and ``torch.optim.AdamW``
as used by the reference backend (rollouts/training/backends/fsdp.py:289-322, 398-479). With a
CPU/gloo group the same class runs the textbook equivalent with ordinary collectives, which is
what the multi-rank CPU tests compare against ``torch.optim.AdamW``.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops._util import check_rc, status_tensor, stream_handle
from .symm import PeerComm, _lib


@dataclass
class ParamSpec:
    name: str
    shape: tuple[int, ...]
    offset: int        # element offset inside the flat buckets
    numel: int
    chunk: int


class FlatBuckets:
    """Flat bf16 parameter and gradient storage with per-parameter views."""

    def __init__(self, comm: PeerComm, named_shapes: list[tuple[str, tuple[int, ...]]], chunk_of=None,
                 dtype: torch.dtype = torch.bfloat16):
        self.comm = comm
        align = 8 * comm.world
        self.specs: dict[str, ParamSpec] = {}
        self.chunks: list[tuple[int, int]] = []  # (offset, length) per chunk, length % align == 0
        off = 0
        cur_chunk, chunk_start = None, 0
        for name, shape in named_shapes:
            c = chunk_of(name) if chunk_of else 0
            if cur_chunk is None:
                cur_chunk = c
            if c != cur_chunk:
                off = -(-off // align) * align
                self.chunks.append((chunk_start, off - chunk_start))
                chunk_start, cur_chunk = off, c
            n = 1
            for s in shape:
                n *= s
            n_pad = -(-n // 8) * 8  # keep every parameter 16-byte aligned for TMA
            self.specs[name] = ParamSpec(name, tuple(shape), off, n, len(self.chunks))
            off += n_pad
        off = -(-off // align) * align
        self.chunks.append((chunk_start, off - chunk_start))
        self.numel = off
        self.dtype = dtype
        self.params_buf = comm.alloc((self.numel,), dtype, zero=True)
        self.grads_buf = comm.alloc((self.numel,), dtype, zero=True)
        self.params, self.grads = self.params_buf.local, self.grads_buf.local

    def param_view(self, name: str) -> torch.Tensor:
        s = self.specs[name]
        return self.params[s.offset:s.offset + s.numel].view(s.shape)

    def grad_view(self, name: str) -> torch.Tensor:
        s = self.specs[name]
        return self.grads[s.offset:s.offset + s.numel].view(s.shape)

    def shard_range(self, chunk: int) -> tuple[int, int]:
        """(element offset, length) of this rank's slice of ``chunk``."""
        off, length = self.chunks[chunk]
        n = length // self.comm.world
        return off + self.comm.rank * n, n


class ShardedAdamW:
    def __init__(self, buckets: FlatBuckets, lr: float = 1e-5, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.0, max_grad_norm: float = 1.0):
        self.b = buckets
        self.comm = buckets.comm
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        dev = buckets.params.device
        self.master, self.exp_avg, self.exp_avg_sq, self.red = [], [], [], []
        for c in range(len(buckets.chunks)):
            off, n = buckets.shard_range(c)
            self.master.append(buckets.params[off:off + n].float().clone())
            self.exp_avg.append(torch.zeros(n, dtype=torch.float32, device=dev))
            self.exp_avg_sq.append(torch.zeros(n, dtype=torch.float32, device=dev))
            self.red.append(torch.zeros(n, dtype=torch.float32, device=dev))
        self.on_gpu = self.comm.on_gpu
        if self.on_gpu:
            self.n_partial = _lib().rb_rs_num_partials()
            self.partial = torch.zeros(self.n_partial, dtype=torch.float32, device=dev)
            self.coef = torch.ones(1, dtype=torch.float32, device=dev)
            self.norm = torch.zeros(1, dtype=torch.float32, device=dev)
            self.grad_slots = [self.comm.new_slot() for _ in buckets.chunks] if len(buckets.chunks) <= 40 else None
            self.norm_slot = self.comm.new_slot()
            self._shared_slot = self.comm.new_slot()
        self._reduced: set[int] = set()
        self._sumsq_cpu = 0.0

    def resync_master(self) -> None:
        """Re-read the fp32 master slices from the bf16 parameters (after loading weights)."""
        for c in range(len(self.b.chunks)):
            off, n = self.b.shard_range(c)
            self.master[c].copy_(self.b.params[off:off + n].float())

    # ---------------------------------------------------------------- phase 1
    def reduce_chunk(self, chunk: int, grad_scale: float = 1.0) -> None:
        """Reduce-scatter one gradient chunk into this rank's fp32 slice (call once its backward is done)."""
        b, comm = self.b, self.comm
        off, length = b.chunks[chunk]
        n = length // comm.world
        scale = grad_scale / comm.world
        if not self.on_gpu:
            g = b.grads[off:off + length].float()
            if comm.world > 1:
                dist.all_reduce(g, group=comm.group)
            mine = g[comm.rank * n:(comm.rank + 1) * n] * scale
            self.red[chunk].copy_(mine)
            self._sumsq_cpu += float((mine * mine).sum())
            self._reduced.add(chunk)
            return
        slot = self.grad_slots[chunk] if self.grad_slots is not None else self._shared_slot
        epoch = comm.signal(slot)  # my gradients for this chunk are final
        ptrs = b.grads_buf.ptrs(off * 2)
        rc = _lib().rb_rs_reduce(ptrs, comm.flags.local.data_ptr(), slot, epoch, comm.rank, comm.world, n, scale,
                                 self.red[chunk].data_ptr(), 0, self.partial.data_ptr(),
                                 status_tensor(b.params.device).data_ptr(), stream_handle(b.params.device))
        check_rc(rc, "rb_rs_reduce")
        self._reduced.add(chunk)

    # ---------------------------------------------------------------- phases 2-4
    def step(self, grad_scale: float = 1.0) -> torch.Tensor:
        """Finish the optimizer step; returns the global gradient norm (a device scalar on GPU)."""
        b, comm = self.b, self.comm
        for c in range(len(b.chunks)):
            if c not in self._reduced:
                self.reduce_chunk(c, grad_scale)
        self.step_count += 1
        b1, b2 = self.betas
        if not self.on_gpu:
            t = torch.tensor([self._sumsq_cpu], dtype=torch.float64)
            if comm.world > 1:
                dist.all_reduce(t, group=comm.group)
            norm = float(t.sqrt())
            coef = min(1.0, self.max_grad_norm / (norm + 1e-6)) if self.max_grad_norm > 0 else 1.0
            bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
            for c in range(len(b.chunks)):
                g = self.red[c] * coef
                self.exp_avg[c].mul_(b1).add_(g, alpha=1 - b1)
                self.exp_avg_sq[c].mul_(b2).addcmul_(g, g, value=1 - b2)
                p = self.master[c]
                p.mul_(1 - self.lr * self.weight_decay)
                p.addcdiv_(self.exp_avg[c] / bc1, (self.exp_avg_sq[c] / bc2).sqrt() + self.eps, value=-self.lr)
                off, length = b.chunks[c]
                if comm.world > 1:
                    parts = [torch.empty_like(p) for _ in range(comm.world)]
                    dist.all_gather(parts, p, group=comm.group)
                    b.params[off:off + length].copy_(torch.cat(parts).to(b.dtype))
                else:
                    b.params[off:off + length].copy_(p.to(b.dtype))
            b.grads.zero_()
            self._reduced.clear()
            self._sumsq_cpu = 0.0
            return torch.tensor(norm)
        dev = b.params.device
        st = status_tensor(dev).data_ptr()
        ep = comm.next_epoch(self.norm_slot)
        rc = _lib().rb_clip_coef(self.partial.data_ptr(), self.n_partial, comm.norm_slots.ptrs(), comm.flags.ptrs(),
                                 self.norm_slot, ep, comm.rank, comm.world, float(self.max_grad_norm),
                                 self.coef.data_ptr(), self.norm.data_ptr(), st, stream_handle(dev))
        check_rc(rc, "rb_clip_coef")
        for c in range(len(b.chunks)):
            off, length = b.chunks[c]
            n = length // comm.world
            rc = _lib().rb_adamw_allgather(
                self.master[c].data_ptr(), self.exp_avg[c].data_ptr(), self.exp_avg_sq[c].data_ptr(),
                self.red[c].data_ptr(), b.params_buf.ptrs(off * 2), comm.rank, comm.world, n, self.lr, b1, b2, self.eps,
                self.weight_decay, self.step_count, self.coef.data_ptr(), stream_handle(dev))
            check_rc(rc, "rb_adamw_allgather")
        comm.barrier()  # every rank's pushes landed; peers are done reading my gradients
        b.grads.zero_()
        self.partial.zero_()
        self._reduced.clear()
        return self.norm

    # ---------------------------------------------------------------- state
    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": [t.cpu() for t in self.master],
                "exp_avg": [t.cpu() for t in self.exp_avg], "exp_avg_sq": [t.cpu() for t in self.exp_avg_sq],
                "rank": self.comm.rank, "world": self.comm.world}

    def load_state_dict(self, sd: dict) -> None:
        assert sd["world"] == self.comm.world and sd["rank"] == self.comm.rank, "optimizer shards are per rank"
        self.step_count = sd["step"]
        for dst, src in ((self.master, sd["master"]), (self.exp_avg, sd["exp_avg"]), (self.exp_avg_sq, sd["exp_avg_sq"])):
            for d, s in zip(dst, src):
                d.copy_(s)


_ = ctypes
