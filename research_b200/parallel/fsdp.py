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
    offset: int        # element offset inside the flat gradient bucket (always the full parameter)
    numel: int
    chunk: int
    p_offset: int = 0  # element offset inside this rank's parameter storage
    sharded: bool = False   # the parameter storage holds rows [rank * rows / world, (rank + 1) * rows / world) only
    owned: bool = False     # the parameter exists on this rank only (an expert of its expert-parallel share)


class FlatBuckets:
    """Flat bf16 parameter and gradient storage with per-parameter views.

    ``shard_rule(name, shape) -> bool`` marks matrices whose ROWS are split over the ranks (sharded-parameter
    training): the parameter storage of a rank then holds its row slab only, the gradient bucket still holds the
    full matrix (backward writes all of it, the reduce-scatter keeps this rank's slab). A chunk holds either sharded
    or unsharded parameters, never both; sharded chunks reduce and update slab by slab and push nothing to the
    peers, whose GEMM launches fetch the slabs when they need the matrix (``ShardedWeight``).

    ``owned_rule(name) -> bool`` marks parameters that exist on this rank ONLY (expert-parallel training: every rank
    lists its own experts, so the names differ between the ranks while the layout is the same). Their chunks are
    neither reduced over the ranks nor gathered: the owner computes the whole gradient (every token routed to the
    expert reaches it), keeps the whole optimizer state and updates in place."""

    def __init__(self, comm: PeerComm, named_shapes: list[tuple[str, tuple[int, ...]]], chunk_of=None,
                 dtype: torch.dtype = torch.bfloat16, shard_rule=None, param_comm: PeerComm | None = None,
                 with_grads: bool = True, owned_rule=None):
        """``param_comm``: allocate the parameter storage in the symmetric memory of ANOTHER (larger) group, so that
        ranks outside ``comm`` (inference engines on their own GPUs) can read it over NVLink; the members of ``comm``
        must be that group's first ranks, in order. ``with_grads=False``: a layout-only instance on such an outside
        rank (it takes part in the collective allocation and knows every offset, but holds no gradients)."""
        self.comm = comm
        W = comm.world
        align = 8 * W
        self.specs: dict[str, ParamSpec] = {}
        self.chunks: list[tuple[int, int]] = []  # (offset, length) per chunk in the gradient bucket, length % align == 0
        self.p_chunks: list[tuple[int, int]] = []  # the same chunks in this rank's parameter storage
        self.chunk_sharded: list[bool] = []
        self.chunk_owned: list[bool] = []
        off = p_off = 0
        cur_chunk, chunk_start, p_chunk_start, cur_sharded, cur_owned = None, 0, 0, False, False

        def close_chunk():
            nonlocal off, p_off
            off = -(-off // align) * align
            self.chunks.append((chunk_start, off - chunk_start))
            if not cur_sharded:
                p_off = p_chunk_start + (off - chunk_start)      # same layout as the gradient chunk
            self.p_chunks.append((p_chunk_start, p_off - p_chunk_start))
            self.chunk_sharded.append(cur_sharded)
            self.chunk_owned.append(cur_owned)

        for name, shape in named_shapes:
            c = chunk_of(name) if chunk_of else 0
            n = 1
            for s in shape:
                n *= s
            sharded = bool(shard_rule(name, tuple(shape))) if (shard_rule is not None and W > 1) else False
            owned = bool(owned_rule(name)) if (owned_rule is not None and W > 1) else False
            assert not (sharded and owned), f"{name}: a parameter is either row-sharded or owned by one rank"
            if sharded:
                assert len(shape) == 2 and shape[0] % W == 0 and (n // W) % 8 == 0, f"{name} {shape} cannot be row-sharded over {W}"
            if cur_chunk is None:
                cur_chunk, cur_sharded, cur_owned = c, sharded, owned
            if c != cur_chunk:
                close_chunk()
                chunk_start, p_chunk_start, cur_chunk, cur_sharded, cur_owned = off, p_off, c, sharded, owned
            assert sharded == cur_sharded, f"chunk {c} mixes sharded and unsharded parameters ({name})"
            assert owned == cur_owned, f"chunk {c} mixes replicated parameters and parameters owned by one rank ({name})"
            n_pad = -(-n // 8) * 8  # keep every parameter 16-byte aligned for TMA
            self.specs[name] = ParamSpec(name, tuple(shape), off, n, len(self.chunks),
                                         p_off if sharded else p_chunk_start + (off - chunk_start), sharded, owned)
            off += n_pad
            if sharded:
                p_off += n // W
        close_chunk()
        self.numel = off
        self.p_numel = p_off
        self.any_sharded = any(self.chunk_sharded)
        self.any_owned = any(self.chunk_owned)
        self.dtype = dtype
        self.params_buf = (param_comm or comm).alloc((self.p_numel,), dtype, zero=True)
        self.params = self.params_buf.local
        if with_grads:
            self.grads_buf = comm.alloc((self.numel,), dtype, zero=True)
            self.grads = self.grads_buf.local
        else:
            self.grads_buf = self.grads = None
        # Gradient windows: the kernels write a gradient view either over what is there (its first write of a
        # window) or on top of it (later micro-batches, tied weights), so the bucket is never zeroed as a whole.
        self.track_writes = False
        self._written: dict[int, int] = {}     # element offset -> end offset of views written in this window
        self._chunk_specs: list[list[ParamSpec]] = [[] for _ in self.chunks]
        for sp in self.specs.values():
            self._chunk_specs[sp.chunk].append(sp)
        # Parameter chunks whose update of the last optimizer step may still be running on another stream / arriving
        # from the peers: chunk -> (event recorded after this rank's update, flag slot, epoch every rank signals)
        self._pending: dict[int, tuple] = {}
        # sharded parameters are gathered into one staging matrix per GEMM launch (the largest sharded matrix)
        self.stage = None
        self._gather_epoch = 0
        if self.any_sharded:
            biggest = max(sp.numel for sp in self.specs.values() if sp.sharded)
            self.stage = torch.empty(biggest, dtype=dtype, device=self.params.device)
            if comm.on_gpu:
                self.gather_count = torch.zeros(64, dtype=torch.int32, device=self.params.device)    # [parts x pieces of a part]
                self.gather_ready = torch.zeros(64, dtype=torch.int32, device=self.params.device)

    # ---------------------------------------------------------------- deferred parameter updates
    def ensure_chunk(self, chunk: int) -> None:
        """Make the current stream wait until ``chunk``'s parameters of the last optimizer step are in place on this
        rank: its own update has run and every peer has pushed its slice (or, sharded chunks, updated its slabs)."""
        t = self._pending.pop(chunk, None)
        if t is not None:
            ev, slot, epoch = t
            torch.cuda.current_stream(self.params.device).wait_event(ev)
            if slot >= 0:
                self.comm.wait(slot, epoch)

    def finish_pending(self) -> None:
        for c in list(self._pending):
            self.ensure_chunk(c)

    def param_view(self, name: str) -> torch.Tensor:
        """The parameter as this rank stores it: the whole tensor, or (row-sharded) this rank's ``[rows / world, cols]`` slab."""
        if self._pending:
            self.finish_pending()
        s = self.specs[name]
        if s.sharded:
            n = s.numel // self.comm.world
            return self.params[s.p_offset:s.p_offset + n].view(s.shape[0] // self.comm.world, s.shape[1])
        return self.params[s.p_offset:s.p_offset + s.numel].view(s.shape)

    def full_param(self, name: str) -> torch.Tensor:
        """The whole parameter; for a row-sharded one a fresh tensor gathered from every rank (a collective on CPU
        groups: every rank must call it; peer reads on the GPU)."""
        if self._pending:
            self.finish_pending()
        s = self.specs[name]
        if not s.sharded:
            return self.param_view(name)
        W = self.comm.world
        mine = self.param_view(name)
        if not self.comm.on_gpu:
            parts = [torch.empty_like(mine) for _ in range(W)]
            dist.all_gather(parts, mine.contiguous(), group=self.comm.group)
            return torch.cat(parts, 0)
        n = s.numel // W
        parts = [self.params_buf.peer_tensor(r)[s.p_offset:s.p_offset + n].view(mine.shape) for r in range(W)]
        return torch.cat(parts, 0)

    def set_param(self, name: str, value: torch.Tensor) -> None:
        """Store ``value`` (the whole parameter) as this rank keeps it."""
        s = self.specs[name]
        v = value.to(device=self.params.device, dtype=self.dtype)
        if s.sharded:
            rows = s.shape[0] // self.comm.world
            v = v[self.comm.rank * rows:(self.comm.rank + 1) * rows]
        self.param_view(name).copy_(v)

    def sharded_weight(self, name: str) -> "ShardedWeight":
        return ShardedWeight(self, self.specs[name])

    def segments(self, chunk: int) -> list[tuple[int, int, int]]:
        """This rank's pieces of a sharded chunk: (offset in the gradient bucket, length, offset inside the rank's shard of the chunk)."""
        W, r = self.comm.world, self.comm.rank
        out, at = [], 0
        for sp in self._chunk_specs[chunk]:
            n = sp.numel // W
            out.append((sp.offset + r * n, n, at))
            at += n
        return out

    def grad_view(self, name: str) -> torch.Tensor:
        s = self.specs[name]
        return self.grads[s.offset:s.offset + s.numel].view(s.shape)

    # ---------------------------------------------------------------- gradient windows
    def begin_window(self) -> None:
        """Forget which gradient views were written: the next write of each view overwrites."""
        self._written.clear()

    def accumulate_into(self, gview: torch.Tensor) -> bool:
        """True when ``gview`` (a view of the gradient bucket) already holds this window's gradients, i.e. the
        caller must add to it; False on its first write of the window, which must overwrite. Without write
        tracking (CPU, or a caller that zeroes the bucket itself) every write accumulates."""
        if not self.track_writes:
            return True
        off = (gview.data_ptr() - self.grads.data_ptr()) // self.grads.element_size()
        end = off + gview.numel()
        prev = self._written.get(off)
        if prev is not None and prev >= end:
            return True
        self._written[off] = end
        return False

    def zero_unwritten(self, chunk: int) -> None:
        """Zero the gradient views of ``chunk`` that nothing wrote in this window (unused parameters, experts
        without tokens): what they hold is the previous step's gradient."""
        if not self.track_writes:
            return
        spans = sorted(self._written.items())
        for sp in self._chunk_specs[chunk]:
            covered = any(a <= sp.offset and sp.offset + sp.numel <= b for a, b in spans)
            if not covered:
                self.grads[sp.offset:sp.offset + sp.numel].zero_()

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
        self.on_gpu = self.comm.on_gpu
        # One rank on a GPU reduces nothing: AdamW reads the bf16 gradient bucket itself and no fp32 copy of the
        # gradients exists (4 bytes per parameter that an 8B model on one 180 GB GPU cannot spare).
        self.direct_grads = self.on_gpu and self.comm.world == 1
        self.master, self.exp_avg, self.exp_avg_sq, self.red = [], [], [], []
        for c in range(len(buckets.chunks)):
            off, n = self._param_shard_range(c)
            self.master.append(buckets.params[off:off + n].float().clone())
            self.exp_avg.append(torch.zeros(n, dtype=torch.float32, device=dev))
            self.exp_avg_sq.append(torch.zeros(n, dtype=torch.float32, device=dev))
            # owned chunks on a GPU keep no fp32 copy of their gradients either: nothing is summed over ranks, AdamW reads
            # the bf16 bucket and the 1 / world of the mean rides in its coefficient (4 bytes per expert parameter saved)
            direct = self.direct_grads or (self.on_gpu and buckets.chunk_owned[c])
            self.red.append(None if direct else torch.zeros(n, dtype=torch.float32, device=dev))
        self.zero_grads_after_step = True
        self.overlap_grid = 0          # CTAs of a reduce launch that shares the GPU with backward (0 = full grid)
        # With a stream here, AdamW and the parameter all-gather of a step run on it chunk by chunk, in the order the
        # next forward pass uses the chunks, and the forward waits chunk by chunk (FlatBuckets.ensure_chunk) instead
        # of after one barrier: the NVLink-bound pushes hide under the next step's first layers.
        self.update_stream = None
        self.update_order: list[int] | None = None
        if self.on_gpu:
            self.n_partial = _lib().rb_rs_num_partials()
            self.partial = torch.zeros(self.n_partial, dtype=torch.float32, device=dev)
            self.coef = torch.ones(1, dtype=torch.float32, device=dev)
            self.coef_owned = torch.ones(1, dtype=torch.float32, device=dev)     # coef / world, for chunks this rank owns
            self.norm = torch.zeros(1, dtype=torch.float32, device=dev)
            self.grad_slots = [self.comm.new_slot() for _ in buckets.chunks]    # one ready flag row per chunk
            self.param_slots = [self.comm.new_slot() for _ in buckets.chunks]
            self.norm_slot = self.comm.new_slot()
        self._reduced: set[int] = set()
        self._passes: dict[int, int] = {}     # reduce launches per chunk since the last step
        self._sumsq_cpu = 0.0

    def _param_shard_range(self, chunk: int) -> tuple[int, int]:
        """(offset, length) inside this rank's parameter storage of the elements whose optimizer state it owns: its
        even slice of an unsharded chunk, or everything it stores of a sharded one (its row slabs)."""
        b = self.b
        p_off, p_len = b.p_chunks[chunk]
        if b.chunk_sharded[chunk] or b.chunk_owned[chunk]:
            return p_off, p_len
        n = p_len // self.comm.world
        return p_off + self.comm.rank * n, n

    def resync_master(self) -> None:
        """Re-read the fp32 master slices from the bf16 parameters (after loading weights)."""
        for c in range(len(self.b.chunks)):
            off, n = self._param_shard_range(c)
            self.master[c].copy_(self.b.params[off:off + n].float())

    # ---------------------------------------------------------------- phase 1
    def reduce_chunk(self, chunk: int, grad_scale: float = 1.0, accumulate: bool = False, overlapped: bool = False) -> None:
        """Reduce-scatter one gradient chunk into this rank's fp32 slice (call once its backward is done).

        ``accumulate`` adds to what earlier passes of the same step reduced (several ``forward_backward`` calls per
        optimizer step); ``overlapped`` marks a launch that runs beside the backward pass on another stream: the wait
        for the peers' flags is then a one-CTA kernel of its own and the reduction uses ``overlap_grid`` CTAs."""
        b, comm = self.b, self.comm
        off, length = b.chunks[chunk]
        n = length // comm.world
        scale = grad_scale / comm.world
        sharded = b.chunk_sharded[chunk]
        owned = b.chunk_owned[chunk]
        if owned and self.on_gpu and overlapped:
            return      # nothing to fetch or copy for an owned chunk: its one pass (the norm) runs in step(), over the final sums
        b.zero_unwritten(chunk)
        self._passes[chunk] = self._passes.get(chunk, 0) + 1
        if not self.on_gpu:
            g = b.grads[off:off + length].float()
            if comm.world > 1 and not owned:
                dist.all_reduce(g, group=comm.group)
            if owned:
                mine = g * scale         # the owner holds the whole gradient already: only the 1 / world of the mean is left
            elif sharded:
                mine = torch.cat([g[o - off:o - off + m] for o, m, _ in b.segments(chunk)]) * scale
            else:
                mine = g[comm.rank * n:(comm.rank + 1) * n] * scale
            if accumulate:
                self.red[chunk].add_(mine)
            else:
                self.red[chunk].copy_(mine)
            self._reduced.add(chunk)
            return
        dev = b.params.device
        st = status_tensor(dev).data_ptr()
        ptrs = b.grads_buf.ptrs(off * 2)
        if self.direct_grads:
            # nothing to reduce: only this chunk's share of the gradient norm (the scale rides in the clip coefficient)
            rc = _lib().rb_rs_reduce_ex(ptrs, None, 0, 0, 0, 1, n, 1.0, None, 0, self.partial.data_ptr(), st, 0,
                                        stream_handle(dev))
            check_rc(rc, "rb_rs_reduce_ex")
            self._reduced.add(chunk)
            return
        if owned:
            # nothing to fetch from the peers: cast, scale and the chunk's share of the gradient norm, all local
            from .symm import ptr_array

            rc = _lib().rb_rs_reduce_ex(ptr_array([b.grads.data_ptr() + off * 2]), None, 0, 0, 0, 1, length, 1.0 / comm.world,
                                        None, 0, self.partial.data_ptr(), st, 0, stream_handle(dev))
            check_rc(rc, "rb_rs_reduce_ex")
            self._reduced.add(chunk)
            return
        slot = self.grad_slots[chunk]
        epoch = comm.signal(slot)  # my gradients for this chunk are final
        flags = comm.flags.local.data_ptr()
        if overlapped or sharded:
            comm.wait(slot, epoch)
            flags = None
        if sharded:
            # one launch per matrix: this rank's row slab of every peer's full gradient
            for g_off, m, at in b.segments(chunk):
                sp_base = g_off - comm.rank * m                    # start of the matrix in the gradient bucket
                rc = _lib().rb_rs_reduce_ex(b.grads_buf.ptrs(sp_base * 2), None, slot, epoch, comm.rank, comm.world, m, scale,
                                            self.red[chunk].data_ptr() + at * 4, int(accumulate), self.partial.data_ptr(), st,
                                            self.overlap_grid if overlapped else 0, stream_handle(dev))
                check_rc(rc, "rb_rs_reduce_ex")
            self._reduced.add(chunk)
            return
        rc = _lib().rb_rs_reduce_ex(ptrs, flags, slot, epoch, comm.rank, comm.world, n, scale,
                                    self.red[chunk].data_ptr(), int(accumulate), self.partial.data_ptr(), st,
                                    self.overlap_grid if overlapped else 0, stream_handle(dev))
        check_rc(rc, "rb_rs_reduce_ex")
        self._reduced.add(chunk)

    # ---------------------------------------------------------------- phases 2-4
    def step(self, grad_scale: float = 1.0) -> torch.Tensor:
        """Finish the optimizer step; returns the global gradient norm (a device scalar on GPU).

        ``grad_scale`` multiplies every gradient (1 / accumulated passes). Chunks that were reduced early carry the
        unscaled sums, so on the GPU the factor is applied with the clip coefficient."""
        b, comm = self.b, self.comm
        early = set(self._reduced)
        for c in range(len(b.chunks)):
            if c not in self._reduced:
                self.reduce_chunk(c, 1.0 if self.on_gpu else grad_scale)
        self.step_count += 1
        b1, b2 = self.betas
        if not self.on_gpu:
            if early and grad_scale != 1.0:
                for c in early:
                    self.red[c].mul_(grad_scale)
            sq = sum(float((self.red[c] * self.red[c]).sum()) for c in range(len(b.chunks)))
            t = torch.tensor([sq], dtype=torch.float64)
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
                off, length = b.p_chunks[c]
                if b.chunk_sharded[c] or b.chunk_owned[c]:
                    b.params[off:off + length].copy_(p.to(b.dtype))        # this rank's slabs / own experts; nothing is pushed
                elif comm.world > 1:
                    parts = [torch.empty_like(p) for _ in range(comm.world)]
                    dist.all_gather(parts, p, group=comm.group)
                    b.params[off:off + length].copy_(torch.cat(parts).to(b.dtype))
                else:
                    b.params[off:off + length].copy_(p.to(b.dtype))
            b.grads.zero_()
            self._reduced.clear()
            self._passes.clear()
            self._sumsq_cpu = 0.0
            return torch.tensor(norm)
        dev = b.params.device
        st = status_tensor(dev).data_ptr()
        if not self.direct_grads and any(v > 1 for v in self._passes.values()):
            # several reduce passes were summed into the fp32 slices: the partial sums of squares of the kernels
            # cover intermediate values, so take the norm from the slices themselves (rare path, plain tensor ops)
            self.partial.zero_()
            terms = [(r * r).sum() for r in self.red if r is not None]
            for c, owned in enumerate(b.chunk_owned):
                if owned:
                    off, length = b.chunks[c]
                    terms.append((b.grads[off:off + length].float() / comm.world).pow(2).sum())
            self.partial[0] = torch.stack(terms).sum()
        ep = comm.next_epoch(self.norm_slot)
        rc = _lib().rb_clip_coef_ex(self.partial.data_ptr(), self.n_partial, comm.norm_slots.ptrs(), comm.flags.ptrs(),
                                    self.norm_slot, ep, comm.rank, comm.world, float(self.max_grad_norm), float(grad_scale),
                                    self.coef.data_ptr(), self.norm.data_ptr(), st, stream_handle(dev))
        check_rc(rc, "rb_clip_coef_ex")
        if b.any_owned:
            torch.div(self.coef, float(comm.world), out=self.coef_owned)
        deferred = self.update_stream is not None
        order = self.update_order if self.update_order is not None else list(range(len(b.chunks)))
        # the clip kernel has consumed the partial sums: clear them on THIS stream, before anything of the next step
        # (its reductions run on this stream or, ordered behind the event below, on the update stream) adds to them
        self.partial.zero_()
        if deferred:
            ev = torch.cuda.Event()
            ev.record()
            self.update_stream.wait_event(ev)
            with torch.cuda.stream(self.update_stream):
                for c in order:
                    self._update_chunk(c, b1, b2)
                    # several ranks: tell the peers that my slice of chunk c is everywhere / my slabs are final
                    epoch = comm.signal(self.param_slots[c]) if comm.world > 1 else 0
                    done = torch.cuda.Event()
                    done.record()
                    b._pending[c] = (done, self.param_slots[c] if comm.world > 1 else -1, epoch)
        else:
            for c in order:
                self._update_chunk(c, b1, b2)
            comm.barrier()  # every rank's pushes landed; peers are done reading my gradients
        if self.zero_grads_after_step:
            b.grads.zero_()
        b.begin_window()
        self._reduced.clear()
        self._passes.clear()
        return self.norm

    def _update_chunk(self, c: int, b1: float, b2: float) -> None:
        """AdamW on this rank's share of chunk ``c`` (current stream), new bf16 values written where they live."""
        b, comm = self.b, self.comm
        dev = b.params.device
        p_off, p_len = b.p_chunks[c]
        if b.chunk_sharded[c] or b.chunk_owned[c]:
            # the rank owns everything it stores of this chunk: update in place, nothing is pushed (the peers'
            # GEMM launches fetch the slabs when they need the matrix)
            from .symm import ptr_array

            if b.chunk_owned[c]:      # the bf16 gradient bucket itself, scaled by coef / world inside the kernel
                grad_ptr, is_bf16, coef = b.grads.data_ptr() + b.chunks[c][0] * 2, 1, self.coef_owned
            else:
                grad_ptr, is_bf16, coef = self.red[c].data_ptr(), 0, self.coef
            rc = _lib().rb_adamw_allgather_ex(
                self.master[c].data_ptr(), self.exp_avg[c].data_ptr(), self.exp_avg_sq[c].data_ptr(),
                grad_ptr, is_bf16, ptr_array([b.params.data_ptr() + p_off * 2]), 0, 1, p_len, self.lr, b1, b2,
                self.eps, self.weight_decay, self.step_count, coef.data_ptr(), stream_handle(dev))
            check_rc(rc, "rb_adamw_allgather_ex")
            return
        off = b.chunks[c][0]
        n = p_len // comm.world
        grad_ptr = b.grads.data_ptr() + off * 2 if self.direct_grads else self.red[c].data_ptr()
        rc = _lib().rb_adamw_allgather_ex(
            self.master[c].data_ptr(), self.exp_avg[c].data_ptr(), self.exp_avg_sq[c].data_ptr(),
            grad_ptr, int(self.direct_grads), b.params_buf.ptrs(p_off * 2), comm.rank, comm.world, n, self.lr, b1, b2,
            self.eps, self.weight_decay, self.step_count, self.coef.data_ptr(), stream_handle(dev))
        check_rc(rc, "rb_adamw_allgather_ex")

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


class ShardedWeight:
    """Handle of one row-sharded matrix ``[rows, cols]``: where every rank keeps its slab, and the staging matrix a
    GEMM launch gathers it into (``ops.gemm`` with ``b_gather=`` for the launch that consumes it, ``carry_gather=`` for a
    launch that fetches it for the next one)."""

    def __init__(self, buckets: FlatBuckets, spec: ParamSpec):
        self.b, self.spec = buckets, spec
        W = buckets.comm.world
        self.rows, self.cols = spec.shape
        self.part_rows = self.rows // W
        self.part_bytes = (spec.numel // W) * 2
        self.peer_ptrs = [p + spec.p_offset * 2 for p in buckets.params_buf.peer_ptrs]
        self.rank, self.world = buckets.comm.rank, W

    @property
    def staged(self) -> torch.Tensor:
        """``[rows, cols]`` view of the staging buffer (valid after a launch that gathered THIS matrix, until the next gather)."""
        return self.b.stage[:self.spec.numel].view(self.rows, self.cols)

    def next_epoch(self) -> int:
        self.b._gather_epoch += 1
        return self.b._gather_epoch

    def local(self) -> torch.Tensor:
        return self.b.param_view(self.spec.name)


_ = ctypes
