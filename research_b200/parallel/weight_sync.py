"""Trainer -> engine weight synchronisation as ONE copy kernel over peer memory.

The trainer keeps its bf16 parameters in a flat (symmetric) bucket under Hugging Face names;
the engine keeps packed tensor-parallel buffers (fused ``q|k|v`` and ``gate|up`` matrices, row or
column slices per TP rank). ``WeightSyncPlan`` precomputes, once, a table of 2-D segments
``(src pointer, dst pointer, rows, cols, strides)`` that maps one layout onto the other; a sync
is then a single launch of ``reshard_copy`` which reads the trainer's memory (local, or another
GPU's over NVLink) and writes the engine's buffers in place - the broadcast and the resharding
copy are the same kernel, no state_dict gather, no per-tensor collective, no disk.

Replaces: ``torch.save`` to /dev/shm + ``POST /update_weights_from_disk``
(rollouts/training/grpo.py:459-474, training/weight_sync.py:34-146) and the per-parameter
``dist.broadcast`` path (training/weight_sync.py:233-282).
"""

from __future__ import annotations

import numpy as np
import torch

from ..ops._util import check_rc, stream_handle
from .symm import _lib

SEG_DTYPE = np.dtype([("src", "<u8"), ("dst", "<u8"), ("src_ld", "<i8"), ("dst_ld", "<i8"), ("rows", "<i4"),
                      ("cols", "<i4"), ("vec_begin", "<i8")])


class WeightSyncPlan:
    def __init__(self, runner, src_specs: dict, src_base_ptr: int, src_elem_size: int = 2,
                 shard_bases: list[int] | None = None):
        """``runner``: the engine's ModelRunner; ``src_specs``: name -> ParamSpec of the trainer's flat
        bucket; ``src_base_ptr``: address of that bucket as seen from the engine's GPU. ``shard_bases``: for a
        trainer with row-sharded parameters, the addresses of EVERY trainer rank's parameter storage as seen from
        the engine's GPU (rank q keeps rows ``[q R / W, (q + 1) R / W)`` of a sharded matrix); a segment that spans
        several slabs is cut at the slab boundaries, each piece read from its owner."""
        assert src_elem_size == 2, "weights travel as bf16"
        self.runner = runner
        self.device = runner.device
        segs: list[tuple[int, int, int, int, int, int]] = []
        cfg = runner.cfg
        tp, r = runner.tp_size, runner.tp_rank
        d = cfg.hidden_size

        def add(name, dst: torch.Tensor, rows, cols, row0=0, col0=0):
            s = src_specs[name]
            src_ld = s.shape[-1] if len(s.shape) > 1 else s.numel
            dst_ld = dst.stride(0) if dst.dim() > 1 else cols
            p_off = getattr(s, "p_offset", s.offset)
            assert cols % 8 == 0 and col0 % 8 == 0, f"{name}: columns must be multiples of 8 ({cols}, {col0})"
            if not getattr(s, "sharded", False):
                segs.append((src_base_ptr + (p_off + row0 * src_ld + col0) * 2, dst.data_ptr(), src_ld, dst_ld, rows, cols))
                return
            assert shard_bases is not None, f"{name} is row-sharded: the plan needs every trainer rank's address"
            part = s.shape[0] // len(shard_bases)            # rows per trainer rank
            row, end = row0, row0 + rows
            while row < end:
                q = row // part
                take = min(end, (q + 1) * part) - row
                segs.append((shard_bases[q] + (p_off + (row - q * part) * src_ld + col0) * 2,
                             dst.data_ptr() + (row - row0) * dst_ld * 2, src_ld, dst_ld, take, cols))
                row += take

        add("model.embed_tokens.weight", runner.embed, cfg.vocab_size, d)
        add("model.norm.weight", runner.final_norm, 1, d)
        if not cfg.tie_word_embeddings:
            add("lm_head.weight", runner.lm_head, cfg.vocab_size, d)
        qn, kn = runner.Hq * runner.D, runner.Hkv * runner.D
        for i, lw in enumerate(runner.layers):
            p = f"model.layers.{i}."
            add(p + "input_layernorm.weight", lw.ln1, 1, d)
            add(p + "post_attention_layernorm.weight", lw.ln2, 1, d)
            a = p + "self_attn."
            add(a + "q_proj.weight", lw.wqkv[:qn], qn, d, row0=r * qn)
            add(a + "k_proj.weight", lw.wqkv[qn:qn + kn], kn, d, row0=r * kn)
            add(a + "v_proj.weight", lw.wqkv[qn + kn:], kn, d, row0=r * kn)
            if lw.bqkv is not None:
                add(a + "q_proj.bias", lw.bqkv[:qn], 1, qn, col0=r * qn)
                add(a + "k_proj.bias", lw.bqkv[qn:qn + kn], 1, kn, col0=r * kn)
                add(a + "v_proj.bias", lw.bqkv[qn + kn:], 1, kn, col0=r * kn)
            if lw.q_norm is not None:
                add(a + "q_norm.weight", lw.q_norm, 1, runner.D)
                add(a + "k_norm.weight", lw.k_norm, 1, runner.D)
            add(a + "o_proj.weight", lw.wo, d, qn, col0=r * qn)
            m = p + "mlp."
            if lw.moe is not None:
                for name, dst, rows, cols, row0, col0 in lw.moe.sync_segments(m):
                    add(name, dst, rows, cols, row0, col0)
            else:
                F = runner.F
                if runner.fuse_swiglu:
                    hb = runner.swiglu_bn // 2   # interleaved blocks: hb gate rows then hb up rows
                    for j in range(F // hb):
                        add(m + "gate_proj.weight", lw.wgu[2 * j * hb:(2 * j + 1) * hb], hb, d, row0=r * F + j * hb)
                        add(m + "up_proj.weight", lw.wgu[(2 * j + 1) * hb:(2 * j + 2) * hb], hb, d, row0=r * F + j * hb)
                else:
                    add(m + "gate_proj.weight", lw.wgu[:F], F, d, row0=r * F)
                    add(m + "up_proj.weight", lw.wgu[F:], F, d, row0=r * F)
                add(m + "down_proj.weight", lw.wd, d, F, col0=r * F)
        _ = tp
        arr = np.zeros(len(segs), dtype=SEG_DTYPE)
        total = 0
        for j, (s_, d_, sld, dld, rows, cols) in enumerate(segs):
            arr[j] = (s_, d_, sld, dld, rows, cols, total)
            total += rows * cols // 8
        self.total_vecs = total
        self.n_segs = len(segs)
        self.bytes = total * 16
        self.table = torch.from_numpy(arr.view(np.uint8).copy()).to(self.device) if self.device.type == "cuda" else None
        self._segs = arr

    def run(self) -> None:
        """Copy every segment (one kernel on the current stream)."""
        if self.device.type != "cuda":
            raise RuntimeError("WeightSyncPlan.run needs a CUDA device; use ModelRunner.load_weights on CPU")
        rc = _lib().rb_reshard_copy(self.table.data_ptr(), self.n_segs, self.total_vecs, stream_handle(self.device))
        check_rc(rc, "rb_reshard_copy")


def sync_engine_from_buckets(engine, buckets, plan: WeightSyncPlan | None = None, src_rank: int | None = None,
                             comm=None) -> WeightSyncPlan | None:
    """Push the trainer's current parameters into ``engine`` and bump its weight version.

    Same process, same GPU: ``src_rank`` is None and the copy is local. Different GPUs of one node:
    ``buckets.params_buf`` is a symmetric buffer and ``src_rank`` names the trainer rank whose
    copy is read over NVLink. On CPU the engine falls back to ``load_weights`` on the views.
    """
    assert not engine.has_pending(), "weight sync while requests are in flight"
    buckets.finish_pending()      # a deferred optimizer step: every parameter chunk must be in place before it is read
    runner = engine.runner
    if runner.device.type != "cuda":
        runner.load_weights({name: buckets.param_view(name) for name in buckets.specs})
    else:
        if plan is None:
            base = buckets.params.data_ptr() if src_rank is None else buckets.params_buf.peer_ptrs[src_rank]
            plan = WeightSyncPlan(runner, buckets.specs, base,
                                  shard_bases=list(buckets.params_buf.peer_ptrs) if buckets.any_sharded else None)
        if comm is not None:
            comm.barrier()  # trainer finished writing the parameters
        plan.run()
        runner.fold_norm_weights()   # raw projections were just rewritten: fold the norm weights in again
        if comm is not None:
            comm.barrier()  # engines finished reading: the trainer may update again
    engine.weight_version += 1
    engine.flush_cache()
    return plan
