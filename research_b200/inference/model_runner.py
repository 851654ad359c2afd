"""Kernel-backed execution of a decoder-only model over the paged KV cache.

The runner owns the packed bf16 weights (fused QKV and gate|up matrices, laid out once and
updated in place so captured CUDA graphs stay valid across weight syncs), the per-layer KV
cache ``[L, num_blocks, Hkv, 16, D]``, the RoPE table, and the static buffers of the decode
step. Two entry points:

* ``prefill``: packed varlen batch of new tokens (eager launches);
* ``decode``: one token per running sequence, replayed from a CUDA graph captured per batch
  size bucket (the reference has no graph capture and no batching:
  rollouts/inference/engine.py:218-246 runs ``model(input_ids)`` per sequence per token).

Every GEMM goes through the tcgen05 kernel (csrc/gemm_sm100.cu); attention, RMSNorm, RoPE+KV
append, SwiGLU and sampling are the kernels in csrc/attn_sm100.cu and csrc/ops_sm100.cu.
"""

from __future__ import annotations

import os

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..ops._util import LAUNCH_COUNT
from ..models.config import ModelConfig

BLOCK = 16


@dataclass
class StepBatch:
    """Host-side description of one packed batch (views into pinned staging memory)."""

    num_rows: int
    num_tokens: int
    max_new: int
    max_blocks: int


class LayerWeights:
    __slots__ = ("ln1", "wqkv", "bqkv", "q_norm", "k_norm", "wo", "ln2", "wgu", "wd", "moe")


class ModelRunner:
    def __init__(self, cfg: ModelConfig, weights: dict[str, torch.Tensor], *, device: torch.device,
                 num_kv_blocks: int, max_batch: int, max_model_len: int, max_prefill_tokens: int,
                 use_cuda_graphs: bool = True, graph_batch_sizes: tuple[int, ...] = (), tp=None, ep=None,
                 dtype: torch.dtype = torch.bfloat16):
        # On a CUDA device every op below is an sm_100a kernel. On CPU the same call sequence
        # runs the PyTorch reference twins of the ops (fp32), which is how the scheduler,
        # paged cache and radix reuse are exercised without a GPU.
        self.on_gpu = device.type == "cuda"
        if self.on_gpu:
            assert cfg.head_dim in (64, 128), "attention kernels are built for head_dim 64 and 128"
            assert dtype == torch.bfloat16, "the CUDA kernels are bf16"
        assert max_batch % 2 == 0 and max_prefill_tokens % 2 == 0
        use_cuda_graphs = use_cuda_graphs and self.on_gpu
        self.cfg = cfg
        self.device = device
        self.tp = tp
        # expert parallelism: attention and dense layers stay whole on every rank (each rank serves its own
        # requests), only the experts of the MoE layers are split; ``ep`` carries the peer-memory context
        self.ep = ep if ep is not None else (tp if getattr(tp, "expert_parallel", False) else None)
        self.tp_size = tp.world if tp is not None else 1
        self.tp_rank = tp.rank if tp is not None else 0
        assert cfg.num_heads % self.tp_size == 0 and cfg.num_kv_heads % self.tp_size == 0
        self.Hq = cfg.num_heads // self.tp_size
        self.Hkv = cfg.num_kv_heads // self.tp_size
        self.D = cfg.head_dim
        self.F = (cfg.intermediate_size // self.tp_size) if cfg.intermediate_size else 0
        self.max_batch = max_batch
        self.max_model_len = max_model_len
        self.max_blocks_per_seq = (max_model_len + BLOCK - 1) // BLOCK
        self.max_prefill_tokens = max_prefill_tokens
        self.num_kv_blocks = num_kv_blocks
        self.use_cuda_graphs = use_cuda_graphs
        self.graph_batch_sizes = tuple(sorted(b for b in graph_batch_sizes if b <= max_batch)) or (max_batch,)
        if self.graph_batch_sizes[-1] < max_batch:
            self.graph_batch_sizes += (max_batch,)
        self.scale = 1.0 / math.sqrt(self.D)
        self.launches_per_decode_step = 0
        # gate|up projection with SwiGLU fused into the GEMM epilogue: weights are stored
        # interleaved in blocks of 128 gate rows + 128 up rows (tile width 256)
        self.swiglu_bn = 256
        self.fuse_swiglu = self.on_gpu and self.F > 0 and self.F % (self.swiglu_bn // 2) == 0
        # RMSNorm folded into the GEMM that consumes it: the norm weight is multiplied into the projection's columns
        # when weights are loaded, the row statistic is computed inside the GEMM from its own A tiles and applied
        # in the epilogue, so the two normalisation launches of a layer disappear (input norm -> qkv, post-attention
        # norm -> gate|up of dense layers; MoE layers keep their norm kernel). The extra reads of the A tiles load
        # the shared-memory pipe that bounds long-K launches: measured per decode step 2.45 -> 2.40 ms at hidden
        # size 896 but 9.82 -> 9.91 ms at 4096, so only narrow models fold
        self.fold_norm = cfg.hidden_size <= 2048 and not os.environ.get("RB_NO_NORM_FOLD")
        # Tensor-parallel decode with the residual stream sharded by ROWS over the ranks ("sequence parallel"): the
        # column-parallel projections (q|k|v, gate|up, lm_head) gather the peers' normalised rows inside the GEMM
        # (all_gather_gemm: the A tiles of remote slabs are loaded from the peers' memory by the TMA producer) and the
        # row-parallel projections (o, down) end in a reduce-scatter epilogue that leaves every rank with its rows
        # of the new residual (gemm_reduce_scatter). No all-reduce, no replicated activations, no barrier between
        # layers. Chosen with RB_TP_MODE=sequence; the default keeps replicated activations and the fused
        # GEMM + all-reduce launches, which measured faster at 2 ranks (8B serving case, batch 64: 6.2 ms per step
        # against 14.3 ms) while every CTA of a gathered GEMM still fetched the remote rows itself.
        self.sp = (tp is not None and self.tp_size > 1 and not cfg.is_moe and not getattr(tp, "expert_parallel", False)
                   and os.environ.get("RB_TP_MODE", "allreduce") == "sequence")
        if self.sp:
            self.fuse_swiglu = False     # plain gate|up rows: the gathered GEMM has the ordinary epilogue
            self.fold_norm = False       # each rank normalises only its own rows, before they are gathered
        # fused GEMM+all-reduce works on row counts that split evenly into 8-row vectors per rank
        self.row_align = tp.row_align if tp is not None else 1
        if self.row_align > 1:
            ra = self.row_align
            assert max_batch % ra == 0, f"max_batch must be a multiple of {ra} with tensor parallelism"
            self.graph_batch_sizes = tuple(sorted({-(-b // ra) * ra for b in self.graph_batch_sizes}))

        bf = dtype
        self.dtype = dtype
        d, L = cfg.hidden_size, cfg.num_layers
        self.embed = torch.empty(cfg.vocab_size, d, dtype=bf, device=device)
        self.final_norm = torch.empty(d, dtype=bf, device=device)
        self.lm_head = self.embed if cfg.tie_word_embeddings else torch.empty(cfg.vocab_size, d, dtype=bf, device=device)
        self.layers: list[LayerWeights] = []
        qkv_rows = (self.Hq + 2 * self.Hkv) * self.D
        self.moe_scratch = None
        for i in range(L):
            lw = LayerWeights()
            lw.ln1 = torch.empty(d, dtype=bf, device=device)
            lw.ln2 = torch.empty(d, dtype=bf, device=device)
            lw.wqkv = torch.empty(qkv_rows, d, dtype=bf, device=device)
            lw.bqkv = torch.empty(qkv_rows, dtype=bf, device=device) if cfg.attention_bias else None
            lw.q_norm = torch.empty(self.D, dtype=bf, device=device) if cfg.qk_norm else None
            lw.k_norm = torch.empty(self.D, dtype=bf, device=device) if cfg.qk_norm else None
            lw.wo = torch.empty(d, self.Hq * self.D, dtype=bf, device=device)
            lw.moe = None
            if cfg.is_moe and i >= cfg.first_k_dense_replace:
                from ..parallel.moe import MoELayerWeights, MoEScratch

                lw.wgu = lw.wd = None
                if self.moe_scratch is None and self.on_gpu:
                    # one fixed-size scratch for all layers: captured graphs keep its addresses
                    self.moe_scratch = MoEScratch(cfg, device, self.ep, capacity=max(max_prefill_tokens, max_batch))
                lw.moe = MoELayerWeights(cfg, device, ep=self.ep, scratch=self.moe_scratch)
            else:
                lw.wgu = torch.empty(2 * self.F, d, dtype=bf, device=device)
                lw.wd = torch.empty(d, self.F, dtype=bf, device=device)
            self.layers.append(lw)
        self.load_weights(weights)

        # KV cache and RoPE table
        self.k_cache = torch.zeros(L, num_kv_blocks, self.Hkv, BLOCK, self.D, dtype=bf, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.rope = ops.rope_table(max_model_len, self.D, cfg.rope_theta, device=device)

        # ---- static decode buffers (graph inputs/outputs) ----
        mb = max_batch
        # one int32 staging vector: tokens | positions | slots | seq_lens | temps | seeds(lo,hi)
        self.meta_fields = 7
        self.meta_dev = torch.zeros(self.meta_fields * mb, dtype=torch.int32, device=device)
        self.meta_host = self._pinned(torch.zeros(self.meta_fields * mb, dtype=torch.int32))
        self.bt_dev = torch.zeros(mb, self.max_blocks_per_seq, dtype=torch.int32, device=device)
        self.bt_host = self._pinned(torch.zeros(mb, self.max_blocks_per_seq, dtype=torch.int32))
        self.out_dev = torch.zeros(2 * mb, dtype=torch.int32, device=device)
        self.out_host = self._pinned(torch.zeros(2 * mb, dtype=torch.int32))
        m = self.meta_dev
        self.d_tokens, self.d_pos, self.d_slots, self.d_lens = m[0:mb], m[mb:2 * mb], m[2 * mb:3 * mb], m[3 * mb:4 * mb]
        self.d_temps = m[4 * mb:5 * mb].view(torch.float32)
        self.d_seeds = m[5 * mb:7 * mb].view(torch.int64)
        self.d_out_tokens = self.out_dev[0:mb]
        self.d_out_logprobs = self.out_dev[mb:2 * mb].view(torch.float32)
        # activations for decode
        self.a_x = tp.alloc((mb, d), bf) if (tp is not None and self.on_gpu) else torch.empty(mb, d, dtype=bf, device=device)
        self.a_h = torch.empty(mb, d, dtype=bf, device=device)
        if self.sp:
            rows = mb // self.tp_size
            self.a_xs = torch.empty(rows, d, dtype=bf, device=device)                       # this rank's rows of the residual
            self.a_hs = tp.alloc((rows, d), bf) if self.on_gpu else torch.empty(rows, d, dtype=bf, device=device)  # read by the peers
            self._sp_slot = tp.comm.new_slot() if self.on_gpu else 0
        self.a_qkv = torch.empty(mb, qkv_rows, dtype=bf, device=device)
        self.a_q = torch.empty(mb, self.Hq * self.D, dtype=bf, device=device)
        self.a_attn = torch.empty(mb, self.Hq * self.D, dtype=bf, device=device)
        self.a_gu = torch.empty(mb, 2 * self.F, dtype=bf, device=device) if self.F else None
        self.a_act = torch.empty(mb, self.F, dtype=bf, device=device) if self.F else None
        self.a_logits = torch.empty(mb, cfg.vocab_size, dtype=torch.float32, device=device)
        # off by default: with four epilogue warps per SM the per-element sampling arithmetic (hash, two logs, exp)
        # is latency-bound and the fused launch measured 0.1 ms slower per 0.5B decode step than GEMM + sampler
        self.fused_sample = self.on_gpu and bool(os.environ.get("RB_FUSED_SAMPLE"))
        self.sample_ws = ops.lm_head_sample_workspace(mb, cfg.vocab_size, device) if self.fused_sample else None
        # split-KV partials for small batches (up to 64 rows x 32 splits)
        self.dec_ws = torch.empty(min(mb, 64) * self.Hq * 32 * (self.D + 2), dtype=torch.float32, device=device)
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.launches_per_graph: dict[int, int] = {}
        self.graph_pool = None

        # prefill staging (pinned): tokens | positions | slots | cu_q | seq_lens | sample_rows | temps | seeds
        T = max_prefill_tokens
        self.pf_host = self._pinned(torch.zeros(3 * T + 6 * (mb + 1), dtype=torch.int32))
        self.pf_dev = torch.zeros_like(self.pf_host, device=device)
        # residual stream of the prefill pass; symmetric when ranks all-reduce into it
        self.pf_x = tp.alloc((T + self.row_align, d), bf) if (tp is not None and self.on_gpu) else None

    def _pinned(self, t: torch.Tensor) -> torch.Tensor:
        return t.pin_memory() if self.on_gpu else t

    # ------------------------------------------------------------------ weights
    def _shard_rows(self, w: torch.Tensor, parts: int, idx: int) -> torch.Tensor:
        n = w.shape[0] // parts
        return w[idx * n:(idx + 1) * n]

    def load_weights(self, weights: dict[str, torch.Tensor]) -> None:
        """Copy HF-named tensors into the packed device buffers (in place)."""
        cfg, tp, r = self.cfg, self.tp_size, self.tp_rank
        dev = self.device

        def put(dst: torch.Tensor, src: torch.Tensor) -> None:
            dst.copy_(src.to(device=dev, dtype=dst.dtype, non_blocking=True))

        put(self.embed, weights["model.embed_tokens.weight"])
        put(self.final_norm, weights["model.norm.weight"])
        if not cfg.tie_word_embeddings:
            put(self.lm_head, weights["lm_head.weight"])
        qn, kn = self.Hq * self.D, self.Hkv * self.D
        for i, lw in enumerate(self.layers):
            p = f"model.layers.{i}."
            put(lw.ln1, weights[p + "input_layernorm.weight"])
            put(lw.ln2, weights[p + "post_attention_layernorm.weight"])
            a = p + "self_attn."
            put(lw.wqkv[:qn], self._shard_rows(weights[a + "q_proj.weight"], tp, r))
            put(lw.wqkv[qn:qn + kn], self._shard_rows(weights[a + "k_proj.weight"], tp, r))
            put(lw.wqkv[qn + kn:], self._shard_rows(weights[a + "v_proj.weight"], tp, r))
            if lw.bqkv is not None:
                put(lw.bqkv[:qn], self._shard_rows(weights[a + "q_proj.bias"], tp, r))
                put(lw.bqkv[qn:qn + kn], self._shard_rows(weights[a + "k_proj.bias"], tp, r))
                put(lw.bqkv[qn + kn:], self._shard_rows(weights[a + "v_proj.bias"], tp, r))
            if lw.q_norm is not None:
                put(lw.q_norm, weights[a + "q_norm.weight"])
                put(lw.k_norm, weights[a + "k_norm.weight"])
            wo = weights[a + "o_proj.weight"]
            cols = wo.shape[1] // tp
            put(lw.wo, wo[:, r * cols:(r + 1) * cols])
            m = p + "mlp."
            if lw.moe is not None:
                lw.moe.load(weights, m)
            else:
                g_ = self._shard_rows(weights[m + "gate_proj.weight"], tp, r)
                u_ = self._shard_rows(weights[m + "up_proj.weight"], tp, r)
                if self.fuse_swiglu:
                    put(lw.wgu, ops.gemm_mod.interleave_gate_up(g_.to(dev), u_.to(dev), self.swiglu_bn))
                else:
                    put(lw.wgu[:self.F], g_)
                    put(lw.wgu[self.F:], u_)
                wd = weights[m + "down_proj.weight"]
                cols = wd.shape[1] // tp
                put(lw.wd, wd[:, r * cols:(r + 1) * cols])
        self.fold_norm_weights()

    def fold_norm_weights(self) -> None:
        """Multiply the norm weights into the columns of the projections that consume the normalised activations.
        Must follow every write of raw weights into ``wqkv`` / ``wgu`` (load and trainer -> engine sync)."""
        if not self.fold_norm:
            return
        for lw in self.layers:
            lw.wqkv.mul_(lw.ln1[None, :])
            if lw.moe is None:
                lw.wgu.mul_(lw.ln2[None, :])

    # ------------------------------------------------------------------ layer math
    def _mlp(self, lw: LayerWeights, h: torch.Tensor, x: torch.Tensor, n: int, static: bool) -> None:
        """x += MLP(post-attention norm of x) for the first n rows; ``h`` is scratch for the normalised rows."""
        cfg = self.cfg
        if lw.moe is not None:
            ops.rmsnorm(x[:n], lw.ln2, cfg.rms_norm_eps, out=h[:n])
            lw.moe.forward(h[:n], x[:n])
            return
        if self.fold_norm:
            src, eps = x, cfg.rms_norm_eps
        else:
            ops.rmsnorm(x[:n], lw.ln2, cfg.rms_norm_eps, out=h[:n])
            src, eps = h, None
        gu = self.a_gu[:n] if static else None
        act = self.a_act[:n] if static else None
        if self.fuse_swiglu:
            act = ops.gemm(src[:n], lw.wgu, out=act, bn=self.swiglu_bn, swiglu=True, norm_eps=eps)
        else:
            gu = ops.gemm(src[:n], lw.wgu, out=gu, norm_eps=eps)
            act = ops.swiglu(gu, out=act)
        self._row_parallel(act, lw.wd, x[:n])

    def _row_parallel(self, a: torch.Tensor, w: torch.Tensor, x: torch.Tensor) -> None:
        """x += a @ w.T, summed over tensor-parallel ranks when sharded."""
        if self.tp is None or self.tp_size == 1:
            ops.gemm(a, w, residual=x, out=x)
        else:
            self.tp.gemm_all_reduce(a, w, x)

    def _forward_layers(self, x, h, n, positions, slots, attn_fn, static: bool):
        cfg = self.cfg
        for li, lw in enumerate(self.layers):
            if self.fold_norm:
                qkv = ops.gemm(x[:n], lw.wqkv, bias=lw.bqkv, out=self.a_qkv[:n] if static else None, norm_eps=cfg.rms_norm_eps)
            else:
                ops.rmsnorm(x[:n], lw.ln1, cfg.rms_norm_eps, out=h[:n])
                qkv = ops.gemm(h[:n], lw.wqkv, bias=lw.bqkv, out=self.a_qkv[:n] if static else None)
            q = ops.rope_kv_append(qkv, positions, slots, self.rope, self.k_cache[li], self.v_cache[li], self.Hq,
                                   self.Hkv, self.D, lw.q_norm, lw.k_norm, cfg.rms_norm_eps,
                                   q_out=self.a_q[:n] if static else None)
            attn = attn_fn(li, q.view(n, self.Hq, self.D))
            self._row_parallel(attn.view(n, self.Hq * self.D), lw.wo, x[:n])
            self._mlp(lw, h, x, n, static)

    # ------------------------------------------------------------------ decode
    def _decode_body_sp(self, bk: int) -> None:
        """One decode step with the residual stream sharded by rows (see ``self.sp``)."""
        cfg, tp = self.cfg, self.tp
        P, r = self.tp_size, self.tp_rank
        rpr = bk // P
        xs, hs = self.a_xs[:rpr], self.a_hs[:rpr]
        eps = cfg.rms_norm_eps
        ops.embedding(self.d_tokens[r * rpr:(r + 1) * rpr], self.embed, out=xs)
        splits = ops.decode_num_splits(bk, self.Hkv, self.max_model_len, head_dim=self.D)
        if bk > 64:
            splits = 1
        bt, lens = self.bt_dev[:bk], self.d_lens[:bk]

        def gathered(w, out, bias=None, out_f32=False):
            tp.publish_device()            # hs holds this rank's rows: tell the peers (epoch counted on the device)
            return tp.all_gather_gemm(hs, w, out, bias=bias, ready_epoch="device", out_f32=out_f32)

        for li, lw in enumerate(self.layers):
            ops.rmsnorm(xs, lw.ln1, eps, out=hs)
            qkv = gathered(lw.wqkv, self.a_qkv[:bk], lw.bqkv)
            q = ops.rope_kv_append(qkv, self.d_pos[:bk], self.d_slots[:bk], self.rope, self.k_cache[li], self.v_cache[li],
                                   self.Hq, self.Hkv, self.D, lw.q_norm, lw.k_norm, eps, q_out=self.a_q[:bk])
            attn = ops.paged_decode(q.view(bk, self.Hq, self.D), self.k_cache[li], self.v_cache[li], bt, lens, self.scale,
                                    splits, out=self.a_attn[:bk].view(bk, self.Hq, self.D), workspace=self.dec_ws)
            # a rank gets the last partial of its rows only after every peer has finished the GEMM above, so hs may
            # be rewritten once this returns
            tp.gemm_reduce_scatter(attn.view(bk, self.Hq * self.D), lw.wo, xs, residual=xs)
            ops.rmsnorm(xs, lw.ln2, eps, out=hs)
            gu = gathered(lw.wgu, self.a_gu[:bk])
            act = ops.swiglu(gu, out=self.a_act[:bk])
            tp.gemm_reduce_scatter(act, lw.wd, xs, residual=xs)
        ops.rmsnorm(xs, self.final_norm, eps, out=hs)
        logits = gathered(self.lm_head, self.a_logits[:bk], out_f32=True)
        self._sample(logits, self.d_temps[:bk], self.d_seeds[:bk], bk)
        tp.comm.barrier(self._sp_slot)     # every peer has read hs: the next step may overwrite it

    def _decode_body(self, bk: int) -> None:
        if self.sp:
            self._decode_body_sp(bk)
            return
        cfg = self.cfg
        x, h = self.a_x, self.a_h
        ops.embedding(self.d_tokens[:bk], self.embed, out=x[:bk])
        splits = ops.decode_num_splits(bk, self.Hkv, self.max_model_len, head_dim=self.D)
        if bk > 64:
            splits = 1
        bt = self.bt_dev[:bk]
        lens = self.d_lens[:bk]

        def attn_fn(li, q):
            return ops.paged_decode(q, self.k_cache[li], self.v_cache[li], bt, lens, self.scale, splits,
                                    out=self.a_attn[:bk].view(bk, self.Hq, self.D), workspace=self.dec_ws)

        self._forward_layers(x, h, bk, self.d_pos[:bk], self.d_slots[:bk], attn_fn, static=True)
        ops.rmsnorm(x[:bk], self.final_norm, cfg.rms_norm_eps, out=h[:bk])
        self._lm_head_sample(h[:bk], self.d_temps[:bk], self.d_seeds[:bk], bk)

    def _lm_head_sample(self, h, temps, seeds, n: int) -> None:
        """Final projection + sampling. On the GPU one GEMM whose epilogue reduces each tile to a sampling record
        (no [n, vocab] fp32 logits are written), then a merge kernel (RB_FUSED_SAMPLE=1); default is the GEMM followed by
        the sampling kernel, which measured faster."""
        if self.on_gpu and self.fused_sample:
            ops.lm_head_sample(h, self.lm_head, temps, seeds, 0, None, self.d_out_tokens[:n], self.d_out_logprobs[:n],
                               workspace=self.sample_ws)
            return
        logits = ops.gemm(h, self.lm_head, out=self.a_logits[:n], out_f32=True)
        self._sample(logits, temps, seeds, n)

    def _sample(self, logits, temps, seeds, n: int) -> None:
        if self.on_gpu:
            ops.sample_with_logprobs(logits, temps, seeds, 0, None, self.d_out_tokens[:n], self.d_out_logprobs[:n])
            return
        # CPU twin: one seeded generator per row so a request reproduces in any batch slot
        for r in range(n):
            g = torch.Generator().manual_seed(int(seeds[r].item()) & 0x7FFFFFFFFFFFFFFF)
            tok, lp = ops.sample_with_logprobs_reference(logits[r:r + 1].float(), temps[r:r + 1], g)
            self.d_out_tokens[r] = int(tok[0])
            self.d_out_logprobs[r] = float(lp[0])

    def bucket(self, n: int) -> int:
        for b in self.graph_batch_sizes:
            if b >= n:
                return b
        return self.max_batch

    def capture_graphs(self) -> None:
        """Capture one decode graph per batch-size bucket (largest first, shared memory pool)."""
        if not self.use_cuda_graphs:
            return
        self.d_lens.zero_()
        self.d_slots.fill_(-1)
        torch.cuda.synchronize(self.device)
        stream = torch.cuda.Stream(self.device)
        ops.set_pdl(True)  # decode kernels overlap their prologue with the previous kernel's tail
        with torch.cuda.stream(stream):
            for bk in sorted(self.graph_batch_sizes, reverse=True):
                self._decode_body(bk)  # warm-up: sets kernel attributes outside capture
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                n0 = LAUNCH_COUNT[0]
                with torch.cuda.graph(g, pool=self.graph_pool, stream=stream):
                    self._decode_body(bk)
                self.launches_per_graph[bk] = LAUNCH_COUNT[0] - n0
                if self.graph_pool is None:
                    self.graph_pool = g.pool()
                self.graphs[bk] = g
        ops.set_pdl(False)
        torch.cuda.synchronize(self.device)
        ops.check_status(self.device)

    def decode(self, n: int, max_blocks: int) -> None:
        """Run one decode step for the ``n`` rows staged in ``meta_host`` / ``bt_host``.

        Host->device: one copy of the packed metadata vector and one 2-D copy of the used
        block-table columns. Device->host: one copy of tokens|logprobs into ``out_host``.
        The caller synchronises before reading ``out_host``.
        """
        bk = self.bucket(n) if (self.use_cuda_graphs or self.row_align > 1) else max(n, 1)
        self.meta_dev.copy_(self.meta_host, non_blocking=True)
        self.bt_dev[:n, :max_blocks].copy_(self.bt_host[:n, :max_blocks], non_blocking=True)
        g = self.graphs.get(bk)
        if g is not None:
            g.replay()
        else:
            self._decode_body(bk)
        self.out_host.copy_(self.out_dev, non_blocking=True)

    def stage_decode_padding(self, n: int) -> None:
        """Mark rows n..bucket as padding (no KV write, empty context)."""
        bk = self.bucket(n) if (self.use_cuda_graphs or self.row_align > 1) else max(n, 1)
        mb = self.max_batch
        mh = self.meta_host
        if bk > n:
            mh[0 * mb + n:0 * mb + bk] = 0
            mh[1 * mb + n:1 * mb + bk] = 0
            mh[2 * mb + n:2 * mb + bk] = -1
            mh[3 * mb + n:3 * mb + bk] = 0
            mh[4 * mb + n:4 * mb + bk] = 0

    # ------------------------------------------------------------------ prefill
    def prefill(self, rows: int, T: int, max_new: int, max_blocks: int, views: dict[str, torch.Tensor]) -> None:
        """Packed varlen prefill of ``T`` new tokens over ``rows`` sequences.

        ``views`` are slices of ``pf_host`` filled by the engine core. Results land in
        ``out_host[:rows]`` / ``out_host[max_batch:max_batch+rows]`` after a synchronise.
        """
        cfg = self.cfg
        dev = self.device
        o = self._pf_offsets()
        Tp = -(-T // self.row_align) * self.row_align  # padded row count (tensor parallel only)
        if Tp > T:
            ph = self.pf_host
            ph[o["tokens"] + T:o["tokens"] + Tp] = 0
            ph[o["positions"] + T:o["positions"] + Tp] = 0
            ph[o["slots"] + T:o["slots"] + Tp] = -1   # padding rows never touch the KV cache
        self.pf_dev.copy_(self.pf_host, non_blocking=True)
        self.bt_dev[:rows, :max_blocks].copy_(self.bt_host[:rows, :max_blocks], non_blocking=True)
        pd = self.pf_dev
        tokens = pd[o["tokens"]:o["tokens"] + Tp]
        positions = pd[o["positions"]:o["positions"] + Tp]
        slots = pd[o["slots"]:o["slots"] + Tp]
        cu_q = pd[o["cu_q"]:o["cu_q"] + rows + 1]
        seq_lens = pd[o["seq_lens"]:o["seq_lens"] + rows]
        sample_rows = pd[o["sample_rows"]:o["sample_rows"] + rows]
        temps = pd[o["temps"]:o["temps"] + rows].view(torch.float32)
        seeds = pd[o["seeds"]:o["seeds"] + 2 * rows].view(torch.int64)
        x = ops.embedding(tokens, self.embed, out=self.pf_x[:Tp] if self.pf_x is not None else None)
        h = torch.empty_like(x)
        bt = self.bt_dev[:rows]
        attn_out = torch.zeros(Tp, self.Hq, self.D, dtype=x.dtype, device=dev) if Tp > T else None

        def attn_fn(li, q):
            return ops.paged_prefill(q, self.k_cache[li], self.v_cache[li], bt, cu_q, seq_lens, max_new, self.scale,
                                     cfg.sliding_window, out=attn_out)

        self._forward_layers(x, h, Tp, positions, slots, attn_fn, static=False)
        last = ops.embedding(sample_rows, x)  # row gather of the last token of every sequence
        hl = ops.rmsnorm(last, self.final_norm, cfg.rms_norm_eps)
        self._lm_head_sample(hl, temps, seeds, rows)
        self.out_host.copy_(self.out_dev, non_blocking=True)
        _ = dev

    def _pf_offsets(self) -> dict[str, int]:
        T, mb = self.max_prefill_tokens, self.max_batch
        return {"tokens": 0, "positions": T, "slots": 2 * T, "cu_q": 3 * T, "seq_lens": 3 * T + (mb + 1),
                "sample_rows": 3 * T + 2 * (mb + 1), "temps": 3 * T + 3 * (mb + 1), "seeds": 3 * T + 4 * (mb + 1)}

    # ------------------------------------------------------------------ teacher forcing
    def score(self, token_ids: torch.Tensor) -> torch.Tensor:
        """Full-sequence logits ``[T, V]`` (fp32) for one sequence, without touching live KV blocks.

        Uses the tail of the KV pool as scratch blocks; meant for tests and logprob checks.
        """
        T = token_ids.numel()
        nblk = (T + BLOCK - 1) // BLOCK
        assert nblk <= self.num_kv_blocks
        dev = self.device
        blocks = torch.arange(self.num_kv_blocks - nblk, self.num_kv_blocks, dtype=torch.int32, device=dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        slots = blocks[torch.div(pos, BLOCK, rounding_mode="floor").long()] * BLOCK + pos % BLOCK
        bt = blocks[None].contiguous()
        cu_q = torch.tensor([0, T], dtype=torch.int32, device=dev)
        lens = torch.tensor([T], dtype=torch.int32, device=dev)
        x = ops.embedding(token_ids.to(device=dev, dtype=torch.int32), self.embed)
        h = torch.empty_like(x)

        def attn_fn(li, q):
            return ops.paged_prefill(q, self.k_cache[li], self.v_cache[li], bt, cu_q, lens, T, self.scale,
                                     self.cfg.sliding_window)

        self._forward_layers(x, h, T, pos, slots.to(torch.int32), attn_fn, static=False)
        hl = ops.rmsnorm(x, self.final_norm, self.cfg.rms_norm_eps)
        return ops.gemm(hl, self.lm_head, out_f32=True)
