"""Trainable decoder whose forward AND backward run on the sm_100a kernels.

Parameters are views into a flat bf16 bucket (``parallel.fsdp.FlatBuckets``); gradients are
accumulated by the kernels straight into the matching views of the gradient bucket (the wgrad
GEMM's epilogue adds into it), so autograd never allocates or copies a weight gradient and
the sharded optimizer can reduce-scatter the bucket in place.

GEMMs: forward ``x @ W^T``; dgrad ``dY @ W`` (B operand MN-major); wgrad ``dY^T @ X`` (both
operands MN-major) - one tcgen05 kernel, no transposes. The lm_head and the loss are fused
and chunked: logits exist only as one ``[rows, V]`` fp32 chunk at a time, from which the
kernel takes per-token log-probability and entropy (forward) and writes bf16 dlogits
(backward); the ``[B,T,V]`` log-softmax of the reference (rollouts/training/losses.py:110-124)
is never materialised.

On CPU the same class evaluates the functional oracle with autograd, which is what the gloo
multi-rank tests train.

Attention core: the tcgen05 flash attention kernels (forward and backward) for head sizes 64 and
128; other head sizes (tiny test models) fall back to ``scaled_dot_product_attention``.
"""

from __future__ import annotations

import math
import os
import re
from collections.abc import Mapping

import torch
import torch.nn.functional as F

from .. import ops
from ..models.config import ModelConfig
from ..models.functional import causal_lm_forward
from ..ops import train as T
from ..ops.flash import flash_attention


# ------------------------------------------------------------------------------ autograd glue
def _rows_ok(t: torch.Tensor) -> torch.Tensor:
    """The GEMM takes any row stride (16-byte aligned rows, unit column stride): only other layouts are copied."""
    if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


class _Linear(torch.autograd.Function):
    """``y = x W^T (+ bias) (+ residual)``; the residual add rides in the GEMM epilogue and its gradient is ``dy``.

    ``sink`` is the gradient bucket: it knows whether a gradient view already holds this window's gradient (the
    wgrad GEMM then adds to it through its residual input) or is written for the first time (plain store, so the
    bucket is never zeroed or re-read as a whole)."""

    @staticmethod
    def forward(ctx, x, w, gw, bias, gb, residual, sink):
        ctx.save_for_backward(x, w)
        ctx.gw, ctx.gb, ctx.has_res, ctx.sink = gw, gb, residual is not None, sink
        return ops.gemm(x, w, bias=bias, residual=residual)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = _rows_ok(dy)
        dx = ops.gemm(dy, w, b_mn_major=True) if ctx.needs_input_grad[0] else None   # [M,N] x [N,K] -> [M,K]
        acc = ctx.sink.accumulate_into(ctx.gw)
        ops.gemm(dy, x, residual=ctx.gw if acc else None, out=ctx.gw, a_mn_major=True, b_mn_major=True)  # gw (+)= dY^T X
        if ctx.gb is not None:
            db = dy.float().sum(0).to(ctx.gb.dtype)
            if ctx.sink.accumulate_into(ctx.gb):
                ctx.gb.add_(db)
            else:
                ctx.gb.copy_(db)
        return dx, None, None, None, None, (dy if ctx.has_res else None), None


class _ShardedLinear(torch.autograd.Function):
    """``y = x W^T (+ bias) (+ residual)`` for a row-sharded ``W`` (``parallel.fsdp.ShardedWeight``).

    Forward: ONE launch gathers the peers' row slabs of ``W`` into the local staging matrix and multiplies, its tiles
    starting part by part as the slabs land (what FSDP2's pre-forward all-gather + ``F.linear`` do in the reference,
    rollouts/training/backends/fsdp.py:289-322). Backward: the weight-gradient launch (which does not need ``W``)
    carries the gather for the data-gradient launch right behind it. ``W`` is never saved for backward."""

    @staticmethod
    def forward(ctx, x, w, gw, bias, gb, residual, sink):
        ctx.save_for_backward(x)
        ctx.w, ctx.gw, ctx.gb, ctx.has_res, ctx.sink = w, gw, gb, residual is not None, sink
        return ops.gemm(x, None, bias=bias, residual=residual, b_gather=w)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = _rows_ok(dy)
        acc = ctx.sink.accumulate_into(ctx.gw)
        need_dx = ctx.needs_input_grad[0]
        ops.gemm(dy, x, residual=ctx.gw if acc else None, out=ctx.gw, a_mn_major=True, b_mn_major=True,
                 carry_gather=ctx.w if need_dx else None)                       # gw (+)= dY^T X, and W arrives
        dx = ops.gemm(dy, ctx.w.staged, b_mn_major=True) if need_dx else None   # [M,N] x [N,K] -> [M,K]
        if ctx.gb is not None:
            db = dy.float().sum(0).to(ctx.gb.dtype)
            if ctx.sink.accumulate_into(ctx.gb):
                ctx.gb.add_(db)
            else:
                ctx.gb.copy_(db)
        return dx, None, None, None, None, (dy if ctx.has_res else None), None


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, gw, eps, sink):
        ctx.save_for_backward(x, w)
        ctx.gw, ctx.eps, ctx.sink = gw, eps, sink
        return ops.rmsnorm(x, w, eps)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx, dw = T.rmsnorm_bwd(x, w, dy.contiguous(), ctx.eps)
        if ctx.sink.accumulate_into(ctx.gw):
            ctx.gw.add_(dw.to(ctx.gw.dtype))
        else:
            ctx.gw.copy_(dw)
        return dx, None, None, None, None


class _RoPE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, table):
        ctx.save_for_backward(positions, table)
        return T.rope(x, positions, table, backward=False)

    @staticmethod
    def backward(ctx, dy):
        positions, table = ctx.saved_tensors
        return T.rope(dy.contiguous(), positions, table, backward=True), None, None


class _SplitQKVRope(torch.autograd.Function):
    """One fused ``[T, (H + 2 Hkv) D]`` projection -> rotated ``q [T,H,D]``, rotated ``k [T,Hkv,D]`` and ``v`` (a view of
    the input). The rotation kernel reads the strided slices in place; backward rotates ``dq`` / ``dk`` back straight
    into the matching columns of one ``d_qkv`` buffer, so the split costs no copy in either direction."""

    @staticmethod
    def forward(ctx, qkv, positions, table, H, Hkv, D):
        ctx.save_for_backward(positions, table)
        ctx.dims = (H, Hkv, D)
        Tn = qkv.shape[0]
        q = T.rope(qkv[:, :H * D].view(Tn, H, D), positions, table, backward=False)
        k = T.rope(qkv[:, H * D:(H + Hkv) * D].view(Tn, Hkv, D), positions, table, backward=False)
        v = qkv[:, (H + Hkv) * D:].view(Tn, Hkv, D)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        positions, table = ctx.saved_tensors
        H, Hkv, D = ctx.dims
        Tn = dq.shape[0]
        d_qkv = torch.empty(Tn, (H + 2 * Hkv) * D, dtype=dq.dtype, device=dq.device)
        T.rope(dq.contiguous(), positions, table, backward=True, out=d_qkv[:, :H * D].view(Tn, H, D))
        T.rope(dk.contiguous(), positions, table, backward=True, out=d_qkv[:, H * D:(H + Hkv) * D].view(Tn, Hkv, D))
        d_qkv[:, (H + Hkv) * D:].view(Tn, Hkv, D).copy_(dv)
        return d_qkv, None, None, None, None, None


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return ops.swiglu(gu)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        return ops.swiglu_backward(gu, dy.contiguous())   # (the kernel indexes dy densely)


class LazyStateDict(Mapping):
    """The model's parameters by name, resolved when asked for: a view of this rank's storage, a gathered row-sharded
    matrix, or (expert-parallel training on GPUs) a view of the owner's storage in peer memory. An engine that loads
    from it copies tensor by tensor, so no second copy of the model exists at any time."""

    def __init__(self, model: "NativeCausalLM"):
        from ..models.weights import param_shapes

        self.model = model
        self.names = list(param_shapes(model.cfg))

    def __getitem__(self, name: str) -> torch.Tensor:
        m, b = self.model, self.model.b
        if name in b.specs:
            return b.full_param(name)
        assert m.ep is not None and m.on_gpu, f"{name} is not stored on this rank"
        rank, _, EL = m.ep
        head, e, tail = re.match(r"(.*\.experts\.)(\d+)(\..*)$", name).groups()
        q = int(e) // EL
        sp = b.specs[f"{head}{int(e) - q * EL + rank * EL}{tail}"]       # my expert at the same place of the layout
        b.finish_pending()
        return b.params_buf.peer_tensor(q)[sp.p_offset:sp.p_offset + sp.numel].view(sp.shape)

    def __iter__(self):
        return iter(self.names)

    def __len__(self) -> int:
        return len(self.names)


class _AllToAllRows(torch.autograd.Function):
    """Rows ``[sum(send), d]`` ordered by destination rank -> rows ``[sum(recv), d]`` ordered by source rank; the
    gradient takes the way back."""

    @staticmethod
    def forward(ctx, x, send, recv, group):
        import torch.distributed as dist

        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = torch.empty(sum(recv), x.shape[1], dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist

        out = torch.empty(sum(ctx.send), g.shape[1], dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv, group=ctx.group)
        return out, None, None, None


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, gtable, sink):
        ctx.save_for_backward(ids)
        ctx.gtable, ctx.sink = gtable, sink
        return ops.embedding(ids, table)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        if not ctx.sink.accumulate_into(ctx.gtable):
            ctx.gtable.zero_()          # rows no token selected carry no gradient
        ctx.gtable.index_add_(0, ids.long(), dy.to(ctx.gtable.dtype))
        return None, None, None, None


class _FusedLogprob(torch.autograd.Function):
    """(h [N,d], W [V,d]) -> per-token log-prob of ``targets`` and entropy, chunked over rows."""

    CHUNK = 2048

    @staticmethod
    def forward(ctx, h, w, gw, targets, need_entropy, sink):
        N = h.shape[0]
        lp = torch.empty(N, dtype=torch.float32, device=h.device)
        lse = torch.empty_like(lp)
        ent = torch.empty_like(lp) if need_entropy else None
        for s in range(0, N, _FusedLogprob.CHUNK):
            e = min(N, s + _FusedLogprob.CHUNK)
            logits = ops.gemm(h[s:e], w, out_f32=True)
            a, b, c = T.logprob_entropy_fwd(logits, targets[s:e], need_entropy)
            lp[s:e], lse[s:e] = a, b
            if need_entropy:
                ent[s:e] = c
        ctx.save_for_backward(h, w, targets, lse, ent if need_entropy else lse)
        ctx.gw, ctx.need_entropy, ctx.sink = gw, need_entropy, sink
        ctx.mark_non_differentiable(lse)
        return lp, (ent if need_entropy else lse.new_zeros(N)), lse

    @staticmethod
    def backward(ctx, g_lp, g_ent, _g_lse):
        h, w, targets, lse, ent = ctx.saved_tensors
        N = h.shape[0]
        dh = torch.empty_like(h)
        g_lp = g_lp.contiguous().float()
        g_ent = g_ent.contiguous().float() if ctx.need_entropy else None
        for s in range(0, N, _FusedLogprob.CHUNK):
            e = min(N, s + _FusedLogprob.CHUNK)
            logits = ops.gemm(h[s:e], w, out_f32=True)
            dl = T.logprob_entropy_bwd(logits, targets[s:e], lse[s:e], ent[s:e] if ctx.need_entropy else None,
                                       g_lp[s:e], g_ent[s:e] if g_ent is not None else None)
            dl = dl.to(h.dtype) if dl.dtype != h.dtype else dl
            ops.gemm(dl, w, out=dh[s:e], b_mn_major=True)
            acc = ctx.sink.accumulate_into(ctx.gw)
            ops.gemm(dl, h[s:e], residual=ctx.gw if acc else None, out=ctx.gw, a_mn_major=True, b_mn_major=True)
        return dh, None, None, None, None, None


# ------------------------------------------------------------------------------ the model
class NativeCausalLM:
    def __init__(self, cfg: ModelConfig, buckets, device: torch.device, activation_checkpointing: bool = False):
        self.cfg = cfg
        self.b = buckets
        self.device = device
        self.on_gpu = device.type == "cuda"
        self.ckpt = activation_checkpointing
        self._params: dict[str, torch.Tensor] = {}
        self._stacked: dict[str, tuple] = {}
        self._experts: dict[str, tuple | None] = {}
        self.ep = getattr(buckets, "expert_parallel", None)      # (rank, ranks, experts per rank) in expert-parallel training
        self._sharded: dict[str, object] = {}
        self._cu_cache: dict[tuple[int, int], torch.Tensor] = {}
        self.trace: dict | None = None
        # called with the index of a gradient chunk once backward has finished every gradient of that chunk
        # (chunk 0 = embedding, 1 + i = layer i, last = final norm / untied lm_head); set per backward pass
        self.on_chunk_grads_final = None
        self.table = ops.rope_table(cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta, device=device) \
            if self.on_gpu else None

    def p(self, name: str) -> torch.Tensor:
        """Autograd leaf sharing storage with the bucket view (its gradient is written by the kernels)."""
        if self.b._pending:
            self.b.ensure_chunk(self.b.specs[name].chunk)     # its update of the last step may still be on its way
        leaf = self._params.get(name)
        if leaf is None:
            leaf = self.b.param_view(name).detach().requires_grad_(True)
            self._params[name] = leaf
        return leaf

    def g(self, name: str) -> torch.Tensor:
        return self.b.grad_view(name)

    def sharded(self, name: str):
        if self.b._pending:
            self.b.ensure_chunk(self.b.specs[name].chunk)
        h = self._sharded.get(name)
        if h is None:
            h = self._sharded[name] = self.b.sharded_weight(name)
        return h

    def stacked(self, names: tuple[str, ...]):
        """(parameter leaf, gradient view) of several matrices that lie back to back in the flat bucket, seen as one
        ``[sum(rows), cols]`` matrix, so that e.g. gate and up projections run as one GEMM; ``(None, None)`` when
        they are not adjacent."""
        key = "+".join(names)
        if self.b._pending and names[0] in self.b.specs:
            self.b.ensure_chunk(self.b.specs[names[0]].chunk)
        if key not in self._stacked:
            specs = [self.b.specs.get(n) for n in names]
            ok = all(sp is not None and not sp.sharded for sp in specs) and all(
                a.offset + a.numel == b.offset and a.shape[1:] == b.shape[1:] and len(a.shape) in (1, 2)
                for a, b in zip(specs, specs[1:]))
            if ok:
                rows = sum(sp.shape[0] for sp in specs)
                shape = (rows,) + tuple(specs[0].shape[1:])
                n = sum(sp.numel for sp in specs)
                o = specs[0].offset
                po = specs[0].p_offset
                leaf = self.b.params[po:po + n].view(shape).detach().requires_grad_(True)
                self._stacked[key] = (leaf, self.b.grads[o:o + n].view(shape))
            else:
                self._stacked[key] = (None, None)
        return self._stacked[key]

    def state_dict(self) -> dict[str, torch.Tensor]:
        """Every parameter by name. Expert-parallel training: the other ranks' experts are fetched too (a collective on
        CPU groups: every rank must call it; peer reads on the GPU), so the result is the whole model on every rank."""
        sd = {n: self.b.full_param(n) for n in self.b.specs}
        if self.ep is not None:
            if not self.on_gpu:
                sd.update({n: v.detach().to(self.b.dtype) for n, v in self._gather_remote_experts().items()})
            else:
                rank, W, _ = self.ep
                b = self.b
                b.finish_pending()
                for c, owned in enumerate(b.chunk_owned):
                    if not owned:
                        continue
                    for q in range(W):
                        if q == rank:
                            continue
                        peer = b.params_buf.peer_tensor(q)
                        for sp in b._chunk_specs[c]:
                            sd[self._expert_name_on(sp.name, q)] = peer[sp.p_offset:sp.p_offset + sp.numel].view(sp.shape).clone()
        return sd

    # ---------------------------------------------------------------- CPU / oracle path
    def _logprobs_cpu(self, input_ids, targets, need_entropy):
        leaves = {n: self.b.full_param(n).detach().float().requires_grad_(True) for n in self.b.specs}
        if self.ep is not None:
            leaves.update(self._gather_remote_experts())
        logits = causal_lm_forward(input_ids.long(), leaves, self.cfg).float()
        lp_all = F.log_softmax(logits, -1)
        safe = targets.long().clamp(min=0)
        lp = lp_all.gather(-1, safe[..., None]).squeeze(-1)
        lp = torch.where(targets >= 0, lp, torch.zeros_like(lp))
        ent = -(lp_all.exp() * lp_all).sum(-1) if need_entropy else None
        self._leaves = leaves
        return lp, ent

    # Expert-parallel training without a GPU: the oracle needs every expert, so the owners' expert storage is gathered
    # for the forward pass and every rank's gradient of an expert travels back to its owner afterwards. The layout of
    # an expert chunk is the same on every rank (rank q's experts are this rank's shifted by (q - rank) * EL).
    def _expert_name_on(self, name: str, q: int) -> str:
        rank, _, EL = self.ep
        head, e, tail = re.match(r"(.*\.experts\.)(\d+)(\..*)$", name).groups()
        return f"{head}{int(e) + (q - rank) * EL}{tail}"

    def _gather_remote_experts(self) -> dict[str, torch.Tensor]:
        import torch.distributed as dist

        rank, W, _ = self.ep
        b, out = self.b, {}
        for c, owned in enumerate(b.chunk_owned):
            if not owned:
                continue
            p_off, p_len = b.p_chunks[c]
            parts = [torch.empty(p_len, dtype=b.dtype) for _ in range(W)]
            dist.all_gather(parts, b.params[p_off:p_off + p_len].contiguous(), group=b.comm.group)
            for q in range(W):
                if q == rank:
                    continue
                for sp in b._chunk_specs[c]:
                    rel = sp.p_offset - p_off
                    out[self._expert_name_on(sp.name, q)] = parts[q][rel:rel + sp.numel].view(sp.shape).float().requires_grad_(True)
        return out

    def collect_cpu_grads(self) -> None:
        """Move autograd ``.grad`` of the CPU leaves into the flat gradient bucket (expert-parallel: an expert's
        gradients of every rank are summed on its owner)."""
        leaves = getattr(self, "_leaves", {})
        for n, leaf in leaves.items():
            if leaf.grad is not None and n in self.b.specs and not self.b.specs[n].owned:
                self.b.grad_view(n).add_(leaf.grad.to(self.b.grads.dtype))
        if self.ep is not None and leaves:
            import torch.distributed as dist

            rank, W, _ = self.ep
            b = self.b
            for c, owned in enumerate(b.chunk_owned):
                if not owned:
                    continue
                off, length = b.chunks[c]
                buf = torch.zeros(W, length, dtype=torch.float32)
                for q in range(W):
                    for sp in b._chunk_specs[c]:
                        leaf = leaves.get(self._expert_name_on(sp.name, q))
                        if leaf is not None and leaf.grad is not None:
                            rel = sp.offset - off
                            buf[q, rel:rel + sp.numel] = leaf.grad.reshape(-1)
                dist.all_reduce(buf, group=b.comm.group)
                b.grads[off:off + length].add_(buf[rank].to(b.grads.dtype))
        self._leaves = {}

    # ---------------------------------------------------------------- kernel path
    def _cu_seqlens(self, B: int, Tn: int) -> torch.Tensor:
        key = (B, Tn)
        cu = self._cu_cache.get(key)
        if cu is None:
            cu = (torch.arange(B + 1, device=self.device) * Tn).to(torch.int32)
            self._cu_cache[key] = cu
        return cu

    def _layer(self, x, i, positions, B, Tn):
        cfg = self.cfg
        pre = f"model.layers.{i}."
        a = pre + "self_attn."
        H, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        sink = self.b

        def lin(inp, name, bias=False, residual=None):
            bn = name.replace(".weight", ".bias")
            bp, bg = (self.p(bn), self.g(bn)) if bias else (None, None)
            if self.b.specs[name].sharded:      # row-sharded weight: gathered inside the consuming GEMM launch
                return _ShardedLinear.apply(inp, self.sharded(name), self.g(name), bp, bg, residual, sink)
            return _Linear.apply(inp, self.p(name), self.g(name), bp, bg, residual, sink)

        def norm(inp, name, eps=cfg.rms_norm_eps):
            return _RMSNorm.apply(inp, self.p(name), self.g(name), eps, sink)

        h = norm(x, pre + "input_layernorm.weight")
        qkv_names = tuple(a + n + "_proj.weight" for n in "qkv")
        wqkv, gqkv = self.stacked(qkv_names)
        bqkv, gbqkv = self.stacked(tuple(n.replace(".weight", ".bias") for n in qkv_names)) if cfg.attention_bias else (None, None)
        fused = wqkv is not None and (not cfg.attention_bias or bqkv is not None)
        if fused:       # q, k and v are neighbours in the bucket: one GEMM forward, dgrad and wgrad
            qkv = _Linear.apply(h, wqkv, gqkv, bqkv, gbqkv, None, sink)
        if fused and not cfg.qk_norm:
            q, k, v = _SplitQKVRope.apply(qkv, positions, self.table, H, Hkv, D)
        else:
            if fused:
                q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], dim=-1)
                q, k, v = q.reshape(-1, H, D), k.reshape(-1, Hkv, D), v.reshape(-1, Hkv, D)
            else:
                q = lin(h, a + "q_proj.weight", cfg.attention_bias).view(-1, H, D)
                k = lin(h, a + "k_proj.weight", cfg.attention_bias).view(-1, Hkv, D)
                v = lin(h, a + "v_proj.weight", cfg.attention_bias).view(-1, Hkv, D)
            if cfg.qk_norm:
                q = norm(q.contiguous(), a + "q_norm.weight")
                k = norm(k.contiguous(), a + "k_norm.weight")
            q = _RoPE.apply(q.contiguous(), positions, self.table)
            k = _RoPE.apply(k.contiguous(), positions, self.table)
        if D in (64, 128):
            # tcgen05 flash attention, forward and backward (csrc/flash_sm100.cu); rows are the B padded sequences
            cu = self._cu_seqlens(B, Tn)
            if v.stride(1) != D or v.stride(2) != 1:
                v = v.contiguous()
            o = flash_attention(q, k, v, cu, cu, Tn, Tn, causal=True, scale=1.0 / math.sqrt(D))
            o = o.reshape(B * Tn, H * D)
        else:
            # head sizes the flash kernel does not cover (tiny test models): library attention
            o = F.scaled_dot_product_attention(
                q.view(B, Tn, H, D).transpose(1, 2), k.view(B, Tn, Hkv, D).transpose(1, 2),
                v.reshape(B, Tn, Hkv, D).transpose(1, 2), is_causal=True, scale=1.0 / math.sqrt(D), enable_gqa=True)
            o = o.transpose(1, 2).reshape(B * Tn, H * D)
        x = lin(o, a + "o_proj.weight", residual=x)
        h = norm(x, pre + "post_attention_layernorm.weight")
        m = pre + "mlp."
        if cfg.is_moe and i >= cfg.first_k_dense_replace:
            return x + self._moe(h, m, lin)
        wgu, ggu = self.stacked((m + "gate_proj.weight", m + "up_proj.weight"))
        if wgu is not None:       # gate and up are neighbours in the bucket: one GEMM forward, dgrad and wgrad
            gu = _Linear.apply(h, wgu, ggu, None, None, None, sink)
        else:
            gu = torch.cat([lin(h, m + "gate_proj.weight"), lin(h, m + "up_proj.weight")], dim=-1)
        return lin(_SwiGLU.apply(gu), m + "down_proj.weight", residual=x)

    def _moe(self, h, m: str, lin):
        """Mixture-of-experts MLP for training (math of models/functional.py::moe_mlp): the router is a tcgen05 GEMM
        through ``_Linear``; the experts run as grouped tcgen05 GEMMs over expert-sorted rows, forward, data gradient
        and weight gradient alike, with no host synchronisation (``ops.moe_train.GroupedExperts``)."""
        cfg = self.cfg
        k, E = cfg.num_experts_per_tok, cfg.num_experts
        logits = lin(h, m + "gate.weight").float()
        if cfg.router_type == "sigmoid":
            scores = logits.sigmoid()
            from ..models.functional import group_limited_choice

            choice = group_limited_choice(scores + self.p(m + "gate.e_score_correction_bias").float(), cfg.n_group, cfg.topk_group)
            idx = choice.topk(k, dim=-1).indices
            wt = scores.gather(-1, idx)
            if cfg.norm_topk_prob:
                wt = wt / (wt.sum(-1, keepdim=True) + 1e-20)
            wt = wt * cfg.routed_scaling_factor
        else:
            wt, idx = logits.softmax(-1).topk(k, dim=-1)
            if cfg.norm_topk_prob:
                wt = wt / wt.sum(-1, keepdim=True)
        experts = self.stacked_experts(m)
        if self.ep is not None:
            assert experts is not None, "expert-parallel training needs the grouped expert kernels (<= 256 experts per rank, d % 64 == 0)"
            out = self._moe_ep(h, idx, wt.float(), experts)
        elif experts is not None:
            from ..ops.moe_train import GroupedExperts, GroupedPlan

            wgu, ggu, wd, gd = experts
            plan = GroupedPlan(idx.to(torch.int32).contiguous(), E, cfg.hidden_size, cfg.moe_intermediate_size)
            out = GroupedExperts.apply(h, wt.float(), wgu, ggu, wd, gd, plan, self.b)
        else:
            out = self._moe_loop(h, m, lin, idx, wt)
        if cfg.n_shared_experts > 0:
            p = m + "shared_experts."
            gu = torch.cat([lin(h, p + "gate_proj.weight"), lin(h, p + "up_proj.weight")], dim=-1)
            out = out + lin(_SwiGLU.apply(gu), p + "down_proj.weight")
        return out

    def _moe_ep(self, h, idx, wt, experts):
        """Routed experts with the experts split over the ranks: every (token, slot) row travels to the owner of its
        expert, the owner runs its experts as grouped GEMMs over everything it received, the results travel back and
        are combined with the routing weights here. Backward takes the same two trips in reverse (the autograd
        functions below), so an expert's weight gradient is complete on its owner and nowhere else. The trips are
        `all_to_all_single` calls of the process group; one host read per layer fetches the split sizes."""
        import torch.distributed as dist

        from ..ops.moe_train import GroupedExperts, GroupedPlan

        rank, W, EL = self.ep
        group = self.b.comm.group
        wgu, ggu, wd, gd = experts
        T, k = idx.shape
        d = h.shape[1]
        flat = idx.reshape(-1)
        order = flat.argsort(stable=True)                                    # rows by expert, hence by owner
        counts = torch.bincount(flat, minlength=W * EL).view(W, EL)         # [owner, local expert] rows I send
        recv_counts = torch.empty_like(counts)                               # [source, local expert] rows I get
        dist.all_to_all_single(recv_counts, counts, group=group)
        sizes = torch.stack([counts.sum(1), recv_counts.sum(1)]).tolist()   # the one host read
        send, recv = [int(x) for x in sizes[0]], [int(x) for x in sizes[1]]
        xs = h.index_select(0, order // k)                                   # [T k, d] in travel order
        xr = _AllToAllRows.apply(xs, send, recv, group)                      # [rows received, d], by source then local expert
        R = xr.shape[0]
        if R > 0:
            eid = torch.arange(EL, device=h.device).repeat(W).repeat_interleave(recv_counts.reshape(-1), output_size=R)
            plan = GroupedPlan(eid.to(torch.int32).view(R, 1).contiguous(), EL, d, self.cfg.moe_intermediate_size)
            ones = torch.ones(R, 1, dtype=torch.float32, device=h.device)
            yr = GroupedExperts.apply(xr.contiguous(), ones, wgu, ggu, wd, gd, plan, self.b)
        else:
            yr = xr                                                           # nothing arrived: this rank's experts idle this pass
        yb = _AllToAllRows.apply(yr, recv, send, group)                      # back home, still in travel order
        w_rows = wt.reshape(-1).index_select(0, order).to(h.dtype)
        return torch.zeros_like(h).index_add(0, order // k, yb * w_rows[:, None])

    def _moe_loop(self, h, m: str, lin, idx, wt):
        """Per-expert loop (one host sync for the counts): layers whose experts do not lie back to back in the bucket,
        more than 256 experts, or ``RB_MOE_GROUPED=0``."""
        cfg = self.cfg
        k, E = cfg.num_experts_per_tok, cfg.num_experts
        flat = idx.reshape(-1)
        order = flat.argsort(stable=True)                       # (token, slot) pairs grouped by expert
        counts = torch.bincount(flat, minlength=E).tolist()     # the one host sync
        tok = order // k
        xs = h.index_select(0, tok)                              # [T*k, d] rows in expert order
        ws = wt.reshape(-1).index_select(0, order).to(h.dtype)
        outs, off = [], 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            xe = xs[off:off + n]
            p = f"{m}experts.{e}."
            gu = torch.cat([lin(xe, p + "gate_proj.weight"), lin(xe, p + "up_proj.weight")], dim=-1)
            outs.append(lin(_SwiGLU.apply(gu), p + "down_proj.weight"))
            off += n
        y = torch.cat(outs, 0) * ws[:, None]
        return torch.zeros_like(h).index_add(0, tok, y)

    def stacked_experts(self, m: str):
        """``(wgu [E*2F, d], its gradient view, wd [E*d, F], its gradient view)`` of the layer whose MLP prefix is ``m``
        when its experts lie back to back in the bucket (gate|up of every expert, then every down projection), else
        None."""
        cfg = self.cfg
        E = cfg.num_experts
        first = f"{m}experts.{0 if self.ep is None else self.ep[0] * self.ep[2]}.gate_proj.weight"
        if self.b._pending and first in self.b.specs:
            self.b.ensure_chunk(self.b.specs[first].chunk)
        if m not in self._experts:
            self._experts[m] = None
            if os.environ.get("RB_MOE_GROUPED", "1") != "0" and E <= 256 and cfg.hidden_size % 64 == 0 and cfg.moe_intermediate_size % 32 == 0:
                mine = range(E) if self.ep is None else range(self.ep[0] * self.ep[2], (self.ep[0] + 1) * self.ep[2])
                wgu, ggu = self.stacked(tuple(f"{m}experts.{e}.{p}.weight" for e in mine for p in ("gate_proj", "up_proj")))
                wd, gd = self.stacked(tuple(f"{m}experts.{e}.down_proj.weight" for e in mine))
                if wgu is not None and wd is not None:
                    self._experts[m] = (wgu, ggu, wd, gd)
        return self._experts[m]

    def logprobs(self, input_ids: torch.Tensor, targets: torch.Tensor, need_entropy: bool = False):
        """Per-token ``log p(targets)`` ``[B,T]`` (and entropy) with autograd through the kernels."""
        if not self.on_gpu:
            return self._logprobs_cpu(input_ids, targets, need_entropy)
        cfg = self.cfg
        B, Tn = input_ids.shape
        ids = input_ids.reshape(-1).to(torch.int32).contiguous()
        positions = torch.arange(Tn, device=self.device, dtype=torch.int32).repeat(B)
        emb = "model.embed_tokens.weight"
        sink = self.b
        x = _Embedding.apply(ids, self.p(emb), self.g(emb), sink)
        trace = self.trace            # set to a dict to record the residual stream (layer-by-layer debugging)
        if trace is not None:
            trace["embed"] = x.detach().view(B, Tn, -1)
        cb = self.on_chunk_grads_final

        def watch(t, chunk):
            # the gradient of a layer's input is complete only after every gradient inside that layer is
            if cb is not None and t.requires_grad:
                t.register_hook(lambda g, c=chunk: cb(c))

        for i in range(cfg.num_layers):
            watch(x, self.b.specs[f"model.layers.{i}.self_attn.o_proj.weight"].chunk)
            if self.ep is not None:      # the layer's own experts are a chunk of their own
                own = self.b.specs.get(f"model.layers.{i}.mlp.experts.{self.ep[0] * self.ep[2]}.gate_proj.weight")
                if own is not None:
                    watch(x, own.chunk)
            if self.ckpt:
                x = torch.utils.checkpoint.checkpoint(self._layer, x, i, positions, B, Tn, use_reentrant=False)
            else:
                x = self._layer(x, i, positions, B, Tn)
            if trace is not None:
                trace[f"layer.{i}"] = x.detach().view(B, Tn, -1)
        head = emb if cfg.tie_word_embeddings else "lm_head.weight"
        watch(x, self.b.specs["model.norm.weight"].chunk)          # final norm (and the untied lm_head)
        h = _RMSNorm.apply(x, self.p("model.norm.weight"), self.g("model.norm.weight"), cfg.rms_norm_eps, sink)
        if trace is not None:
            trace["final_norm"] = h.detach().view(B, Tn, -1)
        tg = targets.reshape(-1).to(torch.int32).contiguous()
        lp, ent, _ = _FusedLogprob.apply(h, self.p(head), self.g(head), tg, need_entropy, sink)
        return lp.view(B, Tn), (ent.view(B, Tn) if need_entropy else None)
