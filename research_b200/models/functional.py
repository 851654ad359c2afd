"""Class-free forward passes in plain ``torch.nn.functional``: the numerics oracle.

Same role and the same math as the reference's extracted functional models
(rollouts/tools/functional_extractor/qwen_functional.py:46-438 for Qwen2,
qwen3_functional.py for QK-norm, llama_functional.py:358-404 for the untied head,
qwen3_next_functional.py:409-490 and glm4_moe_functional.py:230-428 for the two MoE routers).
Weights use Hugging Face parameter names. Works in fp32 (CPU oracle) or bf16.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .config import ModelConfig


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    dt = x.dtype
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return w * xf.to(dt)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    freqs = positions.float()[..., None] * inv_freq
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def attention(x, w, prefix, cfg: ModelConfig, positions, attn_mask=None):
    """x [B,T,d]; returns [B,T,d]. Causal SDPA with GQA by repetition, like the HF module."""
    B, T, _ = x.shape
    H, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    q = F.linear(x, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias"))
    k = F.linear(x, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias"))
    v = F.linear(x, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias"))
    q = q.view(B, T, H, D)
    k = k.view(B, T, Hkv, D)
    v = v.view(B, T, Hkv, D)
    if cfg.qk_norm:
        q = rms_norm(q, w[prefix + "q_norm.weight"], cfg.rms_norm_eps)
        k = rms_norm(k, w[prefix + "k_norm.weight"], cfg.rms_norm_eps)
    cos, sin = rope_cos_sin(positions, D, cfg.rope_theta, x.dtype)  # [B,T,D]
    cos, sin = cos[:, :, None, :], sin[:, :, None, :]
    q = q * cos + rotate_half(q) * sin
    k = k * cos + rotate_half(k) * sin
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    rep = H // Hkv
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    if attn_mask is None:
        causal = torch.ones(T, T, dtype=torch.bool, device=x.device).tril()
        if cfg.sliding_window > 0:
            causal &= ~torch.ones(T, T, dtype=torch.bool, device=x.device).tril(-cfg.sliding_window)
        attn_mask = causal[None, None]
    o = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, scale=1.0 / math.sqrt(D))
    o = o.transpose(1, 2).reshape(B, T, H * D)
    return F.linear(o, w[prefix + "o_proj.weight"])


def dense_mlp(x, w, prefix):
    g = F.linear(x, w[prefix + "gate_proj.weight"])
    u = F.linear(x, w[prefix + "up_proj.weight"])
    return F.linear(F.silu(g) * u, w[prefix + "down_proj.weight"])


def group_limited_choice(choice: torch.Tensor, n_group: int, topk_group: int) -> torch.Tensor:
    """DeepSeek-V3 / GLM-4.5 group-limited routing (glm4_moe_functional.py:278-301): experts form ``n_group``
    contiguous groups, a group scores the sum of its two best choice values, only the ``topk_group`` best groups stay
    eligible and the choice values of all other experts become 0 (not -inf, as in the reference)."""
    if n_group <= 1 or topk_group >= n_group:
        return choice
    N, E = choice.shape
    assert E % n_group == 0 and E // n_group >= 2, "group-limited routing needs equal groups of at least two experts"
    group_scores = choice.view(N, n_group, E // n_group).topk(2, dim=-1).values.sum(-1)
    keep = torch.zeros_like(group_scores, dtype=torch.bool).scatter_(1, group_scores.topk(topk_group, dim=-1).indices, True)
    return choice.masked_fill(~keep.repeat_interleave(E // n_group, dim=1), 0.0)


def route(x2: torch.Tensor, w, prefix: str, cfg: ModelConfig):
    """Router: returns (topk_idx [N,k] int64, topk_weight [N,k] in x dtype)."""
    logits = F.linear(x2.float(), w[prefix + "gate.weight"].float())
    k = cfg.num_experts_per_tok
    if cfg.router_type == "sigmoid":
        scores = logits.sigmoid()
        choice = scores + w[prefix + "gate.e_score_correction_bias"].float()
        choice = group_limited_choice(choice, cfg.n_group, cfg.topk_group)
        idx = choice.topk(k, dim=-1).indices
        wt = scores.gather(-1, idx)
        if cfg.norm_topk_prob:
            wt = wt / (wt.sum(-1, keepdim=True) + 1e-20)
        wt = wt * cfg.routed_scaling_factor
    else:
        probs = logits.softmax(-1)
        wt, idx = probs.topk(k, dim=-1)
        if cfg.norm_topk_prob:
            wt = wt / wt.sum(-1, keepdim=True)
    return idx, wt.to(x2.dtype)


def moe_mlp(x, w, prefix, cfg: ModelConfig):
    """Naive per-expert loop with index_add, as the reference oracles do it."""
    B, T, d = x.shape
    x2 = x.reshape(-1, d)
    idx, wt = route(x2, w, prefix, cfg)
    out = torch.zeros_like(x2)
    for e in range(cfg.num_experts):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = dense_mlp(x2[tok], w, f"{prefix}experts.{e}.")
        out.index_add_(0, tok, h * wt[tok, slot][:, None])
    if cfg.n_shared_experts > 0:
        out = out + dense_mlp(x2, w, prefix + "shared_experts.")
    return out.view(B, T, d)


def decoder_layer_forward(x, w, layer: int, cfg: ModelConfig, positions, attn_mask=None):
    p = f"model.layers.{layer}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg.rms_norm_eps)
    x = x + attention(h, w, p + "self_attn.", cfg, positions, attn_mask)
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
    if cfg.is_moe and layer >= cfg.first_k_dense_replace:
        x = x + moe_mlp(h, w, p + "mlp.", cfg)
    else:
        x = x + dense_mlp(h, w, p + "mlp.")
    return x


def causal_lm_forward(input_ids: torch.Tensor, w: dict, cfg: ModelConfig, positions: torch.Tensor | None = None,
                      attn_mask: torch.Tensor | None = None, return_hidden: bool = False,
                      trace: dict | None = None) -> torch.Tensor:
    """``input_ids [B,T]`` -> logits ``[B,T,V]`` (or final hidden states). ``trace``, when given, receives the
    residual stream after the embedding and after every layer, the final norm and the logits."""
    B, T = input_ids.shape
    if positions is None:
        positions = torch.arange(T, device=input_ids.device)[None].expand(B, T)
    x = F.embedding(input_ids, w["model.embed_tokens.weight"])
    if trace is not None:
        trace["embed"] = x.detach()
    for layer in range(cfg.num_layers):
        x = decoder_layer_forward(x, w, layer, cfg, positions, attn_mask)
        if trace is not None:
            trace[f"layer.{layer}"] = x.detach()
    x = rms_norm(x, w["model.norm.weight"], cfg.rms_norm_eps)
    if trace is not None:
        trace["final_norm"] = x.detach()
    if return_hidden:
        return x
    head = w["model.embed_tokens.weight"] if cfg.tie_word_embeddings else w["lm_head.weight"]
    logits = F.linear(x, head)
    if trace is not None:
        trace["logits"] = logits.detach()
    return logits


def packed_document_mask(cu_seqlens: torch.Tensor, total: int, device=None) -> torch.Tensor:
    """Block-diagonal causal mask ``[1,1,total,total]`` for sequence-packed batches."""
    doc = torch.zeros(total, dtype=torch.long, device=device)
    for i in range(len(cu_seqlens) - 1):
        doc[int(cu_seqlens[i]) : int(cu_seqlens[i + 1])] = i
    same = doc[:, None] == doc[None, :]
    causal = torch.ones(total, total, dtype=torch.bool, device=device).tril()
    return (same & causal)[None, None]
