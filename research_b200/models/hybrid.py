"""Functional oracle of the hybrid (Qwen3-Next style) blocks: gated full attention with partial RoPE,
Gated DeltaNet linear attention, and the top-k-then-softmax router with a sigmoid-gated shared expert
(rollouts/tools/functional_extractor/qwen3_next_functional.py:91-490).

Gated delta rule per head, state ``S`` of shape ``[d_v, d_k]``:

    S_t = a_t * S_{t-1} (I - b_t k_t k_t^T) + b_t v_t k_t^T        o_t = S_t q_t

with decay ``a_t = exp(-exp(A_log) * softplus(alpha_t + dt_bias))`` in (0, 1), write strength
``b_t = sigmoid(beta_t)``, and l2-normalised ``q``, ``k``. Two evaluations are given and tested against
each other: the token-by-token recurrence (also the decode step, it carries the state) and a chunked
form that does the within-chunk work as small dense products (the shape a tensor-core kernel would
take). These are fp32 oracles; no sm_100a kernel exists for this block yet.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .functional import rms_norm, rotate_half


def partial_rope(x: torch.Tensor, positions: torch.Tensor, rotary_dim: int, theta: float) -> torch.Tensor:
    """Rotate only the first ``rotary_dim`` channels of ``x [T, H, D]``."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=x.device) / rotary_dim))
    ang = positions.float()[:, None] * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None, :], torch.cat([ang.sin(), ang.sin()], -1)[:, None, :]
    rot, rest = x[..., :rotary_dim].float(), x[..., rotary_dim:]
    return torch.cat([(rot * cos + rotate_half(rot) * sin).to(x.dtype), rest], -1)


def gated_attention(x: torch.Tensor, w: dict, prefix: str, num_heads: int, num_kv_heads: int, head_dim: int,
                    positions: torch.Tensor, rotary_dim: int, theta: float, eps: float) -> torch.Tensor:
    """Causal GQA where ``q_proj`` also produces a per-channel output gate: ``o * sigmoid(gate)``; q/k RMS-normed per head."""
    T = x.shape[0]
    qg = F.linear(x, w[f"{prefix}.q_proj.weight"]).view(T, num_heads, 2 * head_dim)
    q, gate = qg[..., :head_dim], qg[..., head_dim:]
    k = F.linear(x, w[f"{prefix}.k_proj.weight"]).view(T, num_kv_heads, head_dim)
    v = F.linear(x, w[f"{prefix}.v_proj.weight"]).view(T, num_kv_heads, head_dim)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], eps)
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], eps)
    q, k = partial_rope(q, positions, rotary_dim, theta), partial_rope(k, positions, rotary_dim, theta)
    g = num_heads // num_kv_heads
    s = torch.einsum("qhd,khd->hqk", q.float(), k.float().repeat_interleave(g, 1)) / math.sqrt(head_dim)
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=x.device), 1), float("-inf"))
    o = torch.einsum("hqk,khd->qhd", s.softmax(-1), v.float().repeat_interleave(g, 1)).to(x.dtype)
    o = (o * torch.sigmoid(gate.float()).to(x.dtype)).reshape(T, num_heads * head_dim)
    return F.linear(o, w[f"{prefix}.o_proj.weight"])


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Depthwise causal convolution over time. ``x [T, C]``, ``weight [C, K]``; returns output and the last K-1 inputs."""
    K = weight.shape[1]
    pad = state if state is not None else x.new_zeros(K - 1, x.shape[1])
    xp = torch.cat([pad, x], 0)
    out = F.conv1d(xp.T[None].float(), weight[:, None, :].float(), groups=x.shape[1])[0].T
    return out.to(x.dtype), xp[-(K - 1):] if K > 1 else xp[:0]


def gated_delta_rule_recurrent(q, k, v, a, b, state=None):
    """``q, k [T, H, dk]``, ``v [T, H, dv]``, decay ``a`` and write strength ``b`` ``[T, H]``. Returns ``(o [T,H,dv], S [H,dv,dk])``."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = state.float().clone() if state is not None else q.new_zeros(H, dv, dk, dtype=torch.float32)
    out = []
    qf, kf, vf, af, bf = q.float(), k.float(), v.float(), a.float(), b.float()
    for t in range(T):
        kt, vt = kf[t], vf[t]
        S = af[t][:, None, None] * (S - bf[t][:, None, None] * torch.einsum("hvk,hk,hj->hvj", S, kt, kt))
        S = S + bf[t][:, None, None] * torch.einsum("hv,hk->hvk", vt, kt)
        out.append(torch.einsum("hvk,hk->hv", S, qf[t]))
    return torch.stack(out, 0), S


def gated_delta_rule_chunked(q, k, v, a, b, chunk: int = 16, state=None):
    """Same result, computed chunk by chunk: within a chunk the dependence between tokens is resolved by one
    triangular solve (the ``(I + tril(...))^-1`` of the WY representation) and everything else is dense products."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = state.float().clone() if state is not None else q.new_zeros(H, dv, dk, dtype=torch.float32)
    outs = []
    for s0 in range(0, T, chunk):
        qc, kc, vc = (x[s0:s0 + chunk].float().transpose(0, 1) for x in (q, k, v))          # [H, C, d]
        ac, bc = a[s0:s0 + chunk].float().T, b[s0:s0 + chunk].float().T                     # [H, C]
        C = qc.shape[1]
        g = torch.cumsum(torch.log(ac), 1)                                                  # log of cumulative decay
        decay = torch.exp(g[:, :, None] - g[:, None, :])                                    # [H, i, j] = prod_{j<l<=i} a_l
        # u_i = b_i (v_i - d_{i-1..}...) solves (I + tril(b_i decay_ij k_i.k_j, -1)) U = b (V - G S0 K)
        kk = torch.einsum("hik,hjk->hij", kc, kc)
        L = torch.tril(bc[:, :, None] * decay * kk, -1)
        rhs = bc[:, :, None] * (vc - torch.exp(g)[:, :, None] * torch.einsum("hvk,hik->hiv", S, kc))
        U = torch.linalg.solve_triangular(torch.eye(C, device=q.device) + L, rhs, upper=False)   # [H, C, dv]
        # outputs: inter-chunk part through the carried state, intra-chunk part through U
        attn = torch.tril(decay * torch.einsum("hik,hjk->hij", qc, kc))
        o = torch.exp(g)[:, :, None] * torch.einsum("hvk,hik->hiv", S, qc) + torch.einsum("hij,hjv->hiv", attn, U)
        outs.append(o.transpose(0, 1))
        # state at the end of the chunk
        tail = torch.exp(g[:, -1:] - g)                                                     # decay from token j to chunk end
        S = torch.exp(g[:, -1])[:, None, None] * S + torch.einsum("hj,hjv,hjk->hvk", tail, U, kc)
    return torch.cat(outs, 0), S


def gated_delta_net(x: torch.Tensor, w: dict, prefix: str, num_heads: int, head_k: int, head_v: int, eps: float,
                    chunk: int | None = 16, state: dict | None = None) -> tuple[torch.Tensor, dict]:
    """Full block on ``x [T, hidden]``: projections, causal conv + SiLU on q|k|v, l2-normalised q and k, the gated
    delta rule, gated RMSNorm (``norm(o) * silu(z)``) and the output projection. ``state`` carries conv and S."""
    T = x.shape[0]
    dk, dv = num_heads * head_k, num_heads * head_v
    qkvz = F.linear(x, w[f"{prefix}.in_proj_qkvz.weight"])
    qkv, z = qkvz[:, :2 * dk + dv], qkvz[:, 2 * dk + dv:]
    ba = F.linear(x, w[f"{prefix}.in_proj_ba.weight"]).float()
    beta, alpha = ba[:, :num_heads], ba[:, num_heads:]
    qkv, conv_state = causal_conv1d(qkv, w[f"{prefix}.conv1d.weight"], state.get("conv") if state else None)
    qkv = F.silu(qkv)
    q, k, v = qkv[:, :dk].view(T, num_heads, head_k), qkv[:, dk:2 * dk].view(T, num_heads, head_k), qkv[:, 2 * dk:].view(T, num_heads, head_v)
    q = F.normalize(q.float(), dim=-1) / math.sqrt(head_k)
    k = F.normalize(k.float(), dim=-1)
    a = torch.exp(-torch.exp(w[f"{prefix}.A_log"].float()) * F.softplus(alpha + w[f"{prefix}.dt_bias"].float()))
    b = torch.sigmoid(beta)
    S0 = state.get("S") if state else None
    o, S = gated_delta_rule_recurrent(q, k, v, a, b, S0) if chunk is None else gated_delta_rule_chunked(q, k, v, a, b, chunk, S0)
    o = rms_norm(o.to(x.dtype), w[f"{prefix}.norm.weight"], eps) * F.silu(z.view(T, num_heads, head_v))
    return F.linear(o.reshape(T, dv), w[f"{prefix}.out_proj.weight"]), {"conv": conv_state, "S": S}


def qwen3_next_moe(x: torch.Tensor, w: dict, prefix: str, top_k: int, norm_topk_prob: bool = True) -> torch.Tensor:
    """Softmax over all experts, keep the top-k (renormalised), plus a shared expert scaled by ``sigmoid(x W_g)``."""
    logits = F.linear(x, w[f"{prefix}.gate.weight"]).float()
    probs = logits.softmax(-1)
    top_p, top_i = probs.topk(top_k, dim=-1)
    if norm_topk_prob:
        top_p = top_p / top_p.sum(-1, keepdim=True)
    out = torch.zeros_like(x, dtype=torch.float32)

    def ffn(h, p):
        return F.linear(F.silu(F.linear(h, w[f"{p}.gate_proj.weight"])) * F.linear(h, w[f"{p}.up_proj.weight"]), w[f"{p}.down_proj.weight"])

    for e in top_i.unique().tolist():
        rows, slot = (top_i == e).nonzero(as_tuple=True)
        out.index_add_(0, rows, ffn(x[rows], f"{prefix}.experts.{e}").float() * top_p[rows, slot][:, None])
    shared = ffn(x, f"{prefix}.shared_expert").float() * torch.sigmoid(F.linear(x, w[f"{prefix}.shared_expert_gate.weight"]).float())
    return (out + shared).to(x.dtype)
