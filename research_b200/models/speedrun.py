"""Functional form of the speedrun GPT of the reference's dev tree (dev/speedrun/single-file.py:877-1150): a 12-block
decoder with weightless RMSNorm, QK-norm, half-truncated rotary embedding, per-layer sliding windows over packed
documents, token value embeddings mixed into V, a gate per head on the attention output, relu^2 MLPs, an embedding
"smear" from the previous token, learned mixing with the first-layer stream, U-net skip connections, a "back-out" of
the early layers before the head and logits squashed to (0, 30). Parameters live in a plain dict; ``forward`` is the
oracle (explicit masks, fp32) and uses the tcgen05 flash kernel when ``use_flash`` and the shapes allow.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class SpeedrunConfig:
    vocab_size: int = 50304
    num_layers: int = 12
    num_heads: int = 6
    head_dim: int = 128
    max_seq_len: int = 2048
    block_size: int = 128               # window sizes are multiples of this
    gate_dims: int = 12                 # input slice of the attention / smear gates
    no_attention_layers: tuple[int, ...] = (0, 7)
    no_mlp_layers: tuple[int, ...] = (0,)
    long_window_layers: tuple[int, ...] = (4, 11)
    backout_layer: int = 8
    rope_base: float = 1024.0

    @property
    def dim(self) -> int:
        return self.num_heads * self.head_dim


def norm(x: torch.Tensor) -> torch.Tensor:
    return F.rms_norm(x, (x.shape[-1],))


def init_weights(cfg: SpeedrunConfig, seed: int = 0, zero_init_projections: bool = True) -> dict[str, torch.Tensor]:
    """Uniform(+-sqrt(3) * 0.5 / sqrt(dim)) input projections; output projections, gates and the head start at zero
    (``zero_init_projections=False`` gives them small noise instead, which tests need to see signal)."""
    g = torch.Generator().manual_seed(seed)
    d, L = cfg.dim, cfg.num_layers
    bound = math.sqrt(3.0) * 0.5 / math.sqrt(d)

    def uni(*shape):
        return (torch.rand(*shape, generator=g) * 2 - 1) * bound

    def out(*shape):
        return torch.zeros(*shape) if zero_init_projections else uni(*shape) * 0.5

    w = {"embed": torch.randn(cfg.vocab_size, d, generator=g), "lm_head": out(cfg.vocab_size, d),
         "smear_gate": out(1, cfg.gate_dims)}
    for i in range(3):
        w[f"value_embed.{i}"] = torch.randn(cfg.vocab_size, d, generator=g)
    for i in range(L):
        if i not in cfg.no_attention_layers:
            w[f"blocks.{i}.qkv"] = uni(3 * d, d)
            w[f"blocks.{i}.o"] = out(d, d)
            w[f"blocks.{i}.attn_gate"] = out(cfg.num_heads, cfg.gate_dims)
        if i not in cfg.no_mlp_layers:
            w[f"blocks.{i}.fc"] = uni(4 * d, d)
            w[f"blocks.{i}.proj"] = out(d, 4 * d)
    # scalars: skip gates [L/2] | (x, x0) mix [L,2] | (v, value-embedding) mix [L,2] | smear | back-out
    w["scalars"] = torch.cat([torch.full((L // 2,), -1.5), torch.tensor([1.0, 0.0]).repeat(L), torch.tensor([0.5, 0.5]).repeat(L),
                              torch.zeros(1), torch.full((1,), 0.5)])
    return w


def rotary_tables(cfg: SpeedrunConfig, device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin ``[max_seq_len, head_dim/2]``: a quarter of the pairs rotate (geometric frequencies down from 1 to
    1/base), the rest keep angle zero, i.e. half of every head carries no position."""
    q = cfg.head_dim // 4
    freq = (1.0 / cfg.rope_base) ** torch.linspace(0, 1, q)
    freq = torch.cat([freq, torch.zeros(cfg.head_dim // 2 - q)])
    ang = torch.arange(cfg.max_seq_len, dtype=torch.float32)[:, None] * freq[None]
    return ang.cos().to(device), ang.sin().to(device)


class Yarn:
    """Rotary frequencies that follow the attention window as it grows during training (dev/speedrun/single-file.py:818-849).
    When the long window goes from ``old`` to ``new`` blocks, frequencies that complete many rotations inside the old
    window keep their value (they encode local order) and slow ones are stretched by ``old / new`` so that the positions
    of the new, longer window fall into the range of angles the model already knows; in between, a linear blend by the
    number of rotations (``alpha`` .. ``beta``). The softmax scale grows with the logarithm of the window ratio."""

    def __init__(self, cfg: SpeedrunConfig, attn_scale: float = 0.1):
        self.cfg = cfg
        q = cfg.head_dim // 4
        freq = (1.0 / cfg.rope_base) ** torch.linspace(0, 1, q)
        self.angular_freq = torch.cat([freq, torch.zeros(cfg.head_dim // 2 - q)])
        self.attn_scale = attn_scale
        self.window = None                     # the long window (in blocks) the frequencies are currently set for

    def apply(self, old_window: int, new_window: int, alpha: float = 1.0, beta: float = 32.0) -> None:
        assert old_window > 0 and new_window > 0
        rotations = self.cfg.block_size * old_window * self.angular_freq / (2 * math.pi)
        scaling = old_window / new_window
        blend = torch.clamp((rotations - alpha) / (beta - alpha), 0, 1)
        self.angular_freq = self.angular_freq * (scaling + blend * (1 - scaling))
        self.attn_scale *= 0.2 * math.log(new_window / old_window) + 1
        self.window = new_window

    def follow(self, ws_long: int) -> bool:
        """Call with the long window of every step: rescales when it has changed. True if it did."""
        if self.window is None:
            self.window = ws_long
            return False
        if ws_long == self.window:
            return False
        self.apply(self.window, ws_long)
        return True

    def tables(self, device=None) -> tuple[torch.Tensor, torch.Tensor]:
        ang = torch.arange(self.cfg.max_seq_len, dtype=torch.float32)[:, None] * self.angular_freq[None]
        return ang.cos().to(device), ang.sin().to(device)


def rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x [T, H, D]``; pairs are (i, i + D/2)."""
    c, s = cos[: x.shape[0], None, :], sin[: x.shape[0], None, :]
    x1, x2 = x.float().chunk(2, dim=-1)
    return torch.cat([x1 * c + x2 * s, x2 * c - x1 * s], -1).to(x.dtype)


def _attention_mask(T: int, cu_seqlens: torch.Tensor, window: int, device) -> torch.Tensor:
    pos = torch.arange(T, device=device)
    doc = torch.bucketize(pos, cu_seqlens[1:].to(device), right=True)
    i, j = pos[:, None], pos[None, :]
    return (j <= i) & (i - j <= window) & (doc[:, None] == doc[None, :])


def _attend(q, k, v, cu_seqlens, window: int, scale: float, use_flash: bool) -> torch.Tensor:
    T, H, D = q.shape
    if use_flash and q.is_cuda and D in (64, 128):
        from ..ops.flash import flash_attention      # autograd entry: forward and backward kernels

        cu = cu_seqlens.to(device=q.device, dtype=torch.int32)
        max_len = int((cu[1:] - cu[:-1]).max())
        return flash_attention(q.bfloat16().contiguous(), k.bfloat16().contiguous(), v.bfloat16().contiguous(), cu, cu, max_len,
                               max_len, causal=True, window=window + 1, scale=scale).to(q.dtype)
    mask = _attention_mask(T, cu_seqlens, window, q.device)
    s = torch.einsum("ihd,jhd->hij", q.float(), k.float()) * scale
    p = s.masked_fill(~mask[None], float("-inf")).softmax(-1)
    return torch.einsum("hij,jhd->ihd", p, v.float()).to(q.dtype)


def forward(w: dict[str, torch.Tensor], tokens: torch.Tensor, cfg: SpeedrunConfig, cu_seqlens: torch.Tensor | None = None,
            ws_short: int = 3, ws_long: int = 7, attn_scale: float = 0.1, use_flash: bool = False, yarn: "Yarn | None" = None) -> torch.Tensor:
    """``tokens [T]`` (documents packed back to back, boundaries in ``cu_seqlens``) -> logits ``[T, vocab]`` in (0, 30).
    ``ws_short`` / ``ws_long`` are window lengths in blocks of ``cfg.block_size`` tokens."""
    T, L, H, D, d = tokens.shape[0], cfg.num_layers, cfg.num_heads, cfg.head_dim, cfg.dim
    dev = tokens.device
    if cu_seqlens is None:
        cu_seqlens = torch.tensor([0, T], device=dev)
    sc = w["scalars"]
    skip_w, lambdas, sa_lambdas = sc[: L // 2], sc[L // 2: L // 2 + 2 * L].view(L, 2), sc[L // 2 + 2 * L: L // 2 + 4 * L].view(L, 2)
    smear_lambda, backout_lambda = sc[-2], sc[-1]
    ve = [F.embedding(tokens, w[f"value_embed.{i}"]) for i in range(3)]
    ve = [None, ve[1], ve[2]] + [None] * (L - 6) + [ve[0], ve[1], ve[2]]          # . 1 2 ... 0 1 2
    cos, sin = rotary_tables(cfg, dev) if yarn is None else yarn.tables(dev)
    if yarn is not None:
        attn_scale = yarn.attn_scale

    x = F.embedding(tokens, w["embed"])
    smear = smear_lambda * torch.sigmoid(x[1:, : cfg.gate_dims] @ w["smear_gate"].T)
    x = torch.cat([x[:1], x[1:] + smear * x[:-1]])
    x = x0 = norm(x)
    skips: list[torch.Tensor] = []
    n = L // 2
    x_backout = None
    for i in range(1, L):                                # block 0 has neither attention nor MLP
        if n <= i < L - 1:
            x = x + torch.sigmoid(skip_w[i - n]) * skips.pop()
        x = lambdas[i, 0] * x + lambdas[i, 1] * x0
        if i not in cfg.no_attention_layers:
            h = norm(x)
            qkv = (h @ w[f"blocks.{i}.qkv"].T).view(T, 3 * H, D)
            q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
            q, k = rotary(norm(q), cos, sin), rotary(norm(k), cos, sin)
            v = sa_lambdas[i, 0] * v + (sa_lambdas[i, 1] * ve[i].view(T, H, D) if ve[i] is not None else 0)
            window = (ws_long if i in cfg.long_window_layers else ws_short) * cfg.block_size
            y = _attend(q, k, v, cu_seqlens, window, attn_scale, use_flash)
            y = y * torch.sigmoid(h[:, : cfg.gate_dims] @ w[f"blocks.{i}.attn_gate"].T)[:, :, None]
            x = x + y.reshape(T, d) @ w[f"blocks.{i}.o"].T
        if i not in cfg.no_mlp_layers:
            x = x + F.relu(norm(x) @ w[f"blocks.{i}.fc"].T).square() @ w[f"blocks.{i}.proj"].T
        if i < n:
            skips.append(x)
        if i == cfg.backout_layer:
            x_backout = x
    if x_backout is not None:
        x = x - backout_lambda * x_backout                # early layers serve later context, not the prediction itself
    logits = norm(x) @ w["lm_head"].T
    return 30.0 * torch.sigmoid(logits.float() / 7.5)


def loss(w, tokens, targets, cfg: SpeedrunConfig, **kw) -> torch.Tensor:
    return F.cross_entropy(forward(w, tokens, cfg, **kw), targets)
