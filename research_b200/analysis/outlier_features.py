"""Outlier features of the residual stream, after Dettmers et al. 2022 as applied in dev/outlier-features/
analyze_activations.py: a hidden dimension is an outlier feature when its magnitude reaches ``magnitude`` (6.0) in at
least ``min_layer_frac`` (25 %) of the layers and ``min_token_frac`` (6 %) of the sequence positions."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class OutlierReport:
    dims: list[int]                                  # hidden dimensions that qualify
    layer_frac: dict[int, float]                     # dim -> fraction of layers in which it crosses the threshold
    token_frac: dict[int, float]                     # dim -> fraction of positions (over all layers) in which it does
    max_abs: dict[int, float]
    per_layer_counts: list[int] = field(default_factory=list)   # qualifying dims seen crossing in each layer

    def summary(self) -> str:
        head = f"{len(self.dims)} outlier feature(s)"
        rows = [f"  dim {d}: {self.layer_frac[d]:.0%} of layers, {self.token_frac[d]:.1%} of positions, max |x| {self.max_abs[d]:.1f}"
                for d in self.dims]
        return "\n".join([head, *rows])


def find_outlier_features(activations: dict[str, torch.Tensor] | list[torch.Tensor], magnitude: float = 6.0,
                          min_layer_frac: float = 0.25, min_token_frac: float = 0.06) -> OutlierReport:
    """``activations``: one ``[..., hidden]`` tensor per layer (leading dimensions are flattened into positions)."""
    layers = list(activations.values()) if isinstance(activations, dict) else list(activations)
    assert layers, "no activations"
    d = layers[0].shape[-1]
    layer_hits = torch.zeros(d)
    token_hits = torch.zeros(d)
    max_abs = torch.zeros(d)
    positions = 0
    crossing = []
    for x in layers:
        a = x.detach().float().reshape(-1, d).abs()
        over = a >= magnitude
        crossing.append(over.any(0))
        layer_hits += over.any(0).float()
        token_hits += over.float().sum(0)
        max_abs = torch.maximum(max_abs, a.max(0).values)
        positions += a.shape[0]
    lf, tf = layer_hits / len(layers), token_hits / max(positions, 1)
    dims = [int(i) for i in torch.nonzero((lf >= min_layer_frac) & (tf >= min_token_frac)).flatten()]
    sel = torch.tensor(dims, dtype=torch.long)
    return OutlierReport(dims, {i: float(lf[i]) for i in dims}, {i: float(tf[i]) for i in dims}, {i: float(max_abs[i]) for i in dims},
                         [int(c[sel].sum()) if dims else 0 for c in crossing])


def collect_residual_stream(input_ids: torch.Tensor, weights: dict[str, torch.Tensor], cfg) -> dict[str, torch.Tensor]:
    """Residual stream after the embedding and after every layer (``[B, T, hidden]`` each) from the functional model."""
    from ..models import causal_lm_forward

    trace: dict[str, torch.Tensor] = {}
    causal_lm_forward(input_ids, weights, cfg, trace=trace)
    return {k: v for k, v in trace.items() if k == "embed" or k.startswith("layer.")}


def perplexity(input_ids: torch.Tensor, weights: dict[str, torch.Tensor], cfg) -> float:
    """exp(mean next-token negative log-likelihood) of ``input_ids [B, T]`` under the functional model
    (dev/outlier-features/compute_perplexity.py)."""
    from ..models import causal_lm_forward

    logits = causal_lm_forward(input_ids, weights, cfg).float()
    lp = torch.log_softmax(logits[:, :-1], -1).gather(-1, input_ids[:, 1:, None].long()).squeeze(-1)
    return float(torch.exp(-lp.mean()))
