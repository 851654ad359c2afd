"""Compact tensor pretty-printer for debugging (utils/render.py:8 in the reference)."""

from __future__ import annotations

import torch

_BARS = " ▁▂▃▄▅▆▇█"


def render(t: torch.Tensor, name: str = "tensor", max_items: int = 8, histogram: bool = True) -> str:
    f = t.detach().float().flatten()
    head = ", ".join(f"{v:.4g}" for v in f[:max_items].tolist())
    lines = [f"{name}: shape={tuple(t.shape)} dtype={t.dtype} device={t.device}"]
    if f.numel() == 0:
        return lines[0] + " (empty)"
    finite = f[torch.isfinite(f)]
    lines.append(f"  min={f.min():.4g} max={f.max():.4g} mean={f.mean():.4g} std={f.std() if f.numel() > 1 else 0:.4g} "
                 f"nan={int(torch.isnan(f).sum())} inf={int(torch.isinf(f).sum())}")
    lines.append(f"  [{head}{', ...' if f.numel() > max_items else ''}]")
    if histogram and finite.numel() > 1 and float(finite.max() - finite.min()) > 0:
        h = torch.histc(finite, bins=32)
        h = h / h.max()
        lines.append("  " + "".join(_BARS[min(8, int(v * 8))] for v in h.tolist()))
    return "\n".join(lines)
