"""Optimizer trajectories on two-dimensional test functions (dev/optimizer-visuals/optimizers.py:49-147 implements SGD,
momentum and Adam by hand for such pictures): hand-written update rules, the classic test surfaces, the path each
optimizer takes from a start point, and a character-cell rendering for a terminal."""

from __future__ import annotations

import math
from typing import Callable

import torch

Surface = Callable[[torch.Tensor], torch.Tensor]

SURFACES: dict[str, tuple[Surface, tuple[float, float], tuple[float, float]]] = {
    # name -> (f(xy), minimiser, default start)
    "rosenbrock": (lambda p: (1 - p[0]) ** 2 + 100 * (p[1] - p[0] ** 2) ** 2, (1.0, 1.0), (-1.2, 1.0)),
    "beale": (lambda p: (1.5 - p[0] + p[0] * p[1]) ** 2 + (2.25 - p[0] + p[0] * p[1] ** 2) ** 2 + (2.625 - p[0] + p[0] * p[1] ** 3) ** 2,
              (3.0, 0.5), (1.0, 1.5)),
    "quadratic": (lambda p: 0.5 * (10 * p[0] ** 2 + p[1] ** 2), (0.0, 0.0), (2.0, 2.0)),
}


def sgd_step(p, g, state, lr=1e-3, momentum=0.0, nesterov=False):
    if momentum:
        buf = state.setdefault("buf", torch.zeros_like(p))
        buf.mul_(momentum).add_(g)
        g = g + momentum * buf if nesterov else buf
    return p - lr * g


def adam_step(p, g, state, lr=1e-2, b1=0.9, b2=0.999, eps=1e-8):
    t = state["t"] = state.get("t", 0) + 1
    m = state.setdefault("m", torch.zeros_like(p))
    v = state.setdefault("v", torch.zeros_like(p))
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    return p - lr * (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + eps)


def rmsprop_step(p, g, state, lr=1e-2, alpha=0.99, eps=1e-8):
    v = state.setdefault("v", torch.zeros_like(p))
    v.mul_(alpha).addcmul_(g, g, value=1 - alpha)
    return p - lr * g / (v.sqrt() + eps)


OPTIMIZERS = {"sgd": sgd_step, "momentum": lambda p, g, s, **kw: sgd_step(p, g, s, momentum=0.9, **kw),
              "nesterov": lambda p, g, s, **kw: sgd_step(p, g, s, momentum=0.9, nesterov=True, **kw),
              "adam": adam_step, "rmsprop": rmsprop_step}


def trajectory(surface: str | Surface, optimizer: str, steps: int = 200, start: tuple[float, float] | None = None, **hyper) -> torch.Tensor:
    """``[steps + 1, 2]`` points visited from ``start`` (gradients by autograd, float64)."""
    f, _, default_start = SURFACES[surface] if isinstance(surface, str) else (surface, None, (0.0, 0.0))
    p = torch.tensor(start or default_start, dtype=torch.float64)
    step, state, path = OPTIMIZERS[optimizer], {}, [p.clone()]
    for _ in range(steps):
        q = p.clone().requires_grad_(True)
        (g,) = torch.autograd.grad(f(q), q)
        p = step(p, g, state, **hyper).detach()
        if not torch.isfinite(p).all():
            break
        path.append(p.clone())
    return torch.stack(path)


def render(surface: str, paths: dict[str, torch.Tensor], width: int = 60, height: int = 24, span: float = 2.5) -> str:
    """Character-cell picture: level sets of log(1 + f) as shades, each path drawn with the first letter of its name,
    the minimiser as ``*``."""
    f, best, _ = SURFACES[surface]
    cx, cy = best
    xs = torch.linspace(cx - span, cx + span, width, dtype=torch.float64)
    ys = torch.linspace(cy + span, cy - span, height, dtype=torch.float64)
    z = torch.log1p(torch.stack([torch.stack([f(torch.stack([x, y])) for x in xs]) for y in ys]))
    shades = " .:-=+#"
    zn = (z - z.min()) / (z.max() - z.min() + 1e-12)
    grid = [[shades[min(int(v * (len(shades) - 1) + 0.5), len(shades) - 1)] for v in row] for row in zn]

    def cell(pt):
        c = int(round(float((pt[0] - xs[0]) / (xs[-1] - xs[0]) * (width - 1))))
        r = int(round(float((ys[0] - pt[1]) / (ys[0] - ys[-1]) * (height - 1))))
        return (r, c) if 0 <= r < height and 0 <= c < width else None

    for name, path in paths.items():
        for pt in path:
            rc = cell(pt)
            if rc:
                grid[rc[0]][rc[1]] = name[0].upper()
    rc = cell(torch.tensor(best))
    if rc:
        grid[rc[0]][rc[1]] = "*"
    return "\n".join("".join(row) for row in grid)


def distance_to_minimum(surface: str, path: torch.Tensor) -> float:
    return float(math.dist(path[-1].tolist(), SURFACES[surface][1]))
