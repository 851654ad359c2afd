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


# a long, narrow, rotated valley: steep across, shallow along; what momentum and per-coordinate scaling are for
def _narrow_valley(p: torch.Tensor, steep: float = 50.0, theta: float = math.pi / 6) -> torch.Tensor:
    u = math.cos(theta) * p[0] + math.sin(theta) * p[1]
    v = -math.sin(theta) * p[0] + math.cos(theta) * p[1]
    return 0.5 * (u ** 2 + steep * v ** 2)


SURFACES["narrow_valley"] = (_narrow_valley, (0.0, 0.0), (2.0, -1.0))


def compare(surface: str, optimizers: dict[str, dict] | None = None, steps: int = 300) -> dict[str, dict]:
    """Every optimizer from the same start on ``surface``: final distance to the minimiser, final value, steps taken and the
    first step at which the value fell below 1 % of the start value (dev/optimizer-visuals/compare_optimizers.py)."""
    f = SURFACES[surface][0]
    optimizers = optimizers or {"sgd": {"lr": 0.01}, "momentum": {"lr": 0.01}, "nesterov": {"lr": 0.01}, "rmsprop": {"lr": 0.02}, "adam": {"lr": 0.05}}
    out = {}
    for name, hyper in optimizers.items():
        path = trajectory(surface, name, steps, **hyper)
        values = [float(f(p)) for p in path]
        target = 0.01 * values[0]
        out[name] = {"final_distance": distance_to_minimum(surface, path), "final_value": values[-1], "steps": len(path) - 1,
                     "steps_to_1pct": next((i for i, v in enumerate(values) if v <= target), None), "diverged": len(path) - 1 < steps or values[-1] > 1e6 * max(values[0], 1e-12), "path": path}   # left the float range, or ran away
    return out


def landscape(surface: str, resolution: int = 50, span: float = 2.5) -> dict:
    """Values of the surface on a ``resolution`` x ``resolution`` grid around its minimiser (for contour plots)."""
    f, (cx, cy), _ = SURFACES[surface]
    xs = torch.linspace(cx - span, cx + span, resolution, dtype=torch.float64)
    ys = torch.linspace(cy - span, cy + span, resolution, dtype=torch.float64)
    z = torch.stack([torch.stack([f(torch.stack([x, y])) for x in xs]) for y in ys])
    return {"x": xs.tolist(), "y": ys.tolist(), "z": z.tolist(), "minimum": [cx, cy]}


def export_viz_data(surface: str, results: dict[str, dict], path=None, resolution: int = 50) -> dict:
    """Paths, values along them and the landscape grid in one JSON-able dict (what a plotting front end needs;
    dev/optimizer-visuals/viz_data.py), optionally written to ``path``."""
    import json

    f = SURFACES[surface][0]
    data = {"surface": surface, "landscape": landscape(surface, resolution),
            "trajectories": {name: {"points": r["path"].tolist(), "values": [float(f(p)) for p in r["path"]],
                                    "final_distance": r["final_distance"], "diverged": r["diverged"]} for name, r in results.items()}}
    if path is not None:
        with open(path, "w") as fh:
            json.dump(data, fh)
    return data


def momentum_rank_experiment(input_dim: int = 32, output_dim: int = 32, true_rank: int = 4, n_samples: int = 512, steps: int = 300, lr: float = 1e-2,
                             noise: float = 0.01, seed: int = 0, record_every: int = 25) -> dict:
    """Does Adam's first-moment matrix become low-rank during training? Linear regression ``Y = W X`` whose true ``W`` has
    rank ``true_rank``; Adam on the mean squared error, written out by hand; the singular values of the moment matrix
    ``M`` are recorded every ``record_every`` steps (dev/optimizer-visuals/measure_momentum_rank.py). Returned per record:
    the step, the loss, the singular values, the EFFECTIVE rank exp(entropy of the normalised spectrum), and the share of
    the spectrum's energy in its top ``true_rank`` values."""
    g = torch.Generator().manual_seed(seed)
    w_true = (torch.randn(output_dim, true_rank, generator=g, dtype=torch.float64) @ torch.randn(true_rank, input_dim, generator=g, dtype=torch.float64)) / math.sqrt(true_rank)
    x = torch.randn(input_dim, n_samples, generator=g, dtype=torch.float64)
    y = w_true @ x + noise * torch.randn(output_dim, n_samples, generator=g, dtype=torch.float64)
    w = torch.zeros(output_dim, input_dim, dtype=torch.float64)
    m, v = torch.zeros_like(w), torch.zeros_like(w)
    b1, b2, eps = 0.9, 0.999, 1e-8
    records = []
    for t in range(1, steps + 1):
        err = w @ x - y
        grad = 2.0 * err @ x.T / err.numel()
        m = b1 * m + (1 - b1) * grad
        v = b2 * v + (1 - b2) * grad * grad
        w = w - lr * (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + eps)
        if t % record_every == 0 or t == 1 or t == steps:
            s = torch.linalg.svdvals(m)
            p = s / s.sum().clamp_min(1e-300)
            records.append({"step": t, "loss": float((err ** 2).mean()), "singular_values": s.tolist(),
                            "effective_rank": float(torch.exp(-(p * (p.clamp_min(1e-300)).log()).sum())),
                            "top_energy": float((s[:true_rank] ** 2).sum() / (s ** 2).sum().clamp_min(1e-300))})
    return {"true_rank": true_rank, "shape": [output_dim, input_dim], "records": records,
            "weight_error": float((w - w_true).norm() / w_true.norm())}
