"""Layer-by-layer divergence hunting between two implementations of the same model
(rollouts/tools/functional_extractor/debug_toolkit.py:200, verify.py:346).

Both sides produce a *trace*: ``name -> tensor`` for the embedding output, the residual stream after
every layer, the final norm and the logits (``causal_lm_forward(..., trace=...)`` for the oracle,
``NativeCausalLM.trace`` for the kernel path). ``compare_traces`` walks them in order and reports, per
point, the maximum and relative error and where the first point beyond tolerance is - which is the
layer to open up next. ``verify_against_oracle`` wraps the common case.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class TracePoint:
    name: str
    max_abs: float
    rel: float            # ||a - b|| / ||b||
    ok: bool


@dataclass
class TraceReport:
    points: list[TracePoint]

    @property
    def first_divergence(self) -> TracePoint | None:
        return next((p for p in self.points if not p.ok), None)

    @property
    def ok(self) -> bool:
        return self.first_divergence is None

    def format(self) -> str:
        lines = [f"{'point':<14}{'max |diff|':>12}{'rel':>12}"]
        for p in self.points:
            lines.append(f"{p.name:<14}{p.max_abs:>12.3e}{p.rel:>12.3e}{'' if p.ok else '   <-- beyond tolerance'}")
        fd = self.first_divergence
        lines.append("all points within tolerance" if fd is None else f"first divergence at {fd.name}")
        return "\n".join(lines)


def _order(name: str) -> tuple[int, int]:
    if name == "embed":
        return (0, 0)
    if name.startswith("layer."):
        return (1, int(name.split(".")[1]))
    return (2, 0) if name == "final_norm" else (3, 0)


def compare_traces(got: dict, want: dict, rel_tol: float = 2e-2, abs_tol: float = 0.0) -> TraceReport:
    pts = []
    for name in sorted(set(got) & set(want), key=_order):
        a, b = got[name].float().cpu().reshape(-1), want[name].float().cpu().reshape(-1)
        assert a.shape == b.shape, f"{name}: shapes differ {tuple(got[name].shape)} vs {tuple(want[name].shape)}"
        diff = (a - b)
        rel = float(diff.norm() / b.norm().clamp_min(1e-12))
        mx = float(diff.abs().max())
        pts.append(TracePoint(name, mx, rel, rel <= rel_tol or mx <= abs_tol))
    return TraceReport(pts)


def oracle_trace(input_ids: torch.Tensor, weights: dict, cfg, dtype=torch.float32) -> dict:
    from .functional import causal_lm_forward

    w = {k: v.detach().to("cpu", dtype) for k, v in weights.items()}
    trace: dict = {}
    causal_lm_forward(input_ids.cpu().long(), w, cfg, trace=trace)
    return trace


def verify_against_oracle(model, input_ids: torch.Tensor, rel_tol: float = 3e-2) -> TraceReport:
    """``model``: a ``NativeCausalLM``. Runs it with tracing on and compares with the fp32 oracle on the same weights."""
    model.trace = {}
    try:
        targets = torch.zeros_like(input_ids)
        with torch.no_grad():
            model.logprobs(input_ids.to(model.device), targets.to(model.device))
        got = dict(model.trace)
    finally:
        model.trace = None
    want = oracle_trace(input_ids, model.state_dict(), model.cfg)
    return compare_traces(got, want, rel_tol)
