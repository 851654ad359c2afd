"""Muon: SGD-momentum whose 2-D updates are orthogonalised with the Polar Express iteration
(dev/speedrun/single-file.py:386-686; Amsel, Persson, Musco, Gower, arXiv 2505.16932).

Each of the five iterations is three GEMM-shaped products, all on the tcgen05 kernel:
``A = X X^T`` and ``B = b A + c A A`` through ``ops.gemm_symmetric`` (only the lower-triangle tiles
are computed, the epilogue mirrors them) and ``X <- a X + B X`` through the scaled-residual epilogue.
The reference runs the first two as Triton kernels and the third as ``baddbmm``.

``Muon`` keeps one momentum buffer per parameter. With ``torch.distributed`` initialised the
parameters are dealt round-robin to ranks: a rank orthogonalises only the updates it owns and the
results are exchanged with one ``all_gather`` per step over a flat bf16 buffer (gradients are assumed
to be already averaged, which is what the sharded trainer produces).
"""

from __future__ import annotations

import torch

from .. import ops

# (a, b, c) per iteration, computed in the paper for 5 iterations, safety factor 2e-2, cushion 2
POLAR_EXPRESS_COEFFS = [
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
]


def _pad8(x: torch.Tensor) -> tuple[torch.Tensor, tuple[int, int]]:
    """The kernels want both extents to be multiples of 8; zero padding does not change the iteration."""
    n, m = x.shape
    pn, pm = -n % 8, -m % 8
    if pn or pm:
        x = torch.nn.functional.pad(x, (0, pm, 0, pn))
    return x.contiguous(), (n, m)


def polar_express(G: torch.Tensor, coeffs=POLAR_EXPRESS_COEFFS) -> torch.Tensor:
    """Approximate the orthogonal polar factor of a 2-D ``G`` in bf16 (returns bf16, shape of ``G``)."""
    assert G.dim() == 2
    X = G.to(torch.bfloat16)
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.T
    X = X / (X.float().norm() * (1 + 2e-2) + 1e-6).to(X.dtype)
    X, (n, m) = _pad8(X)
    for a, b, c in coeffs:
        A = ops.gemm_symmetric(X)                                   # X X^T              [n, n]
        B = ops.gemm_symmetric(A, alpha=c, beta=b, residual=A)      # b A + c A A (A symmetric)
        X = ops.gemm(B, X, residual=X, b_mn_major=True, alpha=1.0, beta=a)   # a X + B X
    X = X[:n, :m]
    return X.T if transposed else X


def polar_express_reference(G: torch.Tensor, coeffs=POLAR_EXPRESS_COEFFS) -> torch.Tensor:
    X = G.float()
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.T
    X = X / (X.norm() * (1 + 2e-2) + 1e-6)
    for a, b, c in coeffs:
        A = X @ X.T
        X = a * X + (b * A + c * A @ A) @ X
    return X.T if transposed else X


class Muon(torch.optim.Optimizer):
    """``lr`` scales the orthogonalised update (times ``max(1, rows/cols)**0.5``); decoupled weight decay."""

    def __init__(self, params, lr: float = 0.02, momentum: float = 0.95, nesterov: bool = True, weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self) -> None:
        dist = torch.distributed
        world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        rank = dist.get_rank() if world > 1 else 0
        for group in self.param_groups:
            params = [p for p in group["params"] if p.grad is not None]
            updates: list[torch.Tensor | None] = []
            for i, p in enumerate(params):
                assert p.dim() == 2, "Muon is for 2-D parameters; use AdamW for the rest"
                st = self.state[p]
                if "momentum" not in st:
                    st["momentum"] = torch.zeros_like(p.grad, dtype=torch.float32)
                buf = st["momentum"]
                buf.lerp_(p.grad.float(), 1 - group["momentum"])
                g = p.grad.float().lerp(buf, group["momentum"]) if group["nesterov"] else buf
                updates.append(polar_express(g) if i % world == rank else None)
            if world > 1:
                sizes = [p.numel() for p in params]
                per_rank = max(sum(s for i, s in enumerate(sizes) if i % world == r) for r in range(world))
                mine = torch.zeros(per_rank, dtype=torch.bfloat16, device=params[0].device)
                off = 0
                for i, u in enumerate(updates):
                    if u is not None:
                        mine[off:off + sizes[i]] = u.reshape(-1)
                        off += sizes[i]
                gathered = torch.empty(world * per_rank, dtype=torch.bfloat16, device=mine.device)
                dist.all_gather_into_tensor(gathered, mine)
                offs = [0] * world
                for i, p in enumerate(params):
                    r = i % world
                    updates[i] = gathered[r * per_rank + offs[r]: r * per_rank + offs[r] + sizes[i]].view_as(p)
                    offs[r] += sizes[i]
            for p, u in zip(params, updates):
                if group["weight_decay"]:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                scale = max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                p.add_(u.to(p.dtype), alpha=-group["lr"] * scale)
