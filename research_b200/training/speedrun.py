"""Pre-training driver in the style of the speedrun script of the dev tree (dev/speedrun/single-file.py:1367-1560):
the functional speedrun GPT, Muon on the 2-D block matrices and Adam on embeddings, head, gates and scalars, a
constant-then-linear-cooldown learning rate, a sliding-window length that grows during the run, Muon momentum
warm-up, BOS-aligned packed batches. Runs on CPU for tests (explicit-mask attention) and on a GPU with the flash
kernel (``use_flash``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator

import torch

from ..models import speedrun as M
from .muon import Muon


@dataclass
class SpeedrunHyper:
    num_iterations: int = 1000
    cooldown_frac: float = 0.45           # final share of the run over which the learning rate falls linearly
    adam_lr: float = 0.008
    muon_lr: float = 0.05
    ws_short_final: int = 3               # window lengths in blocks at the end of the run
    ws_long_final: int = 13
    ws_steps: int = 3                     # the windows reach their final length in this many equal stages
    muon_momentum_warmup: int = 300
    attn_scale: float = 0.1


def get_lr(step: int, h: SpeedrunHyper) -> float:
    """Multiplier on every group's base rate: 1 until the cool-down starts, then linear to 0.1."""
    x = step / max(h.num_iterations, 1)
    if x < 1 - h.cooldown_frac:
        return 1.0
    w = (1 - x) / max(h.cooldown_frac, 1e-9)
    return w * 1.0 + (1 - w) * 0.1


def get_windows(step: int, h: SpeedrunHyper) -> tuple[int, int]:
    """(short, long) window lengths in blocks: they grow in ``ws_steps`` stages over the run."""
    stage = min(int(step / max(h.num_iterations, 1) * h.ws_steps), h.ws_steps - 1) + 1
    return max(1, h.ws_short_final * stage // h.ws_steps), max(1, h.ws_long_final * stage // h.ws_steps)


def get_muon_momentum(step: int, h: SpeedrunHyper, lo: float = 0.85, hi: float = 0.95) -> float:
    f = min(step / max(h.muon_momentum_warmup, 1), 1.0)
    return (1 - f) * lo + f * hi


def make_optimizers(w: dict[str, torch.Tensor], h: SpeedrunHyper):
    matrices = [p for n, p in w.items() if n.startswith("blocks.") and p.dim() == 2 and "gate" not in n]
    rest = [p for n, p in w.items() if not (n.startswith("blocks.") and p.dim() == 2 and "gate" not in n)]
    adam = torch.optim.Adam(rest, lr=h.adam_lr, betas=(0.8, 0.95), eps=1e-10)
    muon = Muon(matrices, lr=h.muon_lr, momentum=0.95)
    for opt in (adam, muon):
        for g in opt.param_groups:
            g["initial_lr"] = g["lr"]
    return adam, muon


def train(cfg: M.SpeedrunConfig, batches: Iterator[tuple[torch.Tensor, torch.Tensor, torch.Tensor]], h: SpeedrunHyper,
          seed: int = 0, device: str | torch.device = "cpu", use_flash: bool = False, log_every: int = 0) -> tuple[dict, list[float]]:
    """Runs ``h.num_iterations`` steps (or until ``batches`` ends); returns the weights and the loss per step."""
    dev = torch.device(device)
    w = {k: v.to(dev).requires_grad_(True) for k, v in M.init_weights(cfg, seed=seed).items()}
    adam, muon = make_optimizers(w, h)
    yarn = M.Yarn(cfg, h.attn_scale)
    losses: list[float] = []
    for step in range(h.num_iterations):
        try:
            inputs, targets, cu = next(batches)
        except StopIteration:
            break
        ws_short, ws_long = get_windows(step, h)
        yarn.follow(ws_long)                          # the rotary frequencies and the softmax scale follow the growing window
        loss = M.loss(w, inputs.to(dev).long(), targets.to(dev).long(), cfg, cu_seqlens=cu.to(dev), ws_short=ws_short, ws_long=ws_long,
                      use_flash=use_flash, yarn=yarn)
        loss.backward()
        mult = get_lr(step, h)
        for opt in (adam, muon):
            for g in opt.param_groups:
                g["lr"] = g["initial_lr"] * mult
        for g in muon.param_groups:
            g["momentum"] = get_muon_momentum(step, h)
        adam.step()
        muon.step()
        for p in w.values():
            p.grad = None
        losses.append(float(loss.detach()))
        if log_every and step % log_every == 0:
            print(f"step {step}: loss {losses[-1]:.4f} lr x{mult:.2f} windows {ws_short}/{ws_long}", flush=True)
    return {k: v.detach() for k, v in w.items()}, losses
