"""Tiny end-to-end check on cuda:0 used by ``__graft_entry__.smoke``."""

from __future__ import annotations

import torch


def run_smoke() -> None:
    assert torch.cuda.is_available(), "smoke() needs a CUDA device"
    from . import ops

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    a = torch.randn(256, 512, device=dev).bfloat16()
    b = torch.randn(384, 512, device=dev).bfloat16()
    c = ops.gemm(a, b)
    ref = a.float() @ b.float().t()
    assert (c.float() - ref).abs().max().item() < 1.0
    try:
        from .inference.smoke import engine_smoke
    except ImportError:
        engine_smoke = None
    if engine_smoke is not None:
        engine_smoke(dev)
    torch.cuda.synchronize()
    ops.check_status()
    print("smoke ok")
