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
    train_smoke(dev)
    torch.cuda.synchronize()
    ops.check_status()
    print("smoke ok")


def train_smoke(device: torch.device) -> None:
    """One forward + backward + optimizer step on the kernel path (tcgen05 GEMMs, flash attention at head size 64,
    fused log-prob loss, sharded AdamW kernels)."""
    from .models import get_preset
    from .training.backends.native import NativeTrainingBackend

    cfg = get_preset("tiny-qwen2", num_layers=2, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=512)
    backend = NativeTrainingBackend(cfg, None, device=device, loss_fn="sft", lr=1e-3)
    ids = torch.randint(0, cfg.vocab_size, (2, 160), generator=torch.Generator().manual_seed(0))
    m = backend.forward_backward({"input_ids": ids, "labels": ids.clone()}).wait()
    o = backend.optim_step().wait()
    assert m["loss"] == m["loss"] and o["grad_norm"] > 0, (m, o)
