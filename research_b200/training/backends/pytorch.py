"""Single-device training backend (API of rollouts/training/backends/pytorch.py:42)."""

from __future__ import annotations

from .native import NativeTrainingBackend


class PyTorchTrainingBackend(NativeTrainingBackend):
    """One GPU (or CPU): micro-batched forward/backward, fused clip + AdamW, checkpoints.

    Differences from the reference class of the same name: the model is the kernel-backed
    ``NativeCausalLM`` instead of an HF module, and ``optim_step`` is one fused kernel family
    instead of ``clip_grad_norm_`` + ``optimizer.step()``.
    """

    def __init__(self, model_config, weights=None, **kw):
        kw.pop("comm", None)
        super().__init__(model_config, weights, comm=None, **kw)
