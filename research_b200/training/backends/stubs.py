"""Placeholders the reference also ships as stubs: JAX and torchax backends
(rollouts/training/backends/jax_backend.py:29, torchax_backend.py:27). Every method raises
``NotImplementedError``; they exist so configuration code can name them. The third stub of the reference,
the torch.func backend, is a working backend here (``backends/torch_func.py``)."""

from __future__ import annotations


class _Unavailable:
    _why = "not implemented"

    def __init__(self, *a, **k):
        raise NotImplementedError(f"{type(self).__name__}: {self._why}")

    def forward_backward(self, batch):
        raise NotImplementedError

    def optim_step(self):
        raise NotImplementedError

    def get_weights(self):
        raise NotImplementedError

    def load_weights(self, weights):
        raise NotImplementedError


class JAXTrainingBackend(_Unavailable):
    _why = "JAX is not part of this framework (sm_100a CUDA only)"


class TorchaxTrainingBackend(_Unavailable):
    _why = "torchax is not part of this framework (sm_100a CUDA only)"
