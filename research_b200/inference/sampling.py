"""Sampling entry points of the engine (rollouts/inference/sampling.py:10-103).

``sample_with_logprobs`` dispatches to the CUDA kernel for device tensors (Gumbel-max with a
counter-based generator, one pass over the logits) and to the PyTorch twin on CPU. In both,
the log-probability comes from the unscaled logits.
"""

from __future__ import annotations

import torch

from ..ops import sampling as _s


def sample_with_logprobs(logits: torch.Tensor, temperatures: torch.Tensor, seeds: torch.Tensor | None = None,
                         step: int = 0, generator: torch.Generator | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    assert logits.dim() == 2 and temperatures.shape == (logits.shape[0],)
    if logits.is_cuda:
        tok, lp = _s.sample_with_logprobs(logits.float().contiguous(), temperatures.float(), seeds, step)
        return tok.long(), lp
    return _s.sample_with_logprobs_reference(logits, temperatures.float(), generator)


def sample_greedy(logits: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return sample_with_logprobs(logits, torch.zeros(logits.shape[0], device=logits.device))


def compute_logprobs_for_tokens(logits: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits)[..., token]`` for ``logits [..., V]``."""
    flat = logits.reshape(-1, logits.shape[-1])
    toks = token_ids.reshape(-1)
    if flat.is_cuda:
        out = _s.token_logprobs(flat.float().contiguous(), toks.to(torch.int32))
    else:
        out = torch.log_softmax(flat.float(), -1).gather(-1, toks.long()[:, None]).squeeze(-1)
    return out.reshape(token_ids.shape)
