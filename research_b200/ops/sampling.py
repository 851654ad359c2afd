"""Seeded sampling with log-probabilities (csrc/ops_sm100.cu) and the reference twin.

Semantics of the reference sampler (rollouts/inference/sampling.py:10-58): the token is drawn
from ``softmax(logits / T)`` (argmax when ``T == 0``) while the reported log-probability is
``log_softmax(logits)[token]`` of the UNSCALED logits, i.e. the true policy probability.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _native
from ._util import check_rc, ptr, stream_handle

c_int, c_ll, c_ull, c_vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_void_p


def _lib() -> ctypes.CDLL:
    lib = _native.load("rb_ops")
    if not getattr(lib, "_rb_typed_s", False):
        lib.rb_sample_logprob.argtypes = [c_vp, c_ll, c_int, c_int, c_vp, c_vp, c_vp, c_ull, c_vp, c_vp, c_vp]
        lib.rb_sample_logprob.restype = c_int
        lib.rb_sample_logprob_split.argtypes = [c_vp, c_ll, c_int, c_int, c_vp, c_vp, c_vp, c_ull, c_vp, c_vp, c_vp, c_vp, c_int, c_vp]
        lib.rb_sample_logprob_split.restype = c_int
        lib.rb_token_logprob.argtypes = [c_vp, c_ll, c_int, c_int, c_vp, c_vp, c_vp]
        lib.rb_token_logprob.restype = c_int
        lib._rb_typed_s = True
    return lib


def sample_with_logprobs_reference(logits: torch.Tensor, temperatures: torch.Tensor, generator=None):
    """PyTorch twin of the reference sampler: returns (tokens int64 [B], logprobs fp32 [B])."""
    logits = logits.float()
    logprobs = torch.log_softmax(logits, dim=-1)
    greedy = temperatures <= 0
    safe_t = torch.where(greedy, torch.ones_like(temperatures), temperatures)
    probs = torch.softmax(logits / safe_t[:, None], dim=-1)
    sampled = torch.multinomial(probs, 1, generator=generator).squeeze(-1)
    tokens = torch.where(greedy, logits.argmax(-1), sampled)
    return tokens, logprobs.gather(-1, tokens[:, None]).squeeze(-1)


def sample_with_logprobs(logits, temperatures, seeds=None, step: int = 0, step_tensor=None, out_tokens=None,
                         out_logprobs=None):
    """Sample one token per row of fp32 ``logits [B, V]``.

    ``seeds`` (uint64 per row, stored as int64) and ``step`` select the random stream, so a
    request reproduces its samples regardless of which batch slot it occupies.
    """
    if not logits.is_cuda:
        g = None
        if seeds is not None:
            g = torch.Generator().manual_seed(int(seeds[0].item()) * 1000003 + step)
        return sample_with_logprobs_reference(logits, temperatures, g)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    B, V = logits.shape
    if seeds is None:
        seeds = torch.zeros(B, dtype=torch.int64, device=logits.device)
    if out_tokens is None:
        out_tokens = torch.empty(B, dtype=torch.int32, device=logits.device)
    if out_logprobs is None:
        out_logprobs = torch.empty(B, dtype=torch.float32, device=logits.device)
    part, tickets = _split_scratch(logits.device, B)
    rc = _lib().rb_sample_logprob_split(ptr(logits), logits.stride(0), B, V, ptr(temperatures), ptr(seeds), ptr(step_tensor),
                                        step, ptr(out_tokens), ptr(out_logprobs), ptr(part), ptr(tickets), 0,
                                        stream_handle(logits.device))
    check_rc(rc, "rb_sample_logprob_split")
    return out_tokens, out_logprobs


_SPLIT_SCRATCH: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
_SPLIT_KEEP: list = []


def _split_scratch(device: torch.device, rows: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-device chunk records ([rows, 8 chunks, 4] fp32) and row tickets of the split sampler; launches on one
    stream run in order, so one pair serves them all. Never shrinks (captured graphs keep the address)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    cur = _SPLIT_SCRATCH.get(idx)
    if cur is None or cur[1].numel() < rows:
        n = max(rows, 1024)
        if cur is not None:
            _SPLIT_KEEP.append(cur)       # a captured graph may still point at the old pair
        _SPLIT_SCRATCH[idx] = (torch.empty(n * 8 * 4, dtype=torch.float32, device=device),
                               torch.zeros(n, dtype=torch.int32, device=device))
    return _SPLIT_SCRATCH[idx]


def token_logprobs(logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits)[token]`` per row without materialising the log-softmax."""
    if not logits.is_cuda:
        return torch.log_softmax(logits.float(), -1).gather(-1, tokens.long()[:, None]).squeeze(-1)
    assert logits.dtype == torch.float32 and tokens.dtype == torch.int32
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.float32, device=logits.device)
    rc = _lib().rb_token_logprob(ptr(logits), logits.stride(0), B, V, ptr(tokens), ptr(out), stream_handle(logits.device))
    check_rc(rc, "rb_token_logprob")
    return out
