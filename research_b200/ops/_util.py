"""Helpers shared by the kernel wrappers: raw pointers, the current stream, the status word."""

from __future__ import annotations

import ctypes

import torch

STATUS_NAMES = {
    0: "ok",
    1: "timeout: producer waited for a free smem stage",
    2: "timeout: MMA issuer waited for TMA data",
    3: "timeout: epilogue waited for the accumulator",
    4: "timeout: MMA issuer waited for TMEM to drain",
    5: "timeout: wait on a flag written by another GPU",
    6: "index out of range (block table / slot / token / expert)",
    7: "bad argument",
}

_status: dict[int, torch.Tensor] = {}


class KernelStatusError(RuntimeError):
    """A kernel recorded a non-zero status word (bounded wait ran out, bad index, ...)."""


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream_handle(device: torch.device | None = None) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def status_tensor(device: torch.device | int | None = None) -> torch.Tensor:
    """One int32 status word per device, written by kernels with atomicCAS(0 -> code)."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _status[idx]


def check_status(device: torch.device | int | None = None, reset: bool = True) -> None:
    """Synchronise, read the status word and raise if a kernel reported a failure."""
    st = status_tensor(device)
    code = int(st.item())
    if code != 0:
        if reset:
            st.zero_()
        raise KernelStatusError(f"kernel status {code}: {STATUS_NAMES.get(code, 'unknown')}")


# Number of kernel launches issued through the wrappers (every wrapper reports exactly one
# launch per call through check_rc; the split-KV merge adds its own).
LAUNCH_COUNT = [0]


def check_rc(rc: int, what: str, launches: int = 1) -> None:
    LAUNCH_COUNT[0] += launches
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def require_bf16_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.bfloat16:
            raise TypeError("expected CUDA bfloat16 tensors")
