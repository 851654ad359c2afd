"""Thin helpers over ``torch.distributed`` (rollouts/training/distributed_utils.py:37-390):
process-group bootstrap from the environment, a gloo side group for CPU objects, rank helpers,
generic collectives and ``distributed_masked_whiten`` for advantage whitening."""

from __future__ import annotations

import os
from datetime import timedelta

import torch
import torch.distributed as dist

_GLOO_GROUP: dist.ProcessGroup | None = None


def init_process_group(backend: str | None = None, timeout_s: float = 1800.0) -> None:
    """Initialise the default group from ``RANK`` / ``WORLD_SIZE`` / ``MASTER_*`` (no-op if done)."""
    if dist.is_initialized():
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend=backend, init_method="env://", timeout=timedelta(seconds=timeout_s))


def init_gloo_group() -> dist.ProcessGroup:
    global _GLOO_GROUP
    assert dist.is_initialized(), "call init_process_group first"
    if _GLOO_GROUP is None:
        _GLOO_GROUP = dist.new_group(backend="gloo")
    return _GLOO_GROUP


def get_gloo_group() -> dist.ProcessGroup:
    return _GLOO_GROUP if _GLOO_GROUP is not None else init_gloo_group()


def get_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def is_main_process() -> bool:
    return get_rank() == 0


def barrier() -> None:
    if get_world_size() > 1:
        dist.barrier()


def all_reduce(tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
    if get_world_size() == 1:
        return tensor
    ops = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "mean": dist.ReduceOp.SUM}
    dist.all_reduce(tensor, op=ops[op])
    if op == "mean":
        tensor /= get_world_size()
    return tensor


def all_gather(tensor: torch.Tensor) -> list[torch.Tensor]:
    if get_world_size() == 1:
        return [tensor]
    out = [torch.empty_like(tensor) for _ in range(get_world_size())]
    dist.all_gather(out, tensor.contiguous())
    return out


def broadcast(tensor: torch.Tensor, src: int = 0) -> torch.Tensor:
    if get_world_size() > 1:
        dist.broadcast(tensor, src=src)
    return tensor


def distributed_masked_whiten(values: torch.Tensor, mask: torch.Tensor, shift_mean: bool = True, eps: float = 1e-8) -> torch.Tensor:
    """Whiten ``values`` over masked entries using statistics pooled across ranks (one float32[3] all-reduce)."""
    m = mask.to(values.dtype)
    stats = torch.stack([(values * m).sum(), (values * values * m).sum(), m.sum()]).float()
    stats = all_reduce(stats, "sum")
    count = stats[2].clamp(min=1)
    mean = stats[0] / count
    var = (stats[1] / count - mean * mean).clamp(min=0)
    var = var * count / (count - 1).clamp(min=1)  # unbiased, like torch.var
    out = (values - mean) * torch.rsqrt(var + eps)
    if not shift_mean:
        out = out + mean
    return out


def cleanup() -> None:
    global _GLOO_GROUP
    _GLOO_GROUP = None
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def print_rank_0(message: str) -> None:
    if is_main_process():
        print(message, flush=True)
