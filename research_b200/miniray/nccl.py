"""Environment set-up for ``torch.distributed`` / NCCL ranks (miniray/nccl.py:16-200)."""

from __future__ import annotations

import os
from dataclasses import asdict, dataclass

_KEYS = ("MASTER_ADDR", "MASTER_PORT", "WORLD_SIZE", "RANK", "LOCAL_RANK", "CUDA_VISIBLE_DEVICES", "NCCL_NVLS_ENABLE")


@dataclass(frozen=True)
class NCCLConfig:
    master_addr: str
    master_port: int
    world_size: int
    rank: int
    local_rank: int = 0
    cuda_visible_devices: str | None = None
    nvls: bool = False   # in-switch reduction is opt-in: a rank dying with NVLS-bound memory faults its peers

    def to_dict(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_dict(d: dict) -> "NCCLConfig":
        return NCCLConfig(**d)


def setup_nccl_env(cfg: NCCLConfig) -> dict[str, str | None]:
    """Export the rendezvous variables; returns the previous values for ``restore_nccl_env``."""
    assert 0 <= cfg.rank < cfg.world_size
    old = {k: os.environ.get(k) for k in _KEYS}
    os.environ.update({"MASTER_ADDR": cfg.master_addr, "MASTER_PORT": str(cfg.master_port),
                       "WORLD_SIZE": str(cfg.world_size), "RANK": str(cfg.rank), "LOCAL_RANK": str(cfg.local_rank),
                       "NCCL_NVLS_ENABLE": "1" if cfg.nvls else "0"})
    if cfg.cuda_visible_devices is not None:
        os.environ["CUDA_VISIBLE_DEVICES"] = cfg.cuda_visible_devices
    return old


def restore_nccl_env(old: dict[str, str | None]) -> None:
    for k, v in old.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


def create_nccl_configs(master_addr: str, master_port: int, nodes: list[int]) -> list[NCCLConfig]:
    """``nodes[i]`` = GPUs on node i; ranks are numbered node by node."""
    world = sum(nodes)
    out, rank = [], 0
    for gpus in nodes:
        for local in range(gpus):
            out.append(NCCLConfig(master_addr, master_port, world, rank, local))
            rank += 1
    return out
