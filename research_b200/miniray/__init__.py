"""miniray: process launch, worker channels, multi-node cluster, NCCL env, GPU affinity."""

from .cluster import Cluster, NodeConfig
from .gpu_affinity import get_gpu_cpu_set, get_gpu_numa_node, set_gpu_affinity
from .nccl import NCCLConfig, create_nccl_configs, restore_nccl_env, setup_nccl_env
from .remote_worker import RemoteWorker
from .worker import SharedMemory, Worker, shutdown_workers, spawn_training_workers, wait_any
from .worker_server import WorkerServer

__all__ = ["Cluster", "NodeConfig", "get_gpu_cpu_set", "get_gpu_numa_node", "set_gpu_affinity", "NCCLConfig",
           "create_nccl_configs", "restore_nccl_env", "setup_nccl_env", "RemoteWorker", "SharedMemory", "Worker",
           "shutdown_workers", "spawn_training_workers", "wait_any", "WorkerServer"]
