"""Multi-GPU layer: symmetric peer memory, fused tensor-parallel GEMM collectives, the sharded
optimizer with in-kernel reduce-scatter / all-gather, trainer->engine weight sync, MoE dispatch."""

from .ep import ExpertParallel, PeerFailure
from .fsdp import FlatBuckets, ShardedAdamW
from .symm import PeerComm, SymmBuffer
from .tp import TensorParallel
from .weight_sync import WeightSyncPlan, sync_engine_from_buckets

__all__ = ["ExpertParallel", "PeerFailure", "FlatBuckets", "ShardedAdamW", "PeerComm", "SymmBuffer", "TensorParallel", "WeightSyncPlan",
           "sync_engine_from_buckets"]
