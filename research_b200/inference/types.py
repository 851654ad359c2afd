"""Configuration, output and per-sequence state types of the inference engine.

Public surface kept from the reference (rollouts/inference/types.py:16-171): ``EngineConfig``,
``SamplingParams``, ``SchedulerConfig``, ``SchedulerOutput``, ``TrainingSample``,
``InferenceContext``, ``Sequence``/``SequenceStatus``. Fields the reference declares but never
uses (``cache_type``, ``tensor_parallel_size``, ``gpu_memory_utilization``) are honoured here.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Literal


@dataclass(frozen=True)
class EngineConfig:
    model_path: str = ""
    cache_type: Literal["paged", "radix", "none"] = "radix"
    block_size: int = 16
    max_batch_size: int = 256
    max_model_len: int = 8192
    gpu_memory_utilization: float = 0.9
    tensor_parallel_size: int = 1
    # additions
    max_tokens_per_batch: int = 0          # 0 -> max_batch_size * 512 like the reference engine
    num_kv_blocks: int = 0                 # 0 -> sized from gpu_memory_utilization
    use_cuda_graphs: bool = True
    graph_batch_sizes: tuple[int, ...] = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 160, 192, 224, 256)
    dtype: str = "bfloat16"
    seed: int = 0
    ignore_eos: bool = False
    expert_parallel_size: int = 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    max_tokens: int = 256
    stop_token_ids: frozenset[int] = frozenset()
    seed: int | None = None


@dataclass(frozen=True)
class SchedulerConfig:
    max_batch_size: int
    max_tokens_per_batch: int
    block_size: int


@dataclass(frozen=True)
class TrainingSample:
    """One finished generation, ready for RL training."""

    prompt_tokens: tuple[int, ...]
    completion_tokens: tuple[int, ...]
    logprobs: tuple[float, ...]
    ref_logprobs: tuple[float, ...] | None
    weight_version: int
    finish_reason: Literal["stop", "length"]
    cached_tokens: int = 0


@dataclass(frozen=True)
class SchedulerOutput:
    prefill_seqs: tuple[int, ...]
    decode_seqs: tuple[int, ...]
    preempted_seqs: tuple[int, ...]


@dataclass(frozen=True)
class InferenceContext:
    """Everything an attention layer needs for one forward pass (explicit, immutable)."""

    is_prefill: bool
    slot_mapping: tuple[int, ...] | None = None
    block_tables: tuple[tuple[int, ...], ...] | None = None
    seq_lens: tuple[int, ...] | None = None
    max_seq_len: int = 0
    block_mask: object | None = None
    # additions for varlen prefill with cached prefixes
    query_lens: tuple[int, ...] | None = None
    sliding_window: int = 0


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


@dataclass
class Sequence:
    seq_id: int
    token_ids: list[int]
    block_ids: list[int]
    num_prompt_tokens: int
    status: SequenceStatus
    temperature: float
    max_tokens: int
    stop_token_ids: frozenset[int]
    output_logprobs: list[float] = field(default_factory=list)

    def append_token(self, token_id: int, logprob: float) -> None:
        assert self.status == SequenceStatus.RUNNING
        self.token_ids.append(token_id)
        self.output_logprobs.append(logprob)

    @property
    def num_generated(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def is_finished(self) -> bool:
        return self.status == SequenceStatus.FINISHED

    def to_training_sample(self, weight_version: int) -> TrainingSample:
        assert self.status == SequenceStatus.FINISHED
        return TrainingSample(
            prompt_tokens=tuple(self.token_ids[: self.num_prompt_tokens]),
            completion_tokens=tuple(self.token_ids[self.num_prompt_tokens :]),
            logprobs=tuple(self.output_logprobs),
            ref_logprobs=None,
            weight_version=weight_version,
            finish_reason="stop" if self.token_ids[-1] in self.stop_token_ids else "length",
        )
