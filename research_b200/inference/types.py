"""Value types of the inference engine: what configures it, what a request asks for, what a step schedules, what comes
back for training, and the host-side view of one sequence.

The names are the reference's public surface (rollouts/inference/types.py:16-171), so code written against it keeps
working; three fields it declares without using them (``cache_type``, ``tensor_parallel_size``,
``gpu_memory_utilization``) select real behaviour here, and the engine-specific knobs (CUDA-graph batch sizes, KV pool
size, expert parallelism) are added. The engine's own sequences live in the C++ core; ``Sequence`` is the Python mirror
the pure-function scheduler and its tests work on.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Literal

CacheKind = Literal["paged", "radix", "none"]
FinishReason = Literal["stop", "length"]

# decode batch sizes for which a CUDA graph is captured; a batch runs in the smallest graph that holds it
DEFAULT_GRAPH_BATCHES = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 160, 192, 224, 256)


# ------------------------------------------------------------------------------------------- requests and results
@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    max_tokens: int = 256
    stop_token_ids: frozenset[int] = frozenset()
    seed: int | None = None

    def stops_at(self, token_id: int) -> bool:
        return token_id in self.stop_token_ids


@dataclass(frozen=True)
class TrainingSample:
    """A finished generation in the form RL training consumes: token ids on both sides, the sampling log-probabilities
    of the completion, and the version of the weights that produced it (for off-policy corrections)."""

    prompt_tokens: tuple[int, ...]
    completion_tokens: tuple[int, ...]
    logprobs: tuple[float, ...]
    ref_logprobs: tuple[float, ...] | None
    weight_version: int
    finish_reason: FinishReason
    cached_tokens: int = 0                 # prompt tokens served from the prefix cache

    @property
    def tokens(self) -> tuple[int, ...]:
        return self.prompt_tokens + self.completion_tokens

    @property
    def sum_logprob(self) -> float:
        return float(sum(self.logprobs))


# ------------------------------------------------------------------------------------------- engine and scheduler
@dataclass(frozen=True)
class EngineConfig:
    model_path: str = ""
    cache_type: CacheKind = "radix"
    block_size: int = 16
    max_batch_size: int = 256
    max_model_len: int = 8192
    gpu_memory_utilization: float = 0.9
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    max_tokens_per_batch: int = 0          # 0: max_batch_size * 512
    num_kv_blocks: int = 0                 # 0: sized from gpu_memory_utilization
    use_cuda_graphs: bool = True
    graph_batch_sizes: tuple[int, ...] = DEFAULT_GRAPH_BATCHES
    dtype: str = "bfloat16"
    seed: int = 0
    ignore_eos: bool = False

    def token_budget(self) -> int:
        return self.max_tokens_per_batch or self.max_batch_size * 512


@dataclass(frozen=True)
class SchedulerConfig:
    max_batch_size: int
    max_tokens_per_batch: int
    block_size: int

    def blocks_for(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)


@dataclass(frozen=True)
class SchedulerOutput:
    """Sequence ids of one step: prompts to prefill, sequences to decode, sequences pushed back to the waiting queue."""

    prefill_seqs: tuple[int, ...]
    decode_seqs: tuple[int, ...]
    preempted_seqs: tuple[int, ...]

    @property
    def idle(self) -> bool:
        return not (self.prefill_seqs or self.decode_seqs)


@dataclass(frozen=True)
class InferenceContext:
    """What the attention layers of one forward pass need, passed explicitly instead of through globals: where the new
    keys and values go (``slot_mapping``), which cache blocks every sequence owns, how long the sequences are, and for
    prefill over cached prefixes how many of the tokens are new (``query_lens``)."""

    is_prefill: bool
    slot_mapping: tuple[int, ...] | None = None
    block_tables: tuple[tuple[int, ...], ...] | None = None
    seq_lens: tuple[int, ...] | None = None
    max_seq_len: int = 0
    block_mask: object | None = None
    query_lens: tuple[int, ...] | None = None
    sliding_window: int = 0


# ------------------------------------------------------------------------------------------- one sequence, host side
class SequenceStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class Sequence:
    seq_id: int
    token_ids: list[int]                   # prompt followed by what has been generated
    block_ids: list[int]
    num_prompt_tokens: int
    status: SequenceStatus
    temperature: float
    max_tokens: int
    stop_token_ids: frozenset[int]
    output_logprobs: list[float] = field(default_factory=list)

    @property
    def num_generated(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def is_finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED

    def hit_limit(self) -> FinishReason | None:
        """Why generation should end now, if it should: a stop token was produced, or the token allowance is used up."""
        if self.num_generated and self.token_ids[-1] in self.stop_token_ids:
            return "stop"
        return "length" if self.num_generated >= self.max_tokens else None

    def append_token(self, token_id: int, logprob: float) -> None:
        if self.status is not SequenceStatus.RUNNING:
            raise AssertionError(f"sequence {self.seq_id} is {self.status.value}, not running")
        self.token_ids.append(token_id)
        self.output_logprobs.append(logprob)

    def to_training_sample(self, weight_version: int) -> TrainingSample:
        if not self.is_finished:
            raise AssertionError(f"sequence {self.seq_id} has not finished")
        n = self.num_prompt_tokens
        ended_on_stop = bool(self.num_generated) and self.token_ids[-1] in self.stop_token_ids
        return TrainingSample(tuple(self.token_ids[:n]), tuple(self.token_ids[n:]), tuple(self.output_logprobs), None, weight_version,
                              "stop" if ended_on_stop else "length")
