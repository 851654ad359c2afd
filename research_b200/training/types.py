"""Data types shared by rollout generation, training backends and loops.

Public surface kept from the reference (rollouts/training/types.py:18-660): ``Status``,
``Sample``, ``RolloutBatch``, ``RolloutConfig``, ``SFTTrainingConfig``, ``TrainerConfig``,
``RLTrainingConfig``, ``TrainFuture`` and ``ImmediateTrainFuture``. Futures are awaitable with
``asyncio`` (the reference uses ``trio.Event``); ``result()`` can also be read synchronously
once ``done()``.
"""

from __future__ import annotations

import asyncio
import threading
from dataclasses import asdict, dataclass, field
from enum import Enum
from typing import Any, Callable, Generic, TypeVar

T = TypeVar("T")


class Status(Enum):
    PENDING = "pending"
    COMPLETED = "completed"
    TRUNCATED = "truncated"
    ABORTED = "aborted"
    FAILED = "failed"


@dataclass
class Sample:
    """One training example: a prompt, the generated response as tokens, its mask and reward."""

    id: str = ""
    index: int | None = None
    group_index: int | None = None
    input: dict[str, Any] = field(default_factory=dict)
    prompt: str | list[dict[str, str]] = ""
    ground_truth: Any | None = None
    trajectory: Any | None = None
    tokens: list[int] = field(default_factory=list)
    response_length: int = 0
    loss_mask: list[float] = field(default_factory=list)
    reward: float = 0.0
    rollout_log_probs: list[float] | None = None
    score: Any | None = None
    environment_state: dict[str, Any] | None = None
    status: Status = Status.PENDING
    metadata: dict[str, Any] = field(default_factory=dict)
    weight_version: int = 0

    @property
    def response(self) -> str:
        """Text of the response when the sample came from an agent trajectory or carries one."""
        if "response_text" in self.metadata:
            return str(self.metadata["response_text"])
        traj = self.trajectory
        if traj is not None and getattr(traj, "messages", None):
            for m in reversed(traj.messages):
                if getattr(m, "role", None) == "assistant":
                    c = getattr(m, "content", "")
                    return c if isinstance(c, str) else str(c)
        return ""

    @property
    def response_tokens(self) -> list[int]:
        return self.tokens[len(self.tokens) - self.response_length:] if self.response_length else []

    def to_dict(self) -> dict[str, Any]:
        d = {
            "id": self.id, "index": self.index, "group_index": self.group_index, "input": self.input,
            "prompt": self.prompt, "ground_truth": self.ground_truth, "tokens": list(self.tokens),
            "response_length": self.response_length, "loss_mask": list(self.loss_mask), "reward": self.reward,
            "rollout_log_probs": list(self.rollout_log_probs) if self.rollout_log_probs is not None else None,
            "status": self.status.value, "metadata": self.metadata, "weight_version": self.weight_version,
            "environment_state": self.environment_state,
        }
        if self.score is not None and hasattr(self.score, "to_dict"):
            d["score"] = self.score.to_dict()
        return d

    @staticmethod
    def from_dict(data: dict[str, Any]) -> "Sample":
        d = dict(data)
        d.pop("score", None)
        status = d.pop("status", "pending")
        known = {f for f in Sample.__dataclass_fields__}
        s = Sample(**{k: v for k, v in d.items() if k in known})
        s.status = Status(status) if not isinstance(status, Status) else status
        return s


@dataclass
class RolloutBatch:
    """A batch of finished rollouts in columnar form."""

    tokens: list[list[int]]
    loss_masks: list[list[float]]
    rewards: list[float]
    response_lengths: list[int]
    group_indices: list[int] = field(default_factory=list)
    rollout_log_probs: list[list[float]] | None = None
    samples: list[Sample] = field(default_factory=list)
    metadata: dict[str, Any] = field(default_factory=dict)

    def __len__(self) -> int:
        return len(self.tokens)


@dataclass
class RolloutConfig:
    batch_size: int
    n_samples_per_prompt: int = 1
    over_sampling_factor: float = 1.0
    generate_fn: Callable | None = None
    score_fn: Callable | None = None
    filter_fn: Callable | None = None

    def to_dict(self) -> dict[str, Any]:
        return {"batch_size": self.batch_size, "n_samples_per_prompt": self.n_samples_per_prompt,
                "over_sampling_factor": self.over_sampling_factor,
                "generate_fn": getattr(self.generate_fn, "__name__", None),
                "score_fn": getattr(self.score_fn, "__name__", None),
                "filter_fn": getattr(self.filter_fn, "__name__", None)}

    @staticmethod
    def from_dict(data: dict[str, Any], generate_fn=None, score_fn=None, filter_fn=None) -> "RolloutConfig":
        return RolloutConfig(batch_size=data["batch_size"], n_samples_per_prompt=data.get("n_samples_per_prompt", 1),
                             over_sampling_factor=data.get("over_sampling_factor", 1.0), generate_fn=generate_fn,
                             score_fn=score_fn, filter_fn=filter_fn)


@dataclass(frozen=True)
class SFTTrainingConfig:
    num_steps: int
    batch_size: int
    log_every: int = 100
    checkpoint_every: int = 500

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    @staticmethod
    def from_dict(data: dict[str, Any]) -> "SFTTrainingConfig":
        return SFTTrainingConfig(**data)


@dataclass(frozen=True)
class TrainerConfig:
    """Micro-batching and clipping. Give ``micro_batch_size`` or ``num_minibatches``, not both."""

    micro_batch_size: int | None = None
    num_minibatches: int | None = None
    max_grad_norm: float | None = 1.0

    def __post_init__(self) -> None:
        assert not (self.micro_batch_size is not None and self.num_minibatches is not None), \
            "set micro_batch_size or num_minibatches, not both"
        assert self.micro_batch_size is None or self.micro_batch_size > 0
        assert self.num_minibatches is None or self.num_minibatches > 0

    def get_num_minibatches(self, batch_size: int) -> int:
        if self.num_minibatches is not None:
            assert batch_size % self.num_minibatches == 0, "batch must split evenly into minibatches"
            return self.num_minibatches
        if self.micro_batch_size is not None:
            assert batch_size % self.micro_batch_size == 0, "batch must be a multiple of micro_batch_size"
            return batch_size // self.micro_batch_size
        return 1


@dataclass(frozen=True)
class RLTrainingConfig:
    num_steps: int
    sync_every: int = 10
    baseline: float = 0.0
    log_every: int = 10
    checkpoint_every: int = 100

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    @staticmethod
    def from_dict(data: dict[str, Any]) -> "RLTrainingConfig":
        return RLTrainingConfig(**data)


class TrainFuture(Generic[T]):
    """Result of an operation that may still be running (Tinker-style API)."""

    def __init__(self, operation: str = "") -> None:
        self.operation = operation
        self._done = threading.Event()
        self._result: T | None = None
        self._error: BaseException | None = None

    def set_result(self, value: T) -> None:
        self._result = value
        self._done.set()

    def set_exception(self, err: BaseException) -> None:
        self._error = err
        self._done.set()

    def done(self) -> bool:
        return self._done.is_set()

    def wait(self, timeout: float | None = None) -> T:
        if not self._done.wait(timeout):
            raise TimeoutError(f"{self.operation} did not finish in {timeout}s")
        if self._error is not None:
            raise self._error
        return self._result  # type: ignore[return-value]

    async def result(self) -> T:
        while not self._done.is_set():
            await asyncio.sleep(0.001)
        return self.wait(0)


class ImmediateTrainFuture(Generic[T]):
    """A future that is already resolved (synchronous backends)."""

    def __init__(self, result: T, operation: str = "") -> None:
        self._result = result
        self.operation = operation

    def done(self) -> bool:
        return True

    def wait(self, timeout: float | None = None) -> T:
        return self._result

    async def result(self) -> T:
        return self._result
