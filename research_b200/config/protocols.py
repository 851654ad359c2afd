"""Structural interfaces of experiment configs (rollouts/config/protocols.py:20-132).

A config does not inherit from anything here: any object with the right members satisfies the protocol
(``isinstance(cfg, HasModelConfig)`` works because the protocols are runtime-checkable), so projects compose their
own frozen dataclasses and the evaluation / training entry points only ask for the pieces they use.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Callable, Protocol, runtime_checkable

from ..agents.dtypes import Endpoint, EvalConfig, Message


@runtime_checkable
class HasModelConfig(Protocol):
    """Can produce the ``Endpoint`` the agent loop talks to."""

    def to_endpoint(self) -> Endpoint: ...


@runtime_checkable
class HasEnvironmentConfig(Protocol):
    """Names an environment and turns one dataset row into the conversation's first messages."""

    env_name: str

    def prepare_messages(self, sample_data: dict[str, Any]) -> list[Message]: ...


@runtime_checkable
class HasEvaluationConfig(Protocol):
    """Can produce the ``EvalConfig`` of ``agents.evaluation.evaluate`` for a given score function."""

    def to_eval_config(self, *args: Any, **kwargs: Any) -> EvalConfig: ...


@runtime_checkable
class HasOutputConfig(Protocol):
    """Says where results go and what the run is called."""

    output_dir: Path
    experiment_name: str


ScoreFn = Callable[..., Any]

PROTOCOLS = {"model": HasModelConfig, "environment": HasEnvironmentConfig, "evaluation": HasEvaluationConfig,
             "output": HasOutputConfig}
