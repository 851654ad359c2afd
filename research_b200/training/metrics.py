"""Metric sinks: a protocol, a bounded JSONL file logger, an optional W&B logger and a fan-out.

Same surface as the reference (rollouts/training/metrics.py:22-250).
"""

from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Protocol, runtime_checkable


@runtime_checkable
class MetricsLogger(Protocol):
    def log(self, metrics: dict[str, float], step: int) -> None: ...
    def finish(self) -> None: ...


@dataclass
class JSONLLogger:
    """Appends one JSON object per call to ``<log_dir>/metrics.jsonl`` (stops after ``max_lines``)."""

    log_dir: Path | str
    filename: str = "metrics.jsonl"
    max_lines: int = 1_000_000
    _lines: int = field(default=0, init=False)
    _warned: bool = field(default=False, init=False)

    def __post_init__(self) -> None:
        self.log_dir = Path(self.log_dir)
        self.log_dir.mkdir(parents=True, exist_ok=True)
        self.path = self.log_dir / self.filename
        if self.path.exists():
            with open(self.path) as f:
                self._lines = sum(1 for _ in f)

    def log(self, metrics: dict[str, float], step: int) -> None:
        if self._lines >= self.max_lines:
            self._warned = True
            return
        rec: dict[str, Any] = {"step": int(step), "timestamp": time.time()}
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                rec[k] = None if (isinstance(v, float) and (math.isnan(v) or math.isinf(v))) else v
            elif hasattr(v, "item"):
                rec[k] = float(v.item())
            else:
                rec[k] = v
        with open(self.path, "a") as f:
            f.write(json.dumps(rec) + "\n")
        self._lines += 1

    def finish(self) -> None:
        pass


@dataclass
class WandbLogger:
    """Weights & Biases sink; importing wandb is deferred and optional."""

    project: str
    name: str | None = None
    config: dict[str, Any] | None = None
    _run: Any = field(default=None, init=False)

    def __post_init__(self) -> None:
        try:
            import wandb  # type: ignore
        except ImportError as e:  # pragma: no cover - optional dependency
            raise ImportError("WandbLogger needs the wandb package") from e
        self._run = wandb.init(project=self.project, name=self.name, config=self.config)

    def log(self, metrics: dict[str, float], step: int) -> None:
        self._run.log(metrics, step=step)

    def finish(self) -> None:
        self._run.finish()


@dataclass
class CompositeLogger:
    loggers: list[MetricsLogger]

    def log(self, metrics: dict[str, float], step: int) -> None:
        for lg in self.loggers:
            lg.log(metrics, step)

    def finish(self) -> None:
        for lg in self.loggers:
            lg.finish()


def compute_stats_from_jsonl(path: Path | str, keys: list[str] | None = None) -> dict[str, dict[str, float]]:
    """min / max / mean / last of every numeric key in a metrics file."""
    vals: dict[str, list[float]] = {}
    with open(path) as f:
        for line in f:
            rec = json.loads(line)
            for k, v in rec.items():
                if k in ("step", "timestamp") or not isinstance(v, (int, float)):
                    continue
                if keys is None or k in keys:
                    vals.setdefault(k, []).append(float(v))
    return {k: {"min": min(v), "max": max(v), "mean": sum(v) / len(v), "last": v[-1], "count": float(len(v))}
            for k, v in vals.items()}
