"""Prompt iteration for rollouts: immutable ``BufferState`` + pure ``get_samples``.

Contract of the reference (rollouts/training/datasets/data_buffer.py:23-500): deterministic
per-epoch shuffle from ``(seed, epoch)``, wrap-around that bumps ``epoch_id``, GRPO grouping
(``n_samples_per_prompt`` copies that share ``group_index``), loaders for lists, JSONL, parquet
and HF datasets, and the mutable ``DataBuffer`` convenience wrapper with ``save_state`` /
``load_state``.
"""

from __future__ import annotations

import json
import random
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Any, Callable

from ..types import Sample


@dataclass(frozen=True)
class BufferState:
    epoch_id: int = 0
    sample_offset: int = 0
    seed: int = 42


def _shuffle_for_epoch(samples: list[Sample], seed: int, epoch_id: int) -> list[Sample]:
    order = list(range(len(samples)))
    random.Random(seed * 1_000_003 + epoch_id).shuffle(order)
    return [samples[i] for i in order]


def get_samples(samples: list[Sample], state: BufferState, n: int, n_samples_per_prompt: int = 1
                ) -> tuple[list[list[Sample]], BufferState]:
    """Next ``n`` prompts, each repeated ``n_samples_per_prompt`` times; returns the new state."""
    assert n > 0 and len(samples) > 0 and n_samples_per_prompt >= 1
    shuffled = _shuffle_for_epoch(samples, state.seed, state.epoch_id)
    epoch, off = state.epoch_id, state.sample_offset
    global_index = epoch * len(samples) + off
    groups: list[list[Sample]] = []
    while len(groups) < n:
        if off >= len(shuffled):
            epoch, off = epoch + 1, 0
            shuffled = _shuffle_for_epoch(samples, state.seed, epoch)
        base = shuffled[off]
        group = []
        for i in range(n_samples_per_prompt):
            group.append(replace(base, tokens=list(base.tokens), loss_mask=list(base.loss_mask),
                                 metadata=dict(base.metadata), input=dict(base.input), group_index=len(groups),
                                 index=global_index * n_samples_per_prompt + i))
        groups.append(group)
        off += 1
        global_index += 1
    return groups, BufferState(epoch_id=epoch, sample_offset=off, seed=state.seed)


def get_samples_flat(samples: list[Sample], state: BufferState, n: int, n_samples_per_prompt: int = 1
                     ) -> tuple[list[Sample], BufferState]:
    groups, new_state = get_samples(samples, state, n, n_samples_per_prompt)
    return [s for g in groups for s in g], new_state


def state_to_dict(state: BufferState) -> dict[str, Any]:
    return {"epoch_id": state.epoch_id, "sample_offset": state.sample_offset, "seed": state.seed}


def state_from_dict(data: dict[str, Any]) -> BufferState:
    return BufferState(epoch_id=int(data.get("epoch_id", 0)), sample_offset=int(data.get("sample_offset", 0)),
                       seed=int(data.get("seed", 42)))


# ------------------------------------------------------------------------------------ loaders
def _to_sample(row: dict[str, Any], prompt_key: str, answer_key: str | None, idx: int,
               transform: Callable[[dict], dict] | None = None) -> Sample:
    if transform is not None:
        row = transform(row)
    meta = {k: v for k, v in row.items() if k not in (prompt_key, answer_key)}
    return Sample(id=str(row.get("id", idx)), index=idx, prompt=row[prompt_key],
                  ground_truth=row.get(answer_key) if answer_key else None, input=dict(row), metadata=meta)


def load_samples_from_list(prompts: list[Any], ground_truths: list[Any] | None = None) -> list[Sample]:
    out = []
    for i, p in enumerate(prompts):
        if isinstance(p, Sample):
            out.append(p)
        elif isinstance(p, dict) and "prompt" in p:
            out.append(_to_sample(p, "prompt", "answer" if "answer" in p else None, i))
        else:
            out.append(Sample(id=str(i), index=i, prompt=p, ground_truth=ground_truths[i] if ground_truths else None))
    return out


def load_samples_from_jsonl(path: str | Path, prompt_key: str = "prompt", answer_key: str | None = "answer",
                            limit: int | None = None, transform=None) -> list[Sample]:
    out = []
    with open(path) as f:
        for i, line in enumerate(f):
            if limit is not None and i >= limit:
                break
            line = line.strip()
            if line:
                out.append(_to_sample(json.loads(line), prompt_key, answer_key, i, transform))
    return out


def load_samples_from_parquet(path: str | Path, prompt_key: str = "prompt", answer_key: str | None = "answer",
                              limit: int | None = None, transform=None) -> list[Sample]:
    import pandas as pd

    df = pd.read_parquet(path)
    if limit is not None:
        df = df.head(limit)
    return [_to_sample(r, prompt_key, answer_key, i, transform) for i, r in enumerate(df.to_dict("records"))]


def load_samples_from_hf(name: str, split: str = "train", prompt_key: str = "question", answer_key: str | None = "answer",
                         limit: int | None = None, transform=None, **kwargs) -> list[Sample]:
    try:
        from datasets import load_dataset  # type: ignore
    except ImportError as e:
        raise ImportError("load_samples_from_hf needs the `datasets` package") from e
    ds = load_dataset(name, split=split, **kwargs)
    if limit is not None:
        ds = ds.select(range(min(limit, len(ds))))
    return [_to_sample(dict(r), prompt_key, answer_key, i, transform) for i, r in enumerate(ds)]


@dataclass
class DataBuffer:
    """Mutable convenience wrapper: keeps the state and hands out prompts."""

    prompts: list[Any]
    seed: int = 42
    ground_truths: list[Any] | None = None

    def __post_init__(self) -> None:
        assert len(self.prompts) > 0, "DataBuffer needs at least one prompt"
        self._samples = load_samples_from_list(self.prompts, self.ground_truths)
        self._state = BufferState(seed=self.seed)

    @property
    def state(self) -> BufferState:
        return self._state

    def get_prompts(self, n: int) -> list[Any]:
        groups, self._state = get_samples(self._samples, self._state, n, 1)
        return [g[0].prompt for g in groups]

    def get_sample_groups(self, n: int, n_samples_per_prompt: int = 1) -> list[list[Sample]]:
        groups, self._state = get_samples(self._samples, self._state, n, n_samples_per_prompt)
        return groups

    def save_state(self) -> dict[str, Any]:
        return state_to_dict(self._state)

    def load_state(self, state: dict[str, Any]) -> None:
        self._state = state_from_dict(state)
