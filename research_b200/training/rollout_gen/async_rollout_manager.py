"""Asynchronous rollout generation with over-sampling, group filtering, an overflow cache of
surplus samples, abort, and resumable state (rollouts/training/rollout_gen/
async_rollout_manager.py:27-310). Concurrency is ``asyncio`` (the reference uses trio)."""

from __future__ import annotations

import asyncio
import inspect
from dataclasses import dataclass, field
from typing import Any

from ..datasets.data_buffer import DataBuffer
from ..types import RolloutBatch, RolloutConfig, Sample, Status
from .rollout_generation import convert_to_batch


@dataclass
class AsyncRolloutManager:
    data_buffer: DataBuffer
    config: RolloutConfig
    max_concurrency: int = 64
    partial_samples: list[Sample] = field(default_factory=list)   # surplus kept for the next batch
    _abort: bool = field(default=False, init=False)
    _step: int = field(default=0, init=False)

    async def _call_generate(self, prompts: list[Any], **kw) -> list[Sample]:
        fn = self.config.generate_fn
        assert fn is not None, "RolloutConfig.generate_fn is required"
        out = fn(prompts, **kw)
        if inspect.isawaitable(out):
            out = await out
        return list(out)

    @staticmethod
    def _adopt(group: list[Sample], out: list[Sample]) -> list[Sample]:
        """Give every generated sample the group / index / ground truth of the prompt it answers: one per prompt in
        order, or (a generate function that returns several samples per prompt, e.g. one per branch) the prompt named
        by ``metadata["source_prompt"]``."""
        for j, dst in enumerate(out):
            k = dst.metadata.get("source_prompt", j) if isinstance(dst.metadata, dict) else j
            if not 0 <= k < len(group):
                continue
            src = group[k]
            dst.group_index, dst.index = src.group_index, src.index
            if dst.ground_truth is None:
                dst.ground_truth = src.ground_truth
            if dst.status == Status.PENDING:
                dst.status = Status.COMPLETED
        return out

    async def _generate_group(self, group: list[Sample], sem: asyncio.Semaphore, **kw) -> list[Sample]:
        async with sem:
            if self._abort:
                return []
            out = await self._call_generate([s.prompt for s in group], **kw)
        return self._adopt(group, out)

    async def _generate_samples_parallel(self, groups: list[list[Sample]], **kw) -> list[list[Sample]]:
        if getattr(self.config.generate_fn, "batched", False):
            # an in-process engine batches continuously on its own: hand it every prompt of every group in ONE call
            # (one call per group would run the engine at a batch of n_samples_per_prompt, group after group)
            if self._abort:
                return [[] for _ in groups]
            flat = await self._call_generate([s.prompt for g in groups for s in g], **kw)
            out, at = [], 0
            for g in groups:
                out.append(self._adopt(g, flat[at:at + len(g)]))
                at += len(g)
            return out
        sem = asyncio.Semaphore(self.max_concurrency)
        return list(await asyncio.gather(*[self._generate_group(g, sem, **kw) for g in groups]))

    def _score(self, samples: list[Sample], score_fn) -> None:
        fn = score_fn or self.config.score_fn
        if fn is None:
            return
        for s in samples:
            score = fn(s)
            s.score = score
            s.reward = float(getattr(score, "reward", score))

    def _apply_filter(self, groups: list[list[Sample]]) -> list[list[Sample]]:
        if self.config.filter_fn is None:
            return groups
        return [g for g in groups if g and self.config.filter_fn(g)]

    async def generate_batch(self, score_fn=None, **kw) -> RolloutBatch:
        """Collect ``batch_size`` prompt groups that pass the filter (over-sampling as configured)."""
        need = self.config.batch_size
        n_per = self.config.n_samples_per_prompt
        kept: list[list[Sample]] = []
        # surplus from the previous call first
        cached, self.partial_samples = self.partial_samples, []
        by_group: dict[int, list[Sample]] = {}
        for s in cached:
            by_group.setdefault(s.group_index or 0, []).append(s)
        kept.extend(by_group.values())
        rounds = 0
        while len(kept) < need and not self._abort:
            want = max(1, int((need - len(kept)) * self.config.over_sampling_factor + 0.999))
            groups = self.data_buffer.get_sample_groups(want, n_per)
            done = await self._generate_samples_parallel(groups, **kw)
            for g in done:
                self._score(g, score_fn)
            kept.extend(self._apply_filter([g for g in done if g]))
            rounds += 1
            assert rounds < 1000, "filter rejects every group"
        use, extra = kept[:need], kept[need:]
        self.partial_samples = [s for g in extra for s in g]
        samples = []
        for gi, g in enumerate(use):
            for s in g:
                s.group_index = gi
                samples.append(s)
        if self._abort:
            for s in samples:
                s.status = Status.ABORTED
        self._step += 1
        return convert_to_batch(samples, step=self._step, rounds=rounds, cached=len(cached))

    def request_abort(self) -> None:
        self._abort = True

    def state_dict(self) -> dict[str, Any]:
        return {"buffer_state": self.data_buffer.save_state(), "step": self._step,
                "partial_samples": [s.to_dict() for s in self.partial_samples]}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.data_buffer.load_state(state["buffer_state"])
        self._step = int(state.get("step", 0))
        self.partial_samples = [Sample.from_dict(d) for d in state.get("partial_samples", [])]


async def generate_rollout_batch(data_buffer: DataBuffer, config: RolloutConfig, **kw) -> RolloutBatch:
    return await AsyncRolloutManager(data_buffer, config).generate_batch(**kw)
