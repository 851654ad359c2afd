"""Asyncio front of an in-process engine: concurrent coroutines share the engine's batches.

``InferenceEngine.generate`` blocks until its own requests finish, so N agent loops that each call it take N
turns at batch size one. ``AsyncEngineBatcher.generate`` instead queues the request, hands control back to the
event loop, and a single driver task steps the engine for everybody: requests submitted by different coroutines
between two steps run in the same continuous batch. Single-threaded (the engine is only touched from the event
loop), so no locking is needed.

The reference reaches the same effect through its HTTP servers, which batch concurrent requests
(rollouts/providers/sglang.py, rollouts/training/agent_integration.py:193-272 runs the agents under one nursery).
"""

from __future__ import annotations

import asyncio

from .types import SamplingParams, TrainingSample


class AsyncEngineBatcher:
    def __init__(self, engine):
        self.engine = engine
        self._futures: dict[int, asyncio.Future] = {}
        self._task: asyncio.Task | None = None
        self.steps = 0
        self.max_rows = 0          # largest number of rows any step ran (prefill + decode)

    async def generate(self, prompt_tokens: list[int], params: SamplingParams) -> TrainingSample:
        loop = asyncio.get_running_loop()
        sid = self.engine.add_request(list(prompt_tokens), params)
        fut: asyncio.Future = loop.create_future()
        self._futures[sid] = fut
        if self._task is None or self._task.done():
            self._task = loop.create_task(self._drive())
        return await fut

    async def _drive(self) -> None:
        try:
            while self._futures:
                await asyncio.sleep(0)      # every coroutine that is ready to submit does so before the next step
                for sid, sample in self.engine._step_with_ids():
                    fut = self._futures.pop(sid, None)
                    if fut is not None and not fut.done():
                        fut.set_result(sample)
                self.steps += 1
                self.max_rows = max(self.max_rows, sum(self.engine.last_step_rows))
                if not self.engine.has_pending() and self._futures:   # requests vanished (aborted): do not spin
                    for fut in self._futures.values():
                        if not fut.done():
                            fut.set_exception(RuntimeError("request left the engine without a result"))
                    self._futures.clear()
        except Exception as e:  # noqa: BLE001 - hand the failure to every waiter
            for fut in self._futures.values():
                if not fut.done():
                    fut.set_exception(e)
            self._futures.clear()


def batcher_for(engine) -> AsyncEngineBatcher:
    """The engine's batcher (one per engine, created on first use)."""
    b = getattr(engine, "_async_batcher", None)
    if b is None:
        b = AsyncEngineBatcher(engine)
        engine._async_batcher = b
    return b
