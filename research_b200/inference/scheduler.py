"""Continuous-batching policy as a pure function (rollouts/inference/scheduler.py:15-108).

Decode running sequences first (preempting the overflow beyond ``max_batch_size``), then admit
waiting sequences while the batch-size, token-budget and free-block limits hold. The engine
runs the C++ twin of this policy (csrc/engine_core.cpp); ``schedule_native`` exposes that twin
over plain arrays so tests can check both give the same answer.
"""

from __future__ import annotations

import ctypes

from .. import _native
from .types import SchedulerConfig, SchedulerOutput, Sequence, SequenceStatus


def schedule(waiting: list[Sequence], running: list[Sequence], num_free_blocks: int, config: SchedulerConfig) -> SchedulerOutput:
    assert config.max_batch_size > 0 and config.block_size > 0
    prefill: list[int] = []
    decode: list[int] = []
    preempted: list[int] = []
    blocks = num_free_blocks
    tokens = 0
    for seq in running:
        assert seq.status == SequenceStatus.RUNNING, f"expected RUNNING, got {seq.status}"
        if len(decode) >= config.max_batch_size:
            preempted.append(seq.seq_id)
            continue
        decode.append(seq.seq_id)
        tokens += 1
    for seq in waiting:
        assert seq.status == SequenceStatus.WAITING, f"expected WAITING, got {seq.status}"
        if len(prefill) + len(decode) >= config.max_batch_size:
            break
        n = len(seq.token_ids)
        if tokens + n > config.max_tokens_per_batch:
            break
        need = config.blocks_for(n)
        if need > blocks:
            break
        prefill.append(seq.seq_id)
        blocks -= need
        tokens += n
    return SchedulerOutput(tuple(prefill), tuple(decode), tuple(preempted))


def can_schedule_any(waiting: list[Sequence], running: list[Sequence], num_free_blocks: int, config: SchedulerConfig) -> bool:
    if running:
        return True
    if not waiting:
        return False
    return config.blocks_for(len(waiting[0].token_ids)) <= num_free_blocks


def schedule_native(waiting: list[Sequence], running: list[Sequence], num_free_blocks: int, config: SchedulerConfig) -> SchedulerOutput:
    """Same policy evaluated by the C++ engine core."""
    lib = _native.load("rb_engine_core")
    LL, I = ctypes.c_longlong, ctypes.c_int
    nr, nw = len(running), len(waiting)
    r_ids = (LL * max(nr, 1))(*[s.seq_id for s in running])
    w_ids = (LL * max(nw, 1))(*[s.seq_id for s in waiting])
    w_len = (I * max(nw, 1))(*[len(s.token_ids) for s in waiting])
    pre, dec, pmt = (LL * max(nw, 1))(), (LL * max(nr, 1))(), (LL * max(nr, 1))()
    counts = (I * 3)()
    lib.rb_schedule_pure(r_ids, nr, w_ids, w_len, nw, num_free_blocks, config.max_batch_size,
                         config.max_tokens_per_batch, config.block_size, pre, dec, pmt, counts)
    return SchedulerOutput(tuple(pre[: counts[0]]), tuple(dec[: counts[1]]), tuple(pmt[: counts[2]]))
