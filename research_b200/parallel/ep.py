"""Expert-parallel serving context: data-parallel attention, expert-parallel MoE, engines in lock step.

Every rank runs a whole engine of its own (scheduler, KV cache, attention and dense weights) on its own
requests; only the experts are split over the ranks. The MoE layers' dispatch and combine are collectives
(peer stores plus device barriers, ``parallel/moe.py``), so every rank has to run the same number of MoE
forwards in the same order. ``agree`` is the control plane for that: before each step the ranks exchange what
they are about to run (the maximum of a few flags: on GPUs one small kernel that stores the values into every peer's
memory, waits for the peers' flags and reduces, `PeerComm.agree_max`; on CPU groups a gloo all-reduce) and a rank with
nothing of its own runs an idle pass, which feeds the MoE layers a padding batch.

The reference serves MoE models through external engines only (rollouts/inference/backends.py:1-60 starts
SGLang / vLLM servers); this is the in-tree equivalent of their ``--dp --enable-dp-attention --ep`` mode.
"""

from __future__ import annotations

from datetime import timedelta

import torch
import torch.distributed as dist

from .symm import PeerComm


class PeerFailure(RuntimeError):
    """A rank of the expert-parallel group did not answer the per-step agreement in time (it exited, hung or lost
    its connection). Raised on the host before anything is launched for the step, so no kernel is left waiting on
    the missing rank's barriers."""


class ExpertParallel:
    def __init__(self, comm: PeerComm, cpu_group=None, timeout_s: float = 120.0):
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        self.timeout_s = timeout_s
        # GPUs exchange the flags through peer memory; the host-side group is only for ranks without one
        self.device_agree = bool(comm.on_gpu) and self.world > 1
        if cpu_group is None and self.world > 1 and not self.device_agree:
            # agreement travels over a host-side group of its own: it never queues behind device work, and its
            # timeout doubles as the failure detector of the lock-step loop
            cpu_group = dist.new_group(backend="gloo", timeout=timedelta(seconds=timeout_s))
        self.cpu_group = cpu_group
        self._buf = torch.zeros(4, dtype=torch.int32)
        self.agreements = 0

    def agree(self, *flags: int) -> tuple[int, ...]:
        """Element-wise maximum of up to four small integers over the ranks."""
        assert len(flags) <= 4
        if self.world == 1:
            return tuple(int(f) for f in flags)
        if self.device_agree:
            # the wait inside the kernel is bounded by the same timeout the host-side group would use; a peer that
            # stays silent that long is reported before anything else is launched for the step
            got = self.comm.agree_max(flags, budget_s=self.timeout_s)
            if got is None:
                raise PeerFailure(f"rank {self.rank}: expert-parallel agreement failed after {self.agreements} steps: "
                                  f"a peer did not answer within {self.timeout_s:.0f} s")
            self.agreements += 1
            return got
        self._buf.zero_()
        for i, f in enumerate(flags):
            self._buf[i] = int(f)
        try:
            dist.all_reduce(self._buf, op=dist.ReduceOp.MAX, group=self.cpu_group)
        except Exception as e:  # noqa: BLE001 - gloo reports a lost or silent peer as a RuntimeError / timeout
            raise PeerFailure(f"rank {self.rank}: expert-parallel agreement failed after {self.agreements} steps: {e}") from e
        self.agreements += 1
        return tuple(int(v) for v in self._buf[:len(flags)])
