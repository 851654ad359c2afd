"""Symmetric peer memory and flag-based synchronisation between the GPUs of one node.

``PeerComm`` is the transport layer under every fused compute+collective kernel: it allocates
buffers that every rank maps into its own address space (``torch.distributed._symmetric_memory``
does the CUDA VMM allocation and the handle exchange; NVLS multicast binding is switched off so
kernels only use plain peer loads/stores), and it owns the flag words used for barriers and
ready signals. Flag values are monotonically increasing epochs, so nothing is ever reset.

On CPU (gloo ranks, used by the tests) the same object degrades to ordinary collectives so the
host-side logic of the training backend and weight sync runs without a GPU.

The reference has no equivalent: its communication is ``torch.distributed`` NCCL calls only
(rollouts/training/distributed_utils.py:37-360).
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native
from ..ops._util import check_rc, status_tensor, stream_handle

MAX_RANKS = 8
_VP, _I, _LL, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _lib():
    lib = _native.load("rb_comm")
    if not getattr(lib, "_rb_typed", False):
        PP = ctypes.POINTER(_VP)
        lib.rb_symm_barrier.argtypes = [PP, _I, _I, _I, _I, _VP, _VP, _VP]
        lib.rb_symm_signal.argtypes = [PP, _I, _I, _I, _I, _VP]
        lib.rb_symm_wait.argtypes = [_VP, _I, _I, _I, _VP, _VP]
        lib.rb_rs_reduce.argtypes = [PP, _VP, _I, _I, _I, _I, _LL, _F, _VP, _I, _VP, _VP, _VP]
        lib.rb_clip_coef.argtypes = [_VP, _I, PP, PP, _I, _I, _I, _I, _F, _VP, _VP, _VP, _VP]
        lib.rb_adamw_allgather.argtypes = [_VP, _VP, _VP, _VP, PP, _I, _I, _LL, _F, _F, _F, _F, _F, _I, _VP, _VP]
        lib.rb_reshard_copy.argtypes = [_VP, _I, _LL, _VP]
        lib.rb_pull_sum.argtypes = [PP, _VP, _VP, _LL, _I, _VP]
        lib.rb_symm_wait_budget.argtypes = [_VP, _I, _I, _I, _VP, ctypes.c_ulonglong, _VP]
        lib.rb_symm_signal_counter.argtypes = [PP, _I, _I, _I, _VP, _VP]
        lib.rb_symm_signal_counter.restype = _I
        lib.rb_rs_reduce_ex.argtypes = [PP, _VP, _I, _I, _I, _I, _LL, _F, _VP, _I, _VP, _VP, _I, _VP]
        lib.rb_clip_coef_ex.argtypes = [_VP, _I, PP, PP, _I, _I, _I, _I, _F, _F, _VP, _VP, _VP, _VP]
        lib.rb_adamw_allgather_ex.argtypes = [_VP, _VP, _VP, _VP, _I, PP, _I, _I, _LL, _F, _F, _F, _F, _F, _I, _VP, _VP]
        lib.rb_pull_sum_sync.argtypes = [PP, _VP, _VP, _LL, _I, _I, PP, _I, _VP, PP, _VP, _VP, _VP]
        lib.rb_pull_sum_sync.restype = _I
        lib.rb_symm_agree_max.argtypes = [PP, PP, _I, _I, _I, _VP, _I, _I, _I, _I, _VP, ctypes.c_ulonglong, _VP]
        lib.rb_symm_agree_max.restype = _I
        lib.rb_comm_set_wait_budget_ns.argtypes = [ctypes.c_ulonglong]
        lib.rb_comm_set_wait_budget_ns.restype = None
        lib.rb_comm_get_wait_budget_ns.restype = ctypes.c_ulonglong
        lib.rb_pull_sum.restype = _I
        lib.rb_rs_num_partials.restype = _I
        for f in ("rb_symm_barrier", "rb_symm_signal", "rb_symm_wait", "rb_rs_reduce", "rb_clip_coef",
                  "rb_adamw_allgather", "rb_reshard_copy", "rb_symm_wait_budget", "rb_rs_reduce_ex", "rb_clip_coef_ex",
                  "rb_adamw_allgather_ex"):
            getattr(lib, f).restype = _I
        lib._rb_typed = True
    return lib


def ptr_array(ptrs: list[int]):
    arr = (_VP * MAX_RANKS)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class SymmBuffer:
    """A tensor allocated at the same offset on every rank, with every peer's address known."""

    def __init__(self, local: torch.Tensor, peer_ptrs: list[int], handle=None):
        self.local = local
        self.peer_ptrs = peer_ptrs
        self.handle = handle

    def ptrs(self, byte_offset: int = 0):
        return ptr_array([p + byte_offset for p in self.peer_ptrs])

    def peer_tensor(self, rank: int) -> torch.Tensor:
        """View of rank ``rank``'s buffer in this process (CUDA only)."""
        assert self.handle is not None
        return self.handle.get_buffer(rank, self.local.shape, self.local.dtype)


class PeerComm:
    """Peer-memory context of one process group (one rank per GPU, single node)."""

    NUM_SLOTS = 512     # one ready-flag row per gradient chunk (a layer) plus barriers and the norm exchange

    def __init__(self, group: dist.ProcessGroup | None = None, device: torch.device | None = None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        assert self.world <= MAX_RANKS
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        self.on_gpu = self.device.type == "cuda"
        self._epochs = [0] * self.NUM_SLOTS
        self._next_slot = 1  # slot 0 is the generic barrier
        if self.on_gpu:
            # plain peer loads/stores only: never bind these buffers to an NVLink multicast object
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            self.flags = self.alloc((self.NUM_SLOTS, self.world), torch.int32, zero=True)
            self.norm_slots = self.alloc((self.world,), torch.float32, zero=True)
            # barrier epochs are counted on the device so captured barriers replay correctly
            self.barrier_counters = torch.zeros(self.NUM_SLOTS, dtype=torch.int32, device=self.device)
            self.barrier_host()
        else:
            self.flags = None
            self.norm_slots = None

    # ---------------------------------------------------------------- allocation
    def alloc(self, shape, dtype=torch.bfloat16, zero: bool = False) -> SymmBuffer:
        if not self.on_gpu:
            t = torch.zeros(shape, dtype=dtype)
            return SymmBuffer(t, [t.data_ptr()] * self.world)
        import torch.distributed._symmetric_memory as symm_mem

        t = symm_mem.empty(*shape, dtype=dtype, device=self.device)
        hdl = symm_mem.rendezvous(t, self.group)
        if zero:
            t.zero_()
        return SymmBuffer(t, [int(p) for p in hdl.buffer_ptrs], hdl)

    def new_slot(self) -> int:
        s = self._next_slot
        assert s < self.NUM_SLOTS, "out of flag slots"
        self._next_slot += 1
        return s

    def next_epoch(self, slot: int) -> int:
        self._epochs[slot] += 1
        return self._epochs[slot]

    # ---------------------------------------------------------------- synchronisation
    def barrier_host(self) -> None:
        """Host-level barrier (process group) plus device synchronise; used at set-up only."""
        if self.on_gpu:
            torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def barrier(self, slot: int = 0) -> None:
        """Device-side barrier on the current stream: every rank signals every peer, then waits."""
        if not self.on_gpu:
            dist.barrier(self.group)
            return
        rc = _lib().rb_symm_barrier(self.flags.ptrs(), self.rank, self.world, slot, 0,
                                    self.barrier_counters.data_ptr() + 4 * slot,
                                    status_tensor(self.device).data_ptr(), stream_handle(self.device))
        check_rc(rc, "rb_symm_barrier")

    def signal(self, slot: int) -> int:
        """Publish "my data for this slot is ready" to every peer; returns the epoch signalled."""
        ep = self.next_epoch(slot)
        if self.on_gpu:
            rc = _lib().rb_symm_signal(self.flags.ptrs(), self.rank, self.world, slot, ep, stream_handle(self.device))
            check_rc(rc, "rb_symm_signal")
        else:
            dist.barrier(self.group)
        return ep

    def wait(self, slot: int, epoch: int) -> None:
        """Wait (bounded, on the stream) until every peer signalled ``epoch`` on ``slot``."""
        if self.on_gpu:
            rc = _lib().rb_symm_wait(self.flags.local.data_ptr(), self.world, slot, epoch,
                                     status_tensor(self.device).data_ptr(), stream_handle(self.device))
            check_rc(rc, "rb_symm_wait")

    def flag_ptr(self, slot: int) -> int:
        """Address of this rank's flag row ``[world]`` for ``slot``."""
        return self.flags.local.data_ptr() + slot * self.world * 4

    def agree_max(self, values, budget_s: float = 0.0) -> tuple[int, ...] | None:
        """Element-wise maximum of up to four small integers over the ranks, exchanged through peer memory by one
        small kernel (values stored into every peer's buffer, flags, bounded wait) and read back by the host. Returns
        None when a peer did not answer within ``budget_s`` (0 = the library's wait budget): nothing else was
        launched, the GPU and the context stay usable."""
        vals = [int(v) for v in values] + [0] * (4 - len(values))
        assert len(vals) == 4 and self.on_gpu
        if getattr(self, "_agree", None) is None:
            xchg = self.alloc((2, self.world, 4), torch.int32, zero=True)
            self._agree = (xchg, self.new_slot(), torch.zeros(1, dtype=torch.int32, device=self.device),
                           torch.zeros(5, dtype=torch.int32, device=self.device))
            self.barrier_host()
        xchg, slot, counter, out = self._agree
        rc = _lib().rb_symm_agree_max(xchg.ptrs(), self.flags.ptrs(), self.rank, self.world, slot, counter.data_ptr(),
                                      vals[0], vals[1], vals[2], vals[3], out.data_ptr(), int(budget_s * 1e9), stream_handle(self.device))
        check_rc(rc, "rb_symm_agree_max")
        host = out.tolist()            # the one synchronisation of the exchange
        if not host[4]:
            return None
        return tuple(host[:len(values)])


class LayoutComm:
    """Stand-in for a training group's ``PeerComm`` on a rank that is NOT in that group (an inference engine on its own
    GPU): it only says how many training ranks there are, which is all a parameter layout depends on. Nothing can be
    allocated or synchronised through it."""

    def __init__(self, world: int, device: torch.device):
        self.rank, self.world, self.device, self.group = 0, world, device, None
        self.on_gpu = device.type == "cuda"

    def alloc(self, *a, **kw):
        raise RuntimeError("a layout-only communicator allocates nothing")


class LocalComm(PeerComm):
    """Single-process, single-rank stand-in: the same kernels run with this GPU as its only peer."""

    def __init__(self, device: torch.device | None = None):  # noqa: D107 - no process group involved
        self.group = None
        self.rank, self.world = 0, 1
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        self.on_gpu = self.device.type == "cuda"
        self._epochs = [0] * self.NUM_SLOTS
        self._next_slot = 1
        if self.on_gpu:
            self.flags = self.alloc((self.NUM_SLOTS, 1), torch.int32, zero=True)
            self.norm_slots = self.alloc((1,), torch.float32, zero=True)
            self.barrier_counters = torch.zeros(self.NUM_SLOTS, dtype=torch.int32, device=self.device)
        else:
            self.flags = self.norm_slots = None

    def alloc(self, shape, dtype=torch.bfloat16, zero: bool = False) -> SymmBuffer:
        t = torch.zeros(shape, dtype=dtype, device=self.device)
        return SymmBuffer(t, [t.data_ptr()])

    def barrier_host(self) -> None:
        if self.on_gpu:
            torch.cuda.synchronize(self.device)

    def barrier(self, slot: int = 0) -> None:
        if self.on_gpu:
            super().barrier(slot)

    def signal(self, slot: int) -> int:
        ep = self.next_epoch(slot)
        if self.on_gpu:
            rc = _lib().rb_symm_signal(self.flags.ptrs(), 0, 1, slot, ep, stream_handle(self.device))
            check_rc(rc, "rb_symm_signal")
        return ep
