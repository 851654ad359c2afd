"""Failure detection of the lock-step loop, made on the host: rank 1 leaves between steps (no kernel or collective
in flight); rank 0's next per-step agreement must raise PeerFailure within the group's timeout instead of hanging."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from research_b200.parallel import ExpertParallel, PeerFailure  # noqa: E402
from research_b200.parallel.symm import PeerComm  # noqa: E402

dist.init_process_group("gloo")
rank = dist.get_rank()
ep = ExpertParallel(PeerComm(device=torch.device("cpu")), timeout_s=6.0)
for step in range(3):
    assert ep.agree(rank == 0, step, 1) == (1, step, 1)
if rank == 1:
    print("RANK1_LEAVING", flush=True)
    os._exit(0)            # between steps, without saying goodbye
t0 = time.time()
try:
    ep.agree(1, 0, 1)
    print("NO_FAILURE_SEEN", flush=True)
except PeerFailure as e:
    print(f"PEER_FAILURE_DETECTED after {time.time() - t0:.1f}s: {str(e)[:80]}", flush=True)
os._exit(0)
