"""Multi-rank tests: gloo CPU ranks everywhere; the same worker on real GPUs when >= 2 are visible.

GPU runs use plain peer loads/stores only (no NVLS) and leave between steps, never mid-kernel.
"""

import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(device: str, nproc: int, cases: str, timeout: int = 600) -> str:
    # a rank that is still running 90 s before the limit prints every thread's stack and exits: a host-side deadlock
    # then fails with the place it waited at instead of a bare timeout
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1", OMP_NUM_THREADS="2",
               RB_TEST_DUMP_AFTER=str(max(timeout - 90, 30)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(HERE, "multi_rank_worker.py"), device, cases]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    for _ in range(2):
        # the port picked above was free when probed; another process may have taken it since: pick again
        if proc.returncode == 0 or "EADDRINUSE" not in proc.stderr:
            break
        cmd[cmd.index("--master-port") + 1] = str(_free_port())
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    return proc.stdout


@pytest.mark.parametrize("cases", ["barrier,tp_gemms,ep_agree", "sharded_adamw", "weight_sync_tp_engine", "fsdp_backend_grpo", "fsdp_full_shard", "ep_training", "grpo_expert_parallel", "grpo_disjoint", "moe_ep", "tp_training"])
def test_gloo_two_ranks(cases):
    out = _run("cpu", 2, cases)
    for c in cases.split(","):
        assert f"CASE_OK {c}" in out


@pytest.mark.parametrize("cases", ["barrier,tp_gemms", "sharded_adamw", "fsdp_full_shard", "ep_training", "grpo_disjoint", "grpo_disjoint_tp_engine", "moe_ep", "tp_training"])
def test_gloo_four_ranks(cases):
    """The host-side logic (slab rotation, shard ranges, count matrices, dispatch offsets) at world size 4."""
    out = _run("cpu", 4, cases)
    for c in cases.split(","):
        assert f"CASE_OK {c}" in out


@pytest.mark.gpu
@pytest.mark.parametrize("cases", ["barrier,tp_gemms,ep_agree", "sharded_adamw", "weight_sync_tp_engine", "fsdp_backend_grpo", "fsdp_full_shard", "ep_training", "grpo_expert_parallel", "grpo_disjoint", "grpo_disjoint_tp_engine", "moe_ep", "tp_training"])
def test_gpu_ranks(cases):
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    out = _run("cuda", 2 if n < 4 or cases in ("weight_sync_tp_engine", "tp_training") else 4, cases)
    for c in cases.split(","):
        assert f"CASE_OK {c}" in out


def test_lockstep_tp_serving_two_ranks():
    """Rank 0 takes requests, rank 1 mirrors its admissions and steps (gloo, CPU)."""
    env = dict(os.environ, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "lockstep_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and "LOCKSTEP_OK" in proc.stdout, proc.stdout[-1500:] + proc.stderr[-3000:]


@pytest.mark.parametrize("ranks", [2, 4])
def test_expert_parallel_engines_lockstep_two_ranks(ranks):
    """Engines with split experts serve different request mixes and stay paired (gloo, CPU)."""
    env = dict(os.environ, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "ep_engine_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and proc.stdout.count("EP_ENGINE_OK") == ranks, proc.stdout[-1500:] + proc.stderr[-3000:]


@pytest.mark.gpu
@pytest.mark.parametrize("flags", [["--cuda"], ["--cuda", "--graphs"]])
def test_expert_parallel_engines_gpu(flags):
    """The same lock-step check with the peer-memory dispatch / combine kernels, eager and inside CUDA graphs."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "ep_engine_worker.py"), *flags]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and proc.stdout.count("EP_ENGINE_OK") == 2, proc.stdout[-1500:] + proc.stderr[-3000:]


def test_expert_parallel_peer_failure_is_detected_on_the_host():
    """A rank that leaves between steps makes the survivor's next agreement raise PeerFailure (gloo, CPU)."""
    env = dict(os.environ, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "ep_failure_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert "RANK1_LEAVING" in proc.stdout and "PEER_FAILURE_DETECTED" in proc.stdout, proc.stdout[-1500:] + proc.stderr[-2000:]
