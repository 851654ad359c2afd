"""miniray: fork workers, line protocol, failure detection on the host, TCP server, NCCL env."""

import os
import socket
import sys
import threading
import time

import pytest

from research_b200.miniray import (Cluster, NCCLConfig, NodeConfig, RemoteWorker, SharedMemory, Worker, WorkerServer,
                                   create_nccl_configs, restore_nccl_env, set_gpu_affinity, setup_nccl_env,
                                   shutdown_workers, wait_any)
from research_b200.miniray.worker import decode_message, encode_message


def echo_fn(handle):
    while True:
        msg = handle.recv()
        if msg.get("cmd") == "shutdown":
            return
        handle.send({"echo": msg, "pid": os.getpid(), "env": os.environ.get("MINIRAY_TEST")})


def crash_fn(handle):
    handle.recv()
    raise RuntimeError("injected failure")


def test_message_codecs():
    m = {"a": [1, 2.5, "x"], "b": {"c": None}}
    assert decode_message(encode_message(m)) == m
    assert decode_message(encode_message(m, binary=True)) == m


def test_worker_roundtrip_wait_any_and_shutdown():
    ws = [Worker(echo_fn, env={"MINIRAY_TEST": str(i)}) for i in range(3)]
    for i, w in enumerate(ws):
        w.send({"i": i}, binary=(i == 1))
    got = {}
    deadline = time.time() + 10
    while len(got) < 3 and time.time() < deadline:
        for w in wait_any(ws, timeout=1.0):
            r = w.recv()
            got[r["echo"]["i"]] = r
    assert sorted(got) == [0, 1, 2] and got[2]["env"] == "2" and got[0]["pid"] != os.getpid()
    assert all(w.is_alive() for w in ws)
    shutdown_workers(ws)
    assert not any(w.is_alive() for w in ws)


def test_worker_failure_is_detected_on_the_host():
    w = Worker(crash_fn)
    w.send({"go": 1})
    msg = w.recv(timeout=10)
    assert "injected failure" in msg["error"]
    with pytest.raises(RuntimeError):
        w.wait(timeout=10)
    assert not w.is_alive()
    with pytest.raises((EOFError, TimeoutError, OSError)):
        w.recv(timeout=0.5)


def test_shared_memory():
    shm = SharedMemory.create(4096)
    shm.buf[:5] = b"hello"
    other = SharedMemory.map(os.dup(shm.fd), 4096)
    assert bytes(other.buf[:5]) == b"hello"
    other.close()
    shm.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_worker_server_and_remote_worker_health_check():
    port = _free_port()
    srv = WorkerServer(port, echo_fn, host="127.0.0.1")
    t = threading.Thread(target=srv.serve_forever, kwargs={"max_connections": 1}, daemon=True)
    # signal handlers can only be installed from the main thread: run the accept loop without them
    import signal as _signal
    orig = _signal.signal
    _signal.signal = lambda *a, **k: None
    try:
        t.start()
        time.sleep(0.3)
    finally:
        _signal.signal = orig
    rw = None
    for _ in range(40):
        try:
            rw = RemoteWorker("127.0.0.1", port).connect()
            break
        except OSError:
            time.sleep(0.1)
    assert rw is not None
    assert rw.health_check(timeout=5)
    rw.send({"x": 1})
    assert rw.recv(timeout=5)["echo"] == {"x": 1}
    rw.send({"cmd": "shutdown"})
    rw.close()
    t.join(timeout=10)
    dead = RemoteWorker("127.0.0.1", _free_port())
    assert not dead.health_check()


def test_nccl_env_and_cluster_commands():
    cfgs = create_nccl_configs("10.0.0.1", 29500, [2, 2])
    assert [c.rank for c in cfgs] == [0, 1, 2, 3] and [c.local_rank for c in cfgs] == [0, 1, 0, 1]
    old = setup_nccl_env(cfgs[3])
    assert os.environ["RANK"] == "3" and os.environ["WORLD_SIZE"] == "4" and os.environ["NCCL_NVLS_ENABLE"] == "0"
    restore_nccl_env(old)
    assert os.environ.get("RANK") == old["RANK"]
    assert NCCLConfig.from_dict(cfgs[0].to_dict()) == cfgs[0]
    cl = Cluster([NodeConfig("localhost", 2, 10001), NodeConfig("gpu-b", 2, 10001, ssh_user="me", workdir="/w")])
    assert cl.server_command(cl.nodes[0], "m:f")[0] == sys.executable
    remote = cl.server_command(cl.nodes[1], "m:f")
    assert remote[0] == "ssh" and "me@gpu-b" in remote and "cd /w" in remote[-1]
    assert [c.world_size for c in cl.nccl_configs()] == [4] * 4


def test_gpu_affinity_with_fake_nvml():
    class FakeNVML:
        def nvmlInit(self): pass
        def nvmlShutdown(self): pass
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetCpuAffinity(self, h, n): return [0b11] + [0] * (n - 1)

    before = os.sched_getaffinity(0)
    try:
        cpus = set_gpu_affinity(0, nvml=FakeNVML())
        assert cpus == [0, 1] or cpus == [0]
    finally:
        os.sched_setaffinity(0, before)
    assert set_gpu_affinity(0, nvml=None) is None or isinstance(set_gpu_affinity(0), list)
