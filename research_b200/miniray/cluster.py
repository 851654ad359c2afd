"""Multi-node launch: start a worker server per node (ssh), connect to all of them, hand out
NCCL configs (miniray/cluster.py:19-446)."""

from __future__ import annotations

import shlex
import subprocess
import sys
import time
from dataclasses import dataclass, field

from .nccl import NCCLConfig, create_nccl_configs
from .remote_worker import RemoteWorker


@dataclass(frozen=True)
class NodeConfig:
    host: str
    num_workers: int = 1
    port: int = 10000
    ssh_user: str | None = None
    ssh_port: int = 22
    python: str = sys.executable
    workdir: str | None = None

    @property
    def is_local(self) -> bool:
        return self.host in ("localhost", "127.0.0.1")


@dataclass
class Cluster:
    nodes: list[NodeConfig]
    wait_time: float = 2.0
    workers: list[RemoteWorker] = field(default_factory=list)
    _procs: list[subprocess.Popen] = field(default_factory=list)

    def server_command(self, node: NodeConfig, work_fn: str) -> list[str]:
        cmd = [node.python, "-m", "research_b200.miniray.worker_server", "--port", str(node.port), "--workers",
               str(node.num_workers), "--work-fn", work_fn]
        if node.is_local:
            return cmd
        remote = " ".join(shlex.quote(c) for c in cmd)
        if node.workdir:
            remote = f"cd {shlex.quote(node.workdir)} && {remote}"
        target = f"{node.ssh_user}@{node.host}" if node.ssh_user else node.host
        return ["ssh", "-p", str(node.ssh_port), "-o", "StrictHostKeyChecking=no", target, remote]

    def launch_servers(self, work_fn: str) -> None:
        for node in self.nodes:
            self._procs.append(subprocess.Popen(self.server_command(node, work_fn), start_new_session=True,
                                                cwd=node.workdir if node.is_local else None))

    def connect_to_servers(self, retries: int = 20) -> list[RemoteWorker]:
        for node in self.nodes:
            for _ in range(node.num_workers):
                last: Exception | None = None
                for _attempt in range(retries):
                    try:
                        self.workers.append(RemoteWorker(node.host, node.port).connect())
                        last = None
                        break
                    except OSError as e:
                        last = e
                        time.sleep(0.25)
                if last is not None:
                    raise ConnectionError(f"cannot reach worker server {node.host}:{node.port}: {last}")
        return self.workers

    def start(self, work_fn: str) -> list[RemoteWorker]:
        self.launch_servers(work_fn)
        time.sleep(self.wait_time)
        return self.connect_to_servers()

    def nccl_configs(self, master_port: int = 29500) -> list[NCCLConfig]:
        return create_nccl_configs(self.nodes[0].host if not self.nodes[0].is_local else "127.0.0.1", master_port,
                                   [n.num_workers for n in self.nodes])

    def spawn_distributed_workers(self, master_port: int = 29500) -> list[RemoteWorker]:
        """Send every worker its ``init_nccl`` message (rank, world, master address)."""
        for w, cfg in zip(self.workers, self.nccl_configs(master_port)):
            w.send({"cmd": "init_nccl", "config": cfg.to_dict()})
        return self.workers

    def stop(self) -> None:
        for w in self.workers:
            try:
                w.send({"cmd": "shutdown"})
            except (OSError, AssertionError):
                pass
            w.close()
        self.workers.clear()
        for p in self._procs:
            if p.poll() is None:
                p.terminate()  # the server processes this object started
                try:
                    p.wait(timeout=5)
                except subprocess.TimeoutExpired:
                    p.kill()
        self._procs.clear()
