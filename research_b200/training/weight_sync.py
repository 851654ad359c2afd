"""Engine lifecycle and weight-sync entry points with the reference's names
(rollouts/training/weight_sync.py:34-853).

Three families:
* native (the default here): ``NativeEngine`` wraps the in-process ``InferenceEngine``;
  ``sync_weights_to_engines`` pushes the trainer's bucket into every engine with the reshard-copy
  kernel (``research_b200.parallel.weight_sync``).
* HTTP engines kept for interoperability with external servers: ``SGLangEngine`` / ``VLLMEngine``
  speak ``/update_weights_from_disk`` and ``/collective_rpc``; ``update_*_weights_from_disk``
  are the plain functions. They need the ``httpx`` package and a running server; launching one
  (tmux) is supported through ``launch_cmd`` but nothing here ever kills processes on a GPU.
* NCCL broadcast: ``init_nccl_weight_sync`` / ``sync_weights_nccl`` for a trainer that is in a
  process group with external engines (one broadcast per FLAT BUCKET, not per parameter).
"""

from __future__ import annotations

import asyncio
import shutil
import subprocess
import tempfile
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Protocol, runtime_checkable

import torch
import torch.distributed as dist


def get_fast_sync_dir() -> Path:
    """tmpfs directory for checkpoint hand-off (``/dev/shm`` when present)."""
    base = Path("/dev/shm") if Path("/dev/shm").is_dir() else Path(tempfile.gettempdir())
    d = base / "research_b200_weight_sync"
    d.mkdir(parents=True, exist_ok=True)
    return d


async def _post(url: str, payload: dict, timeout: float) -> dict:
    try:
        import httpx
    except ImportError as e:  # pragma: no cover
        raise ImportError("HTTP engines need the httpx package") from e
    async with httpx.AsyncClient(timeout=timeout) as client:
        r = await client.post(url, json=payload)
        r.raise_for_status()
        return r.json() if r.content else {}


async def update_sglang_weights_from_disk(base_url: str, checkpoint_path: str, timeout: float = 300.0) -> dict:
    return await _post(f"{base_url}/update_weights_from_disk", {"model_path": str(checkpoint_path)}, timeout)


async def update_vllm_weights_from_disk(base_url: str, checkpoint_path: str, timeout: float = 300.0) -> dict:
    return await _post(f"{base_url}/collective_rpc", {"method": "reload_weights", "args": [str(checkpoint_path)]}, timeout)


@runtime_checkable
class InferenceEngineHandle(Protocol):
    """Lifecycle surface shared by every engine kind."""

    name: str

    async def launch(self) -> None: ...
    async def wait_until_ready(self, timeout: float = 120.0) -> None: ...
    async def update_weights_from_checkpoint(self, checkpoint_path: str) -> dict: ...
    async def shutdown(self) -> None: ...


@dataclass
class NativeEngine:
    """In-process engine handle: nothing to launch, weights arrive through peer memory."""

    engine: Any
    name: str = "native"
    _plan: Any = None

    async def launch(self) -> None:
        return None

    async def wait_until_ready(self, timeout: float = 120.0) -> None:
        return None

    async def update_weights_from_checkpoint(self, checkpoint_path: str) -> dict:
        from ..models.weights import load_safetensors_dir

        weights, _ = load_safetensors_dir(checkpoint_path)
        self.engine.update_weights(weights)
        return {"success": True, "weight_version": self.engine.get_weight_version()}

    def update_weights_from_buckets(self, buckets, src_rank: int | None = None, comm=None) -> None:
        from ..parallel.weight_sync import sync_engine_from_buckets

        self._plan = sync_engine_from_buckets(self.engine, buckets, self._plan, src_rank, comm)

    async def shutdown(self) -> None:
        self.engine.shutdown()


@dataclass
class _HTTPEngine:
    model_name: str
    port: int = 30000
    host: str = "127.0.0.1"
    cuda_device_ids: tuple[int, ...] = (0,)
    launch_cmd: list[str] | None = None
    log_path: str | None = None
    name: str = "http"
    mem_fraction: float = 0.7
    extra_args: tuple[str, ...] = ()
    forward_log: bool = True              # a daemon thread copies the server's log lines to the Python logger
    _proc: subprocess.Popen | None = field(default=None, init=False)
    _tail: Any = field(default=None, init=False)
    _tail_stop: Any = field(default=None, init=False)

    def default_launch_cmd(self) -> list[str] | None:
        """The server's own command line when none was given (subclasses know theirs)."""
        return None

    def _start_log_tail(self) -> None:
        """Follow ``log_path`` from where it is now and hand every new line to ``logging`` under ``<name>:<port>``, so that
        the server's start-up and error messages appear in the run's own log (rollouts/training/weight_sync.py:523-553)."""
        import logging
        import threading

        if not (self.forward_log and self.log_path):
            return
        log = logging.getLogger(f"{__name__}.{self.name}:{self.port}")
        stop = self._tail_stop = threading.Event()
        path = self.log_path

        def follow() -> None:
            try:
                with open(path, "r", errors="replace") as f:
                    f.seek(0, 2)
                    pending = ""
                    while not stop.is_set():
                        chunk = f.read()
                        if not chunk:
                            stop.wait(0.2)
                            continue
                        pending += chunk
                        *lines, pending = pending.split("\n")
                        for line in lines:
                            if line.strip():
                                log.info(line.rstrip())
            except OSError:
                return

        self._tail = threading.Thread(target=follow, daemon=True, name=f"{self.name}-log-tail")
        self._tail.start()

    def log_tail(self, n: int = 30) -> str:
        if not self.log_path:
            return ""
        try:
            with open(self.log_path, "r", errors="replace") as f:
                return "".join(f.readlines()[-n:])
        except OSError:
            return ""

    @property
    def base_url(self) -> str:
        return f"http://{self.host}:{self.port}"

    async def launch(self) -> None:
        """Start ``launch_cmd`` as a child process (its own process group); no GPU processes are touched."""
        cmd = self.launch_cmd or self.default_launch_cmd()
        if cmd is None:
            return
        import os

        env = dict(os.environ, CUDA_VISIBLE_DEVICES=",".join(map(str, self.cuda_device_ids)))
        if self.log_path:
            os.makedirs(os.path.dirname(os.path.abspath(self.log_path)), exist_ok=True)
        log = open(self.log_path, "ab") if self.log_path else subprocess.DEVNULL
        self._start_log_tail()
        self._proc = subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)

    async def wait_until_ready(self, timeout: float = 120.0) -> None:
        import httpx

        t0 = time.time()
        while time.time() - t0 < timeout:
            if self._proc is not None and self._proc.poll() is not None:
                raise RuntimeError(f"{self.name} server exited with code {self._proc.returncode} during start-up\n--- log tail ---\n{self.log_tail()}")
            try:
                async with httpx.AsyncClient(timeout=2.0) as c:
                    if (await c.get(f"{self.base_url}/health")).status_code == 200:
                        return
            except Exception:
                pass
            await asyncio.sleep(1.0)
        raise TimeoutError(f"{self.name} server not ready after {timeout}s\n--- log tail ---\n{self.log_tail()}")

    async def shutdown(self) -> None:
        if self._tail_stop is not None:
            self._tail_stop.set()
        if self._proc is not None and self._proc.poll() is None:
            self._proc.terminate()  # exactly the child we started
            try:
                self._proc.wait(timeout=10)
            except subprocess.TimeoutExpired:
                self._proc.kill()


@dataclass
class SGLangEngine(_HTTPEngine):
    name: str = "sglang"

    def default_launch_cmd(self) -> list[str]:
        import sys

        cmd = [sys.executable, "-m", "sglang.launch_server", "--model-path", self.model_name, "--host", self.host, "--port", str(self.port),
               "--mem-fraction-static", str(self.mem_fraction), "--trust-remote-code"]
        if len(self.cuda_device_ids) > 1:
            cmd += ["--tp", str(len(self.cuda_device_ids))]
        return cmd + list(self.extra_args)

    async def update_weights_from_checkpoint(self, checkpoint_path: str) -> dict:
        return await update_sglang_weights_from_disk(self.base_url, checkpoint_path)


@dataclass
class VLLMEngine(_HTTPEngine):
    name: str = "vllm"

    def default_launch_cmd(self) -> list[str]:
        import sys

        cmd = [sys.executable, "-m", "vllm.entrypoints.openai.api_server", "--model", self.model_name, "--host", self.host, "--port", str(self.port),
               "--gpu-memory-utilization", str(self.mem_fraction), "--trust-remote-code"]
        if len(self.cuda_device_ids) > 1:
            cmd += ["--tensor-parallel-size", str(len(self.cuda_device_ids))]
        return cmd + list(self.extra_args)

    async def update_weights_from_checkpoint(self, checkpoint_path: str) -> dict:
        return await update_vllm_weights_from_disk(self.base_url, checkpoint_path)


async def sync_weights_to_engines(engines: list[Any], checkpoint_path: str | None = None, buckets=None,
                                  src_rank: int | None = None, comm=None) -> list[dict]:
    """Update every engine: native engines from ``buckets`` (kernel path), HTTP engines from ``checkpoint_path``."""
    results = []
    http = []
    for e in engines:
        if isinstance(e, NativeEngine) and buckets is not None:
            e.update_weights_from_buckets(buckets, src_rank, comm)
            results.append({"engine": e.name, "success": True})
        else:
            assert checkpoint_path is not None, "HTTP engines need a checkpoint path"
            http.append(e)
    if http:
        outs = await asyncio.gather(*[e.update_weights_from_checkpoint(checkpoint_path) for e in http])
        results.extend({"engine": e.name, **(o or {})} for e, o in zip(http, outs))
    return results


# ------------------------------------------------------------------------------ NCCL broadcast path
@dataclass
class NCCLSyncGroup:
    group: Any
    rank: int
    world_size: int


def init_nccl_weight_sync(master_address: str, master_port: int, rank: int, world_size: int,
                          backend: str | None = None) -> NCCLSyncGroup:
    """Join (or create) the trainer<->engines group; rank 0 is the trainer."""
    if not dist.is_initialized():
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        dist.init_process_group(backend, init_method=f"tcp://{master_address}:{master_port}", rank=rank, world_size=world_size)
        return NCCLSyncGroup(dist.group.WORLD, rank, world_size)
    return NCCLSyncGroup(dist.new_group(list(range(world_size))), rank, world_size)


def sync_weights_nccl(sync: NCCLSyncGroup, flat_params: torch.Tensor, src: int = 0) -> None:
    """One broadcast of the flat parameter bucket (the reference issues one per tensor)."""
    dist.broadcast(flat_params, src=src, group=sync.group)
    dist.barrier(group=sync.group)


def cleanup_nccl_weight_sync(sync: NCCLSyncGroup) -> None:
    if sync.group is not dist.group.WORLD:
        dist.destroy_process_group(sync.group)


_ = shutil
