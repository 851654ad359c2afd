"""Local worker processes: ``fork`` + a ``socketpair`` carrying newline-delimited messages.

Surface of the reference's miniray worker (miniray/worker.py:41-530): ``Worker`` with
``send`` / ``recv`` / ``fileno`` / ``is_alive`` / ``wait``, ``wait_any`` (select over workers),
``SharedMemory`` (memfd or tempfile, zero-copy hand-off of large buffers),
``spawn_training_workers`` (one worker per GPU, ``CUDA_VISIBLE_DEVICES`` set in the child) and
``shutdown_workers``. Children die with their parent (``PR_SET_PDEATHSIG``). Stdlib only.
"""

from __future__ import annotations

import base64
import ctypes
import json
import marshal
import mmap
import os
import select
import signal
import socket
import sys
import tempfile
import time
from typing import Any, Callable

MAX_MESSAGE_BYTES = 100 * 1024 * 1024
PR_SET_PDEATHSIG = 1


def _set_pdeathsig(sig: int = signal.SIGTERM) -> None:
    """Ask the kernel to signal this process when its parent exits (Linux only; best effort)."""
    try:
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        libc.prctl(PR_SET_PDEATHSIG, sig, 0, 0, 0)
    except OSError:
        pass


def encode_message(msg: Any, binary: bool = False) -> bytes:
    """One line per message. ``binary`` uses marshal + base64 (faster for large nested payloads)."""
    if binary:
        return b"M" + base64.b64encode(marshal.dumps(msg)) + b"\n"
    return b"J" + json.dumps(msg, separators=(",", ":")).encode() + b"\n"


def decode_message(line: bytes) -> Any:
    tag, body = line[:1], line[1:].rstrip(b"\n")
    if tag == b"M":
        return marshal.loads(base64.b64decode(body))
    if tag == b"J":
        return json.loads(body)
    return json.loads(line)  # untagged plain JSON from foreign peers


class LineChannel:
    """Buffered newline-delimited framing over a connected socket."""

    def __init__(self, sock: socket.socket):
        self.sock = sock
        self._buf = bytearray()

    def fileno(self) -> int:
        return self.sock.fileno()

    def send(self, msg: Any, binary: bool = False) -> None:
        data = encode_message(msg, binary)
        assert len(data) <= MAX_MESSAGE_BYTES, f"message of {len(data)} bytes exceeds the {MAX_MESSAGE_BYTES} limit"
        self.sock.sendall(data)

    def recv(self, max_size: int = MAX_MESSAGE_BYTES, timeout: float | None = None) -> Any:
        deadline = None if timeout is None else time.monotonic() + timeout
        while True:
            nl = self._buf.find(b"\n")
            if nl >= 0:
                line = bytes(self._buf[:nl + 1])
                del self._buf[:nl + 1]
                return decode_message(line)
            if len(self._buf) > max_size:
                raise ValueError(f"message exceeds max_size={max_size}")
            if deadline is not None:
                left = deadline - time.monotonic()
                if left <= 0 or not select.select([self.sock], [], [], left)[0]:
                    raise TimeoutError("recv timed out")
            chunk = self.sock.recv(1 << 20)
            if not chunk:
                raise EOFError("peer closed the connection")
            self._buf += chunk

    def close(self) -> None:
        try:
            self.sock.close()
        except OSError:
            pass


class SharedMemory:
    """Anonymous shared buffer (``memfd_create`` when available, else an unlinked temp file)."""

    MAX_BYTES = 1 << 30

    def __init__(self, fd: int, size: int):
        self.fd, self.size = fd, size
        self.buf = mmap.mmap(fd, size)

    @staticmethod
    def create(size: int, name: str = "miniray") -> "SharedMemory":
        assert 0 < size <= SharedMemory.MAX_BYTES
        if hasattr(os, "memfd_create"):
            fd = os.memfd_create(name)
        else:  # pragma: no cover
            f = tempfile.TemporaryFile()
            fd = os.dup(f.fileno())
            f.close()
        os.ftruncate(fd, size)
        return SharedMemory(fd, size)

    @staticmethod
    def map(fd: int, size: int) -> "SharedMemory":
        return SharedMemory(fd, size)

    def close(self) -> None:
        self.buf.close()
        os.close(self.fd)


class Worker:
    """A forked child running ``work_fn(handle)`` where ``handle`` is the child's end of the pipe."""

    def __init__(self, work_fn: Callable[["Worker"], Any], *args: Any, env: dict[str, str] | None = None, **kwargs: Any):
        parent_sock, child_sock = socket.socketpair()
        sys.stdout.flush()
        sys.stderr.flush()
        pid = os.fork()
        if pid == 0:  # ---- child
            code = 0
            try:
                _set_pdeathsig()
                parent_sock.close()
                if env:
                    os.environ.update(env)
                self.pid, self._chan, self._is_child = os.getpid(), LineChannel(child_sock), True
                work_fn(self, *args, **kwargs)
            except BaseException as e:  # noqa: BLE001 - report and exit non-zero
                code = 1
                try:
                    import traceback

                    traceback.print_exc()
                    self._chan.send({"error": f"{type(e).__name__}: {e}"})
                except Exception:
                    pass
            finally:
                sys.stdout.flush()
                sys.stderr.flush()
                os._exit(code)
        child_sock.close()
        self.pid, self._chan, self._is_child = pid, LineChannel(parent_sock), False
        self._exit_code: int | None = None

    def send(self, msg: Any, binary: bool = False) -> None:
        self._chan.send(msg, binary)

    def recv(self, max_size: int = MAX_MESSAGE_BYTES, timeout: float | None = None) -> Any:
        return self._chan.recv(max_size, timeout)

    def fileno(self) -> int:
        return self._chan.fileno()

    def is_alive(self) -> bool:
        if self._exit_code is not None:
            return False
        pid, status = os.waitpid(self.pid, os.WNOHANG)
        if pid == 0:
            return True
        self._exit_code = os.waitstatus_to_exitcode(status)
        return False

    def wait(self, timeout: float | None = None, check: bool = True) -> int:
        """Wait for the child to exit; with ``check`` a non-zero exit raises."""
        deadline = None if timeout is None else time.monotonic() + timeout
        while self._exit_code is None:
            pid, status = os.waitpid(self.pid, os.WNOHANG)
            if pid != 0:
                self._exit_code = os.waitstatus_to_exitcode(status)
                break
            if deadline is not None and time.monotonic() > deadline:
                raise TimeoutError(f"worker {self.pid} still running after {timeout}s")
            time.sleep(0.01)
        if check and self._exit_code != 0:
            raise RuntimeError(f"worker {self.pid} exited with code {self._exit_code}")
        return self._exit_code

    def terminate(self) -> None:
        if self.is_alive():
            os.kill(self.pid, signal.SIGTERM)  # exactly the child we forked

    def close(self) -> None:
        self._chan.close()


def wait_any(workers: list[Worker], timeout: float | None = None) -> list[Worker]:
    """Workers that have a message ready (or closed their end)."""
    ready, _, _ = select.select(workers, [], [], timeout)
    return list(ready)


def spawn_training_workers(n: int, work_fn: Callable, *args: Any, master_port: int = 29500, **kwargs: Any) -> list[Worker]:
    """One worker per GPU: rank r sees only GPU r and gets the torch.distributed environment."""
    workers = []
    for rank in range(n):
        env = {"CUDA_VISIBLE_DEVICES": str(rank), "RANK": str(rank), "LOCAL_RANK": "0", "WORLD_SIZE": str(n),
               "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(master_port)}
        workers.append(Worker(work_fn, *args, env=env, **kwargs))
    return workers


def shutdown_workers(workers: list[Worker], timeout: float = 10.0) -> None:
    for w in workers:
        try:
            w.send({"cmd": "shutdown"})
        except OSError:
            pass
    for w in workers:
        try:
            w.wait(timeout, check=False)
        except TimeoutError:
            w.terminate()
            w.wait(timeout, check=False)
        w.close()
