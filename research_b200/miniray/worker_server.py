"""TCP server that forks one worker per connection (miniray/worker_server.py:19-300).

``python -m research_b200.miniray.worker_server --port P --work-fn pkg.mod:fn`` listens, and for
every accepted connection forks a child that runs ``fn(handle)`` with ``handle`` speaking the
line protocol to the client. ``{"cmd": "ping"}`` is answered by the handle itself so health
checks work for any work function that polls ``handle.recv``.
"""

from __future__ import annotations

import argparse
import importlib
import os
import signal
import socket
import sys
from typing import Any, Callable

from .worker import MAX_MESSAGE_BYTES, LineChannel, _set_pdeathsig


class ServerHandle:
    """Child-side channel handed to the work function."""

    def __init__(self, sock: socket.socket):
        self._chan = LineChannel(sock)

    def send(self, msg: Any, binary: bool = False) -> None:
        self._chan.send(msg, binary)

    def recv(self, max_size: int = MAX_MESSAGE_BYTES, timeout: float | None = None) -> Any:
        while True:
            msg = self._chan.recv(max_size, timeout)
            if isinstance(msg, dict) and msg.get("cmd") == "ping":
                self._chan.send({"status": "alive", "pid": os.getpid()})
                continue
            return msg

    def fileno(self) -> int:
        return self._chan.fileno()


def resolve_work_fn(spec: str) -> Callable:
    mod, _, fn = spec.replace(":", ".").rpartition(".")
    return getattr(importlib.import_module(mod), fn)


class WorkerServer:
    def __init__(self, port: int, work_fn: Callable | str, host: str = "0.0.0.0", max_workers: int = 64):
        self.port, self.host, self.max_workers = port, host, max_workers
        self.work_fn = resolve_work_fn(work_fn) if isinstance(work_fn, str) else work_fn
        self.children: set[int] = set()
        self._sock: socket.socket | None = None
        self._stop = False

    def _cleanup(self, *_: Any) -> None:
        self._stop = True
        for pid in list(self.children):
            try:
                os.kill(pid, signal.SIGTERM)  # only children this server forked
            except ProcessLookupError:
                pass
        if self._sock is not None:
            try:
                self._sock.close()
            except OSError:
                pass

    def _reap(self) -> None:
        for pid in list(self.children):
            try:
                done, _ = os.waitpid(pid, os.WNOHANG)
            except ChildProcessError:
                done = pid
            if done:
                self.children.discard(pid)

    def serve_forever(self, max_connections: int | None = None) -> None:
        signal.signal(signal.SIGTERM, self._cleanup)
        signal.signal(signal.SIGINT, self._cleanup)
        self._sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._sock.bind((self.host, self.port))
        self._sock.listen(self.max_workers)
        self._sock.settimeout(0.5)
        served = 0
        while not self._stop and (max_connections is None or served < max_connections):
            self._reap()
            try:
                conn, _addr = self._sock.accept()
            except socket.timeout:
                continue
            except OSError:
                break
            conn.settimeout(None)
            pid = os.fork()
            if pid == 0:
                code = 0
                try:
                    _set_pdeathsig()
                    self._sock.close()
                    self.work_fn(ServerHandle(conn))
                except EOFError:
                    pass
                except BaseException:  # noqa: BLE001
                    import traceback

                    traceback.print_exc()
                    code = 1
                finally:
                    os._exit(code)
            conn.close()
            self.children.add(pid)
            served += 1
        while self.children and max_connections is not None:
            self._reap()
            signal.sigtimedwait([], 0.05) if hasattr(signal, "sigtimedwait") else None
        self._cleanup()


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="miniray worker server")
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--workers", type=int, default=64)
    ap.add_argument("--work-fn", required=True, help="package.module:function")
    args = ap.parse_args(argv)
    WorkerServer(args.port, args.work_fn, args.host, args.workers).serve_forever()
    return 0


if __name__ == "__main__":
    sys.exit(main())
