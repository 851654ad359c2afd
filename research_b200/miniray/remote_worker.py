"""Client side of a worker running on another host (miniray/remote_worker.py:17-265):
same ``send`` / ``recv`` surface as ``Worker`` over TCP, plus ``health_check``."""

from __future__ import annotations

import socket
from typing import Any

from .worker import MAX_MESSAGE_BYTES, LineChannel


class RemoteWorker:
    def __init__(self, host: str, port: int, connect_timeout: float = 10.0):
        self.host, self.port, self.connect_timeout = host, port, connect_timeout
        self._chan: LineChannel | None = None

    def connect(self) -> "RemoteWorker":
        sock = socket.create_connection((self.host, self.port), timeout=self.connect_timeout)
        sock.settimeout(None)
        sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self._chan = LineChannel(sock)
        return self

    def _require(self) -> LineChannel:
        assert self._chan is not None, "call connect() first"
        return self._chan

    def send(self, msg: Any, binary: bool = False) -> None:
        self._require().send(msg, binary)

    def recv(self, timeout: float | None = None, max_size: int = MAX_MESSAGE_BYTES) -> Any:
        return self._require().recv(max_size, timeout)

    def fileno(self) -> int:
        return self._require().fileno()

    def is_alive(self) -> bool:
        return self.health_check(timeout=2.0)

    def health_check(self, timeout: float = 5.0) -> bool:
        """Round trip of ``{"cmd": "ping"}``; the server side answers ``{"status": "alive"}``."""
        if self._chan is None:
            return False
        try:
            self._chan.send({"cmd": "ping"})
            return self._chan.recv(timeout=timeout).get("status") == "alive"
        except (OSError, EOFError, TimeoutError, ValueError, AttributeError):
            return False

    def close(self) -> None:
        if self._chan is not None:
            self._chan.close()
            self._chan = None
