"""One SSH client for every remote-execution need: connection strings, key handling, blocking and streaming commands,
sync and async (shared/shared/ssh_foundation.py:23-600: ``secure_temp_ssh_key``, ``SSHConnectionInfo``,
``UniversalSSHClient``, ``execute_command_sync`` / ``_streaming``, ``test_ssh_connection``).

The transport is ``paramiko`` when it can be imported (the reference adds ``asyncssh`` for the async path; here the
async methods run the blocking ones in a worker thread, so one dependency covers both). ``client_factory`` lets a
caller (or a test) supply any object with paramiko's ``SSHClient`` surface.
"""

from __future__ import annotations

import asyncio
import contextlib
import os
import shlex
import stat
import tempfile
from dataclasses import dataclass
from typing import Any, Callable, Generator, Iterator, Protocol


@contextlib.contextmanager
def secure_temp_ssh_key(private_key_content: str) -> Generator[str, None, None]:
    """Write a private key to a file only its owner can read (0600), yield the path, and remove the file afterwards
    whatever happens. For keys that arrive as text (a secret store, an environment variable)."""
    fd, path = tempfile.mkstemp(prefix="ssh_key_", suffix=".pem")
    try:
        os.fchmod(fd, stat.S_IRUSR | stat.S_IWUSR)
        with os.fdopen(fd, "w") as f:
            f.write(private_key_content if private_key_content.endswith("\n") else private_key_content + "\n")
        yield path
    finally:
        with contextlib.suppress(OSError):
            os.remove(path)


@dataclass
class SSHConnectionInfo:
    hostname: str
    port: int
    username: str
    key_content: str | None = None
    key_path: str | None = None
    timeout: int = 30

    @classmethod
    def from_string(cls, conn_str: str, key_path: str | None = None, timeout: int = 30) -> "SSHConnectionInfo":
        """``user@host:port`` or a whole ``ssh [-p port] [-i key] user@host`` command line."""
        conn_str = conn_str.strip()
        if conn_str.startswith("ssh "):
            return cls._parse_ssh_command(conn_str, key_path, timeout)
        if "@" not in conn_str or ":" not in conn_str:
            raise ValueError(f"Invalid SSH format: {conn_str}. Expected: user@host:port or ssh -p port user@host")
        user_host, port_str = conn_str.rsplit(":", 1)
        username, hostname = user_host.split("@", 1)
        try:
            port = int(port_str)
        except ValueError as e:
            raise ValueError(f"Invalid port number: {port_str}") from e
        return cls(hostname, port, username, key_path=key_path, timeout=timeout)

    @classmethod
    def _parse_ssh_command(cls, ssh_cmd: str, key_path: str | None, timeout: int) -> "SSHConnectionInfo":
        try:
            parts = shlex.split(ssh_cmd)
        except ValueError as e:
            raise ValueError(f"Failed to parse SSH command: {e}") from e
        if not parts or parts[0] != "ssh":
            raise ValueError(f"Invalid SSH command: {ssh_cmd}")
        port, user_host, i = 22, None, 1
        while i < len(parts):
            if parts[i] == "-p" and i + 1 < len(parts):
                try:
                    port = int(parts[i + 1])
                except ValueError as e:
                    raise ValueError(f"Invalid port in SSH command: {parts[i + 1]}") from e
                i += 2
            elif parts[i] == "-i" and i + 1 < len(parts):
                key_path = key_path or parts[i + 1]
                i += 2
            elif parts[i] == "-o" and i + 1 < len(parts):
                i += 2
            elif "@" in parts[i]:
                user_host = parts[i]
                break
            else:
                i += 1
        if not user_host:
            raise ValueError(f"No user@host found in SSH command: {ssh_cmd}")
        username, hostname = user_host.split("@", 1)
        return cls(hostname, port, username, key_path=key_path, timeout=timeout)

    def load_key_content(self) -> str | None:
        if not self.key_path:
            return self.key_content
        try:
            with open(os.path.expanduser(self.key_path)) as f:
                return f.read()
        except OSError as e:
            raise ValueError(f"Failed to load SSH key from {self.key_path}: {e}") from e

    def connection_string(self) -> str:
        return f"{self.username}@{self.hostname}:{self.port}"


class SSHClientProtocol(Protocol):
    def connect(self, conn_info: SSHConnectionInfo) -> bool: ...
    def exec_command(self, command: str, timeout: int = 30) -> tuple[int, str, str]: ...
    def close(self) -> None: ...


class AsyncSSHClientProtocol(Protocol):
    async def aconnect(self, conn_info: SSHConnectionInfo) -> bool: ...
    async def aexec_command(self, command: str, timeout: int = 30) -> tuple[int, str, str]: ...
    async def aclose(self) -> None: ...


def _paramiko_factory():
    import paramiko

    c = paramiko.SSHClient()
    c.set_missing_host_key_policy(paramiko.AutoAddPolicy())
    return c


class UniversalSSHClient:
    """Connect once, run many commands. ``exec_command`` returns ``(exit_code, stdout, stderr)``;
    ``exec_command_streaming`` yields output lines as they arrive and finally ``("exit", code)``."""

    def __init__(self, client_factory: Callable[[], Any] | None = None) -> None:
        self._factory = client_factory or _paramiko_factory
        self._client: Any = None
        self.conn_info: SSHConnectionInfo | None = None
        self.last_error: str | None = None

    # ------------------------------------------------------------------ connection
    def connect(self, conn_info: SSHConnectionInfo) -> bool:
        """True on success; on failure ``last_error`` says why (bad key, refused, timeout) and nothing stays open."""
        self.close()
        self.conn_info, self.last_error = conn_info, None
        try:
            client = self._factory()
            kw: dict[str, Any] = dict(hostname=conn_info.hostname, port=conn_info.port, username=conn_info.username,
                                      timeout=conn_info.timeout, look_for_keys=conn_info.key_path is None and conn_info.key_content is None)
            if conn_info.key_content and not conn_info.key_path:
                with secure_temp_ssh_key(conn_info.key_content) as path:
                    client.connect(key_filename=path, **kw)
            elif conn_info.key_path:
                client.connect(key_filename=os.path.expanduser(conn_info.key_path), **kw)
            else:
                client.connect(**kw)
            self._client = client
            return True
        except Exception as e:  # noqa: BLE001 - every connection problem is reported the same way
            self.last_error = f"{type(e).__name__}: {e}"
            self._client = None
            return False

    @property
    def connected(self) -> bool:
        return self._client is not None

    def close(self) -> None:
        if self._client is not None:
            with contextlib.suppress(Exception):
                self._client.close()
            self._client = None

    def __enter__(self) -> "UniversalSSHClient":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    # ------------------------------------------------------------------ commands
    def exec_command(self, command: str, timeout: int = 30) -> tuple[int, str, str]:
        if self._client is None:
            return -1, "", "not connected"
        try:
            _, out, err = self._client.exec_command(command, timeout=timeout)
            so, se = out.read(), err.read()
            code = out.channel.recv_exit_status()
            return code, so.decode(errors="replace") if isinstance(so, bytes) else so, se.decode(errors="replace") if isinstance(se, bytes) else se
        except Exception as e:  # noqa: BLE001
            return -1, "", f"{type(e).__name__}: {e}"

    def exec_command_streaming(self, command: str, timeout: int | None = None, merge_stderr: bool = True) -> Iterator[str | tuple[str, int]]:
        """Lines of the command's output while it runs (stderr folded in by asking for a pty-less ``2>&1``), then the
        final ``("exit", code)`` item."""
        if self._client is None:
            yield ("exit", -1)
            return
        cmd = f"( {command} ) 2>&1" if merge_stderr else command
        _, out, _ = self._client.exec_command(cmd, timeout=timeout)
        for line in iter(out.readline, ""):
            if isinstance(line, bytes):
                line = line.decode(errors="replace")
            if not line:
                break
            yield line.rstrip("\n")
        yield ("exit", out.channel.recv_exit_status())

    # ------------------------------------------------------------------ async surface
    async def aconnect(self, conn_info: SSHConnectionInfo) -> bool:
        return await asyncio.to_thread(self.connect, conn_info)

    async def aexec_command(self, command: str, timeout: int = 30) -> tuple[int, str, str]:
        return await asyncio.to_thread(self.exec_command, command, timeout)

    async def aclose(self) -> None:
        await asyncio.to_thread(self.close)


def execute_command_sync(conn_info: SSHConnectionInfo, command: str, timeout: int = 30, client_factory=None) -> tuple[int, str, str]:
    """Connect, run one command, disconnect."""
    with UniversalSSHClient(client_factory) as c:
        if not c.connect(conn_info):
            return -1, "", c.last_error or "connection failed"
        return c.exec_command(command, timeout)


def execute_command_streaming(conn_info: SSHConnectionInfo, command: str, on_line: Callable[[str], None] = print,
                              client_factory=None) -> int:
    """Connect, run one command with its output handed to ``on_line`` as it arrives; returns the exit code."""
    with UniversalSSHClient(client_factory) as c:
        if not c.connect(conn_info):
            on_line(f"ssh: {c.last_error}")
            return -1
        code = -1
        for item in c.exec_command_streaming(command):
            if isinstance(item, tuple):
                code = item[1]
            else:
                on_line(item)
        return code


def interactive_ssh_argv(conn_info: SSHConnectionInfo, key_path: str | None = None) -> list[str]:
    """Command line of an interactive ``ssh`` session to the same endpoint (for ``os.execvp`` / ``subprocess``)."""
    argv = ["ssh", "-p", str(conn_info.port), "-o", "StrictHostKeyChecking=no"]
    if key_path or conn_info.key_path:
        argv += ["-i", os.path.expanduser(key_path or conn_info.key_path)]
    return argv + [f"{conn_info.username}@{conn_info.hostname}"]


def test_ssh_connection(conn_info: SSHConnectionInfo, test_both: bool = True, client_factory=None) -> tuple[bool, str]:
    """Round trip of ``echo`` through the sync path and (``test_both``) the async path; ``(ok, message)``."""
    code, out, err = execute_command_sync(conn_info, "echo ssh_ok", client_factory=client_factory)
    if code != 0 or "ssh_ok" not in out:
        return False, f"sync path failed: {err or out or code}"
    if test_both:
        async def run() -> tuple[int, str, str]:
            c = UniversalSSHClient(client_factory)
            try:
                if not await c.aconnect(conn_info):
                    return -1, "", c.last_error or "connection failed"
                return await c.aexec_command("echo ssh_ok")
            finally:
                await c.aclose()

        code, out, err = asyncio.run(run())
        if code != 0 or "ssh_ok" not in out:
            return False, f"async path failed: {err or out or code}"
    return True, f"connected to {conn_info.connection_string()}"


test_ssh_connection.__test__ = False     # a library function, not a pytest case
