"""Remote execution and code deployment over ssh (bifrost/bifrost/client.py:32, deploy.py:171,
job.py:50-267, types.py:234-311).

``RemoteClient`` runs commands, pushes the current git tree as a bundle (only committed content travels,
like the reference's GitDeployment), and manages detached jobs: a job is a ``nohup`` child with its
output in ``<job_dir>/<name>/log`` and its pid / exit code in files beside it, so status and logs can be
read back by later, unrelated connections. The transport is a callable ``run(argv, input=None) ->
(code, stdout, stderr)``; the default uses the local ``ssh`` / ``sh`` binaries.
"""

from __future__ import annotations

import shlex
import subprocess
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable

Transport = Callable[[list[str], bytes | None], tuple[int, str, str]]


def subprocess_transport(argv: list[str], data: bytes | None = None) -> tuple[int, str, str]:
    p = subprocess.run(argv, input=data, capture_output=True)
    return p.returncode, p.stdout.decode(errors="replace"), p.stderr.decode(errors="replace")


@dataclass(frozen=True)
class ProcessSpec:
    command: str
    cwd: str | None = None
    env: dict[str, str] = field(default_factory=dict)
    name: str = "job"

    def shell_line(self) -> str:
        env = " ".join(f"{k}={shlex.quote(v)}" for k, v in self.env.items())
        cd = f"cd {shlex.quote(self.cwd)} && " if self.cwd else ""
        return f"{cd}{env + ' ' if env else ''}{self.command}"


@dataclass(frozen=True)
class JobInfo:
    name: str
    pid: int | None
    status: str            # running | exited | unknown
    exit_code: int | None
    log_path: str


class RemoteError(RuntimeError):
    pass


class RemoteClient:
    """``connection``: ``user@host[:port]`` or ``"local"`` (commands run through ``sh -c`` on this machine)."""

    def __init__(self, connection: str = "local", key: str | None = None, transport: Transport = subprocess_transport,
                 job_dir: str = "~/.bifrost/jobs"):
        self.connection, self.key, self.transport, self.job_dir = connection, key, transport, job_dir

    def _argv(self, command: str) -> list[str]:
        if self.connection == "local":
            return ["sh", "-c", command]
        host, _, port = self.connection.partition(":")
        argv = ["ssh", "-o", "BatchMode=yes", "-o", "StrictHostKeyChecking=accept-new"]
        if port:
            argv += ["-p", port]
        if self.key:
            argv += ["-i", self.key]
        return argv + [host, command]

    def exec(self, command: str, check: bool = False, data: bytes | None = None) -> tuple[int, str, str]:
        code, out, err = self.transport(self._argv(command), data)
        if check and code != 0:
            raise RemoteError(f"{command!r} exited {code}: {err.strip()[:500]}")
        return code, out, err

    # ------------------------------------------------------------------ code push
    def push(self, repo: str | Path, dest: str, ref: str = "HEAD") -> str:
        """Ship ``ref`` of a local git repository to ``dest`` on the target; returns the commit id deployed."""
        repo = Path(repo)
        commit = subprocess.run(["git", "-C", str(repo), "rev-parse", ref], capture_output=True, text=True, check=True).stdout.strip()
        bundle = subprocess.run(["git", "-C", str(repo), "bundle", "create", "-", ref], capture_output=True, check=True).stdout
        q = shlex.quote(dest)
        script = (f"set -e; mkdir -p {q}; cat > {q}/.incoming.bundle; cd {q}; [ -d .git ] || git init -q; "
                  f"git fetch -q .incoming.bundle {shlex.quote(ref)}; git checkout -q -f {commit}; rm -f .incoming.bundle")
        self.exec(script, check=True, data=bundle)
        return commit

    # ------------------------------------------------------------------ detached jobs
    def _jd(self, name: str) -> str:
        return f"{self.job_dir}/{name}"

    def start_job(self, spec: ProcessSpec) -> JobInfo:
        d = self._jd(spec.name)
        inner = f"( {spec.shell_line()} ); echo $? > {d}/exit_code"      # subshell: an `exit` in the command must not skip the record
        script = f"mkdir -p {d} && rm -f {d}/exit_code && (nohup sh -c {shlex.quote(inner)} > {d}/log 2>&1 & echo $! > {d}/pid) && cat {d}/pid"
        _, out, _ = self.exec(script, check=True)
        return JobInfo(spec.name, int(out.strip().splitlines()[-1]), "running", None, f"{d}/log")

    def job_status(self, name: str) -> JobInfo:
        d = self._jd(name)
        code, out, _ = self.exec(f"cat {d}/pid 2>/dev/null; echo '|'; cat {d}/exit_code 2>/dev/null; echo '|'; "
                                 f"kill -0 $(cat {d}/pid 2>/dev/null) 2>/dev/null && echo alive || echo dead")
        pid_s, exit_s, alive = (x.strip() for x in out.split("|"))
        pid = int(pid_s) if pid_s.isdigit() else None
        if exit_s.lstrip("-").isdigit():
            return JobInfo(name, pid, "exited", int(exit_s), f"{d}/log")
        return JobInfo(name, pid, "running" if alive == "alive" else "unknown", None, f"{d}/log")

    def job_logs(self, name: str, tail: int = 50) -> str:
        return self.exec(f"tail -n {int(tail)} {self._jd(name)}/log 2>/dev/null")[1]

    def wait_job(self, name: str, timeout: float = 3600.0, poll: float = 1.0) -> JobInfo:
        deadline = time.monotonic() + timeout
        while True:
            info = self.job_status(name)
            if info.status != "running":
                return info
            if time.monotonic() > deadline:
                raise TimeoutError(f"job {name!r} still running after {timeout}s")
            time.sleep(poll)

    def stop_job(self, name: str) -> None:
        """Terminate exactly the recorded pid of this job (never a pattern match)."""
        self.exec(f"kill $(cat {self._jd(name)}/pid) 2>/dev/null; true")
