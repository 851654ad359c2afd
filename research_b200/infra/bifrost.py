"""Remote execution and code deployment over ssh (bifrost/bifrost/client.py:32, deploy.py:171,
job.py:50-267, types.py:234-311).

``RemoteClient`` runs commands, pushes the current git tree as a bundle (only committed content travels,
like the reference's GitDeployment), and manages detached jobs: a job is a ``nohup`` child with its
output in ``<job_dir>/<name>/log`` and its pid / exit code in files beside it, so status and logs can be
read back by later, unrelated connections. The transport is a callable ``run(argv, input=None) ->
(code, stdout, stderr)``; the default uses the local ``ssh`` / ``sh`` binaries.
"""

from __future__ import annotations

import re
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
        env = "".join(f"export {k}={shlex.quote(v)}; " for k, v in self.env.items())   # exported first, so the command line may expand them
        cd = f"cd {shlex.quote(self.cwd)} && " if self.cwd else ""
        return f"{cd}{env}{self.command}"


@dataclass(frozen=True)
class JobInfo:
    name: str
    pid: int | None
    status: str            # running | exited | unknown
    exit_code: int | None
    log_path: str


class RemoteError(RuntimeError):
    pass


# ------------------------------------------------------------------------------------------- validation of what reaches a shell
_ENV_NAME = re.compile(r"^[A-Za-z_][A-Za-z0-9_]*$")
_JOB_NAME = re.compile(r"^[A-Za-z0-9][A-Za-z0-9._-]{0,63}$")


def validate_job_name(name: str) -> str:
    """Job names become directory names on the target: letters, digits, ``. _ -``, at most 64 characters, no leading dot or dash."""
    if not _JOB_NAME.match(name or "") or ".." in name:
        raise ValueError(f"invalid job name {name!r}: use letters, digits, '.', '_' or '-' (1-64 characters, starting with a letter or digit)")
    return name


def generate_job_name(prefix: str = "job") -> str:
    import secrets

    return validate_job_name(f"{prefix}-{time.strftime('%Y%m%d-%H%M%S')}-{secrets.token_hex(3)}")


def validate_env(env: dict[str, str]) -> dict[str, str]:
    for k, v in env.items():
        if not _ENV_NAME.match(k):
            raise ValueError(f"invalid environment variable name {k!r}")
        if not isinstance(v, str) or "\x00" in v:
            raise ValueError(f"environment variable {k} must be a string without NUL bytes")
    return env


def validate_working_directory(path: str) -> str:
    if not path or "\x00" in path or "\n" in path or ".." in Path(path).parts:
        raise ValueError(f"invalid working directory {path!r}: no empty path, no '..' component, no control characters")
    return path


def make_env_payload(env: dict[str, str]) -> bytes:
    """``NAME='value'`` lines for the loader of ``wrap_with_env_loader``; values are shell-quoted, names validated."""
    validate_env(env)
    return ("".join(f"{k}={shlex.quote(v)}\n" for k, v in env.items())).encode()


def wrap_with_env_loader(command: str) -> str:
    """``command`` preceded by a loader that reads exported variables from standard input: secrets travel on the
    connection's stdin, not in the command line, so they show up neither in ``ps`` on the target nor in shell history or
    logs of commands (bifrost/bifrost/deploy.py:71-89)."""
    return f"set -a; . /dev/stdin; set +a; sh -c {shlex.quote(command)}"


def detect_bootstrap(files: Callable[[str], bool], extra: str | None = None, frozen: bool = False) -> str:
    """The dependency-installation command a checkout needs, from the files it has (``files(name) -> exists``):
    ``uv.lock`` / ``pyproject.toml`` -> ``uv sync``, ``requirements.txt`` -> ``pip install -r``, none -> ``""``."""
    uv = "pip install uv && uv sync" + (" --frozen" if frozen else "") + (f" --extra {shlex.quote(extra)}" if extra else "")
    for name, cmd in (("uv.lock", uv), ("pyproject.toml", uv), ("requirements.txt", "pip install -r requirements.txt")):
        if files(name):
            return cmd
    return ""


def local_changes(repo: str | Path) -> list[str]:
    """Paths of ``repo`` that a push would leave behind: modified, staged or untracked (and not ignored) files
    (bifrost/bifrost/git_sync.py:49-108)."""
    r = subprocess.run(["git", "-C", str(repo), "status", "--porcelain"], capture_output=True, text=True)
    return [line[3:] for line in r.stdout.splitlines() if line.strip()] if r.returncode == 0 else []


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

    def exec_with_env(self, command: str, env: dict[str, str], cwd: str | None = None, check: bool = False) -> tuple[int, str, str]:
        """Run ``command`` with ``env`` exported, the variables sent on standard input (see ``wrap_with_env_loader``)."""
        cd = f"cd {shlex.quote(validate_working_directory(cwd))} && " if cwd else ""
        return self.exec(wrap_with_env_loader(cd + command), check=check, data=make_env_payload(env))

    def detect_bootstrap(self, dest: str, extra: str | None = None, frozen: bool = False) -> str:
        q = self._q(dest)
        return detect_bootstrap(lambda name: self.exec(f"[ -f {q}/{name} ]")[0] == 0, extra, frozen)

    # ------------------------------------------------------------------ code push
    def push(self, repo: str | Path, dest: str, ref: str = "HEAD", bootstrap: str | list[str] | None = None,
             warn: Callable[[str], None] | None = None) -> str:
        """Ship ``ref`` of a local git repository to ``dest`` on the target; returns the commit id deployed.
        ``bootstrap``: command(s) run in ``dest`` afterwards (environment set-up, builds); a failure raises."""
        repo = Path(repo)
        self.not_shipped = local_changes(repo)       # a push ships commits: what is only in the working tree stays behind
        if self.not_shipped and warn is not None:
            warn(f"{len(self.not_shipped)} uncommitted or untracked path(s) are NOT part of this push: " +
                 ", ".join(self.not_shipped[:8]) + (" ..." if len(self.not_shipped) > 8 else ""))
        commit = subprocess.run(["git", "-C", str(repo), "rev-parse", ref], capture_output=True, text=True, check=True).stdout.strip()
        bundle = subprocess.run(["git", "-C", str(repo), "bundle", "create", "-", ref], capture_output=True, check=True).stdout
        q = shlex.quote(dest)
        script = (f"set -e; mkdir -p {q}; cat > {q}/.incoming.bundle; cd {q}; [ -d .git ] || git init -q; "
                  f"git fetch -q .incoming.bundle {shlex.quote(ref)}; git checkout -q -f {commit}; rm -f .incoming.bundle")
        self.exec(script, check=True, data=bundle)
        if bootstrap == "auto":
            bootstrap = self.detect_bootstrap(dest) or None
        for cmd in ([bootstrap] if isinstance(bootstrap, str) else list(bootstrap or [])):
            self.exec(f"cd {q} && {cmd}", check=True)
        return commit

    def push_worktree(self, repo: str | Path, base: str, job: str, ref: str = "HEAD") -> str:
        """One checkout per job: the repository is pushed to ``<base>/repo`` once (updated on later pushes) and ``ref`` is
        checked out into ``<base>/jobs/<job>`` as a git worktree, so that concurrent jobs on one machine never share a
        working tree and an old job's code stays as it ran (bifrost/bifrost/deploy.py:289-440). Returns the worktree path."""
        validate_job_name(job)
        main = f"{base.rstrip('/')}/repo"
        commit = self.push(repo, main, ref)
        tree = f"{base.rstrip('/')}/jobs/{job}"
        self.exec(f"mkdir -p {self._q(base.rstrip('/') + '/jobs')} && cd {self._q(main)} && git worktree add -f --detach {self._q(tree)} {commit}", check=True)
        return tree

    def remove_worktree(self, base: str, job: str) -> bool:
        validate_job_name(job)
        main, tree = f"{base.rstrip('/')}/repo", f"{base.rstrip('/')}/jobs/{job}"
        return self.exec(f"cd {self._q(main)} && git worktree remove --force {self._q(tree)}")[0] == 0


    # ------------------------------------------------------------------ detached jobs
    def _jd(self, name: str) -> str:
        return f"{self.job_dir}/{name}"

    def start_job(self, spec: ProcessSpec) -> JobInfo:
        validate_job_name(spec.name)
        validate_env(spec.env)
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

    # ------------------------------------------------------------------ streaming, paths, files
    def exec_stream(self, command: str):
        """Yield the command's output (stdout and stderr merged) line by line as it appears; the generator's return
        value (``StopIteration.value``) is the exit code (bifrost/bifrost/client.py:383). Streams through a local
        ``ssh`` / ``sh`` child whatever the configured transport is."""
        argv = self._argv(command)
        p = subprocess.Popen(argv, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, bufsize=1)
        drained = False
        try:
            for line in p.stdout:
                yield line.rstrip("\n")
            drained = True
        finally:
            p.stdout.close()
            if not drained and p.poll() is None:      # the consumer stopped early: end exactly this child
                p.terminate()
        return p.wait()

    def expand_path(self, path: str) -> str:
        """``~`` and variables expanded by the target's shell."""
        return self.exec(f"echo {path}", check=True)[1].strip()

    def upload(self, local: str | Path, remote: str) -> int:
        """Copy a file or a directory tree to ``remote`` (created as needed); returns the bytes sent. The payload is a
        tar stream on the command's standard input, so one connection carries any number of files."""
        import io
        import tarfile

        local = Path(local)
        if not local.exists():
            raise FileNotFoundError(local)
        buf = io.BytesIO()
        with tarfile.open(fileobj=buf, mode="w") as tf:
            if local.is_dir():
                for p in sorted(local.rglob("*")):
                    tf.add(p, arcname=str(p.relative_to(local)), recursive=False)
            else:
                tf.add(local, arcname=Path(remote).name if not remote.endswith("/") else local.name)
        dest = remote if local.is_dir() or remote.endswith("/") else str(Path(remote).parent)
        q = shlex.quote(dest) if not dest.startswith("~") else dest
        self.exec(f"mkdir -p {q} && tar -xf - -C {q}", check=True, data=buf.getvalue())
        return buf.getbuffer().nbytes

    def download(self, remote: str, local: str | Path) -> int:
        """Copy a remote file or directory tree to ``local``; returns the number of files written. Content travels
        base64-encoded because the transport returns text."""
        import base64
        import io
        import tarfile

        q = shlex.quote(remote) if not remote.startswith("~") else remote
        _, out, _ = self.exec(f"if [ -d {q} ]; then tar -cf - -C {q} . | base64; elif [ -f {q} ]; then "
                              f"tar -cf - -C $(dirname {q}) $(basename {q}) | base64; else exit 44; fi", check=True)
        local = Path(local)
        is_dir = self.exec(f"[ -d {q} ]")[0] == 0
        n = 0
        with tarfile.open(fileobj=io.BytesIO(base64.b64decode(out)), mode="r") as tf:
            for m in tf.getmembers():
                if not m.isfile() or m.name.startswith("/") or ".." in Path(m.name).parts:
                    continue
                target = (local / m.name) if is_dir else local
                target.parent.mkdir(parents=True, exist_ok=True)
                target.write_bytes(tf.extractfile(m).read())
                n += 1
        return n

    # ------------------------------------------------------------------ single files on the target
    @staticmethod
    def _q(path: str) -> str:
        return path if path.startswith("~") else shlex.quote(path)      # a quoted ~ would not expand

    def ensure_dir(self, path: str) -> None:
        self.exec(f"mkdir -p {self._q(path)}", check=True)

    def path_exists(self, path: str) -> bool:
        return self.exec(f"[ -e {self._q(path)} ]")[0] == 0

    def write_file(self, path: str, content: str | bytes, mode: int | None = None) -> None:
        """Write ``content`` to ``path`` on the target without any shell quoting of the content (it travels on standard
        input) and atomically: a reader sees the old file or the new one, never a partial write
        (bifrost/bifrost/remote_fs.py:22)."""
        q, data = self._q(path), content.encode() if isinstance(content, str) else content
        chmod = f"chmod {mode:o} {q}.incoming && " if mode is not None else ""
        self.exec(f"mkdir -p $(dirname {q}) && cat > {q}.incoming && {chmod}mv -f {q}.incoming {q}", check=True, data=data)

    def read_file(self, path: str) -> str:
        code, out, err = self.exec(f"cat {self._q(path)}")
        if code != 0:
            raise FileNotFoundError(f"{path} on {self.connection}: {err.strip()[:200]}")
        return out

    def remove_file(self, path: str) -> bool:
        """Remove one file (never a directory, never a pattern); True if it existed."""
        q = self._q(path)
        return self.exec(f"[ -f {q} ] && rm -f -- {q}")[0] == 0

    # ------------------------------------------------------------------ servers
    def serve(self, spec: ProcessSpec, port: int, health_path: str = "/health", timeout: float = 600.0, poll: float = 1.0) -> "ServerInfo":
        """Start ``spec`` as a detached job and wait until ``http://127.0.0.1:<port><health_path>`` answers on the target
        (probed there, so no tunnel is needed); raises with the log tail if the job exits first
        (bifrost/bifrost/client.py:638, server.py)."""
        job = self.start_job(spec)
        probe = (f"python3 -c \"import urllib.request,sys; sys.exit(0 if urllib.request.urlopen('http://127.0.0.1:{int(port)}{health_path}',"
                 f" timeout=2).status < 500 else 1)\" 2>/dev/null || curl -sf -o /dev/null http://127.0.0.1:{int(port)}{health_path}")
        deadline = time.monotonic() + timeout
        while True:
            if self.exec(probe)[0] == 0:
                host = "127.0.0.1" if self.connection == "local" else self.connection.partition(":")[0].rpartition("@")[2]
                return ServerInfo(spec.name, job.pid, port, f"http://{host}:{port}", job.log_path)
            info = self.job_status(spec.name)
            if info.status != "running":
                raise RemoteError(f"server {spec.name!r} ended ({info.status}, exit {info.exit_code}) before it answered:\n"
                                  + self.job_logs(spec.name, 30))
            if time.monotonic() > deadline:
                raise TimeoutError(f"server {spec.name!r} did not answer on port {port} within {timeout}s")
            time.sleep(poll)

    def tunnel_argv(self, local_port: int, remote_port: int) -> list[str]:
        """Command line of an ssh port forward to a served port (run it with ``subprocess.Popen``)."""
        if self.connection == "local":
            raise RemoteError("a local target needs no tunnel")
        host, _, port = self.connection.partition(":")
        argv = ["ssh", "-N", "-L", f"{int(local_port)}:127.0.0.1:{int(remote_port)}", "-o", "BatchMode=yes", "-o", "ExitOnForwardFailure=yes"]
        return argv + (["-p", port] if port else []) + (["-i", self.key] if self.key else []) + [host]


@dataclass(frozen=True)
class ServerInfo:
    name: str
    pid: int | None
    port: int
    url: str
    log_path: str


class AsyncRemoteClient:
    """The same operations as coroutines (bifrost/bifrost/async_client.py): each call runs the blocking client in a
    worker thread, so many targets can be driven from one event loop."""

    def __init__(self, *a, **kw):
        self.sync = RemoteClient(*a, **kw)

    def __getattr__(self, name: str):
        import asyncio
        import functools

        fn = getattr(self.sync, name)
        if not callable(fn) or name in ("exec_stream", "tunnel_argv"):
            return fn

        @functools.wraps(fn)
        async def call(*a, **kw):
            return await asyncio.to_thread(fn, *a, **kw)
        return call

    async def exec_stream(self, command: str):
        import asyncio

        proc = await asyncio.create_subprocess_exec(*self.sync._argv(command), stdout=asyncio.subprocess.PIPE,
                                                    stderr=asyncio.subprocess.STDOUT)
        async for raw in proc.stdout:
            yield raw.decode(errors="replace").rstrip("\n")
        await proc.wait()


@dataclass(frozen=True)
class GPUQuery:
    """What to provision when no machine is given (bifrost/bifrost/provision.py:30)."""
    type: str = "B200"
    count: int = 1
    max_price: float | None = None
    min_vram_gb: int | None = None
    spot: bool | None = None

    def condition(self):
        from .broker import q

        cond = q.gpu_type.contains(self.type) & (q.gpu_count >= self.count)
        if self.max_price is not None:
            cond = cond & (q.price_per_hour <= self.max_price)
        if self.min_vram_gb is not None:
            cond = cond & (q.vram_gb >= self.min_vram_gb)
        if self.spot is not None:
            cond = cond & (q.spot == self.spot)
        return cond


def acquire_node(ssh: str | None = None, node_id: str | None = None, provision: GPUQuery | None = None, gpu_client=None,
                 key: str | None = None, ssh_timeout: float = 600.0, poll: float = 5.0, transport: Transport = subprocess_transport,
                 **create_kw):
    """Exactly one of: ``ssh`` (a ``user@host[:port]`` string), ``node_id`` (an instance the broker already tracks) or
    ``provision`` (a query; the cheapest match is created). Returns ``(RemoteClient, instance | None)`` once the target
    answers ``echo ok`` (bifrost/bifrost/provision.py:50). ``gpu_client`` is a ``broker.GPUClient``."""
    if sum(x is not None for x in (ssh, node_id, provision)) != 1:
        raise ValueError("give exactly one of ssh, node_id, provision")
    inst = None
    if ssh is None:
        if gpu_client is None:
            raise ValueError("node_id / provision need a gpu_client")
        if node_id is not None:
            inst = gpu_client.instances.get(node_id.partition(":")[2] or node_id)
            if inst is None:
                raise RemoteError(f"the broker tracks no instance {node_id!r}")
        else:
            inst = gpu_client.create(provision.condition(), **create_kw)
    deadline = time.monotonic() + ssh_timeout
    while True:
        conn = ssh or inst.ssh_connection
        if not conn and inst is not None:
            refresh = getattr(gpu_client.providers[inst.provider], "refresh", None)
            if refresh:
                inst = refresh(inst.instance_id)
                conn = inst.ssh_connection
        if conn:
            client = RemoteClient(conn, key=key, transport=transport)
            if client.exec("echo ok")[1].strip() == "ok":
                return client, inst
        if time.monotonic() > deadline:
            raise TimeoutError(f"no ssh answer from {conn or (inst and inst.instance_id)!r} within {ssh_timeout}s")
        time.sleep(poll)
