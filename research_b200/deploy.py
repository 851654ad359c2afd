"""Describe, check and launch an inference server (rollouts/deploy.py:42-1157).

``ServerConfig`` covers both the native engine (``engine="native"``: ``python -m research_b200.cli
serve ...``) and an external SGLang process (``engine="sglang"``: the command line of the
reference, ``build_sglang_command``). Launching is a plain child process with its output teed to a
log file (no tmux dependency) and a 1 Hz health poll that notices a dead child at once. Remote
hosts are reached through an injectable ``run`` callable (ssh in production, a fake in tests).

Nothing here touches other users' processes: the reference's "kill whatever runs on these GPUs"
preflight is replaced by a check that reports busy GPUs and refuses to continue.
"""

from __future__ import annotations

import shlex
import subprocess
import sys
import time
import urllib.request
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable

Runner = Callable[[str], tuple[int, str]]          # shell command -> (exit code, output)


@dataclass
class ServerConfig:
    model: str = "qwen2.5-0.5b"
    engine: str = "native"                        # native | sglang
    dtype: str = "auto"
    max_model_len: int | None = None
    quantization: str | None = None
    trust_remote_code: bool = True
    attention_backend: str | None = None          # sglang only; "triton" on Blackwell
    gpu_ranks: list[int] = field(default_factory=lambda: [0])
    port: int = 30000
    host: str = "127.0.0.1"
    tensor_parallel_size: int = 1
    gpu_memory_utilization: float = 0.9
    enable_prefix_caching: bool = True
    max_batch_size: int = 256
    ssh_connection: str | None = None             # "user@host[:port]"; None = this machine
    log_dir: str = "logs/servers"
    name: str = "engine-server"

    def __post_init__(self) -> None:
        assert self.model, "model cannot be empty"
        assert 1024 < self.port < 65536, f"invalid port {self.port}"
        assert self.gpu_ranks, "gpu_ranks cannot be empty"
        if self.tensor_parallel_size != len(self.gpu_ranks):
            raise ValueError(f"tensor_parallel_size ({self.tensor_parallel_size}) must match the number of GPUs ({len(self.gpu_ranks)})")

    @property
    def url(self) -> str:
        host = self.ssh_connection.split("@")[-1].split(":")[0] if self.ssh_connection else self.host
        return f"http://{host}:{self.port}"


@dataclass(frozen=True)
class ServerInfo:
    url: str
    pid: int | None
    log_path: str
    command: str


def build_sglang_command(config: ServerConfig) -> str:
    parts = ["python -m sglang.launch_server", f"--model {config.model}", f"--host {config.host}", f"--port {config.port}"]
    if config.tensor_parallel_size > 1:
        parts.append(f"--tp {config.tensor_parallel_size}")
    if config.max_model_len:
        parts.append(f"--context-length {config.max_model_len}")
    if config.dtype != "auto":
        parts.append(f"--dtype {config.dtype}")
    if config.quantization:
        parts.append(f"--quantization {config.quantization}")
    if config.trust_remote_code:
        parts.append("--trust-remote-code")
    parts.append(f"--mem-fraction-static {config.gpu_memory_utilization}")
    if config.enable_prefix_caching:
        parts.append("--enable-radix-cache")
    if config.attention_backend:
        parts += [f"--attention-backend {config.attention_backend}", "--mm-attention-backend triton_attn"]
    return " \\\n    ".join(parts)


def build_native_command(config: ServerConfig) -> str:
    parts = [f"{shlex.quote(sys.executable)} -m research_b200.cli serve", f"--model {shlex.quote(config.model)}",
             f"--host {config.host}", f"--port {config.port}", f"--max-batch-size {config.max_batch_size}",
             f"--cache {'radix' if config.enable_prefix_caching else 'paged'}", f"--gpu-memory-utilization {config.gpu_memory_utilization}"]
    if config.max_model_len:
        parts.append(f"--max-model-len {config.max_model_len}")
    if config.tensor_parallel_size > 1:
        launcher = (f"{shlex.quote(sys.executable)} -m torch.distributed.run --nnodes=1 --nproc-per-node {config.tensor_parallel_size} "
                    f"--master-addr 127.0.0.1 --master-port {config.port + 1000} -m research_b200.cli serve")
        parts[0] = launcher
        parts.append(f"--tp {config.tensor_parallel_size}")
    return " ".join(parts)


SGLANG_VENV = ".venv-sglang"


def generate_bootstrap_command(config: ServerConfig, workdir: str = ".") -> str:
    """What a fresh machine runs once before the launch command (rollouts/deploy.py:124-162). For an external SGLang
    server: an isolated virtual environment that the launch command then uses (created once, reused afterwards). For the
    native engine: build the in-tree CUDA extensions of the checkout in ``workdir`` (a no-op when they are current)."""
    q = shlex.quote(workdir)
    if config.engine == "sglang":
        steps = ['export PATH="$HOME/.local/bin:$PATH"',
                 f'([ -d {SGLANG_VENV} ] && echo "using existing {SGLANG_VENV}") || uv venv {SGLANG_VENV} --python 3.10',
                 f". {SGLANG_VENV}/bin/activate",
                 'uv pip install "sglang[all]" --index-strategy unsafe-best-match',
                 "uv pip show sglang | grep -i '^version' || true"]
    else:
        steps = [f"cd {q}", f"{shlex.quote(sys.executable)} -m research_b200.cli build",
                 f"{shlex.quote(sys.executable)} -c 'import research_b200; print(\"research_b200 importable\")'"]
    return " && ".join(steps)


HttpGet = Callable[[str, dict[str, str]], int]          # url, headers -> HTTP status (raises OSError when unreachable)


def _urllib_status(url: str, headers: dict[str, str]) -> int:
    import urllib.error

    try:
        with urllib.request.urlopen(urllib.request.Request(url, headers=headers), timeout=10) as r:  # noqa: S310
            return r.status
    except urllib.error.HTTPError as e:
        return e.code


def check_model_access(model: str, env: dict[str, str] | None = None, get: HttpGet = _urllib_status) -> tuple[bool, str | None]:
    """Before a deployment that downloads a gated checkpoint: is ``HF_TOKEN`` set, is ``model`` an ``org/name`` id, and does
    the hub let this token see it (rollouts/deploy.py:165-233)? A local directory or a built-in preset needs no token. A
    hub that cannot be reached is a warning, not a refusal: ``(True, "could not verify ...")``."""
    import os

    if Path(model).exists():
        return True, None
    try:
        from .models.config import get_preset

        get_preset(model)
        return True, None
    except (KeyError, AssertionError, ValueError):
        pass
    token = (os.environ if env is None else env).get("HF_TOKEN", "")
    if not token:
        return False, "HF_TOKEN is not set: export HF_TOKEN=hf_... (needed to download the checkpoint)"
    if "/" not in model:
        return False, f"{model!r} is neither a local directory, a built-in preset, nor an 'org/name' model id"
    try:
        status = get(f"https://huggingface.co/api/models/{model}", {"Authorization": f"Bearer {token}"})
    except OSError as e:
        return True, f"could not verify access to {model}: {e}"
    if status == 200:
        return True, None
    return False, {401: "HF_TOKEN is invalid or expired: create a new one at https://huggingface.co/settings/tokens",
                   403: f"access to {model} is denied: accept the model's licence on its hub page with this account",
                   404: f"model not found: {model} (check the name, and that this account may see it)"}.get(
                       status, f"the hub answered HTTP {status} for {model}")


def server_info_to_endpoint(info: ServerInfo, model: str, engine: str = "native", **kw):
    """The ``Endpoint`` agents use to talk to a launched server (OpenAI-compatible routes under ``/v1``)."""
    from .agents.dtypes import Endpoint

    return Endpoint(provider="sglang" if engine == "sglang" else "openai", model=model, api_base=info.url, **kw)


def build_command(config: ServerConfig) -> str:
    env = f"CUDA_VISIBLE_DEVICES={','.join(map(str, config.gpu_ranks))} "
    if config.engine == "sglang":
        return f"([ -d {SGLANG_VENV} ] && . {SGLANG_VENV}/bin/activate); {env}" + build_sglang_command(config)
    return env + build_native_command(config)


def local_runner(cmd: str) -> tuple[int, str]:
    p = subprocess.run(cmd, shell=True, capture_output=True, text=True)
    return p.returncode, (p.stdout + p.stderr).strip()


def ssh_runner(connection: str, key: str | None = None) -> Runner:
    host, _, port = connection.partition(":")
    base = ["ssh", "-o", "BatchMode=yes", "-o", "StrictHostKeyChecking=accept-new"] + (["-p", port] if port else []) + (["-i", key] if key else [])

    def run(cmd: str) -> tuple[int, str]:
        p = subprocess.run(base + [host, cmd], capture_output=True, text=True)
        return p.returncode, (p.stdout + p.stderr).strip()

    return run


def preflight(config: ServerConfig, run: Runner = local_runner, max_used_mib: int = 2048) -> list[str]:
    """Problems that would make the launch fail; an empty list means go. Busy GPUs are reported, never freed."""
    problems = []
    rc, out = run("nvidia-smi --query-gpu=index,memory.used --format=csv,noheader,nounits")
    if rc != 0:
        problems.append(f"nvidia-smi failed: {out[:200]}")
    else:
        used = {}
        for line in out.splitlines():
            try:
                idx, mem = (int(x) for x in line.split(","))
                used[idx] = mem
            except ValueError:
                continue
        for g in config.gpu_ranks:
            if g not in used:
                problems.append(f"GPU {g} does not exist")
            elif used[g] > max_used_mib:
                problems.append(f"GPU {g} is busy ({used[g]} MiB in use); pick another GPU or wait")
    rc, out = run(f"(command -v ss >/dev/null && ss -ltn | grep -q ':{config.port} ') && echo taken || echo free")
    if "taken" in out:
        problems.append(f"port {config.port} is already in use")
    if config.engine == "sglang":
        rc, out = run("python -c 'import sglang'")
        if rc != 0:
            problems.append("sglang is not installed on the target")
    return problems


def wait_until_healthy(url: str, timeout: float = 600.0, alive: Callable[[], bool] | None = None, poll: float = 1.0,
                       probe: Callable[[str], bool] | None = None) -> bool:
    def http_ok(u: str) -> bool:
        try:
            with urllib.request.urlopen(u + "/health", timeout=2) as r:  # noqa: S310
                return r.status == 200
        except OSError:
            return False

    probe = probe or http_ok
    deadline = time.monotonic() + timeout
    while time.monotonic() < deadline:
        if probe(url):
            return True
        if alive is not None and not alive():
            return False          # the child died: no point waiting for the timeout
        time.sleep(poll)
    return False


def deploy_server(config: ServerConfig, wait: bool = True, timeout: float = 600.0) -> ServerInfo:
    """Launch on this machine (remote launches go through ``ssh_runner`` + ``nohup`` of the same command)."""
    cmd = build_command(config)
    log_dir = Path(config.log_dir)
    log_dir.mkdir(parents=True, exist_ok=True)
    log_path = log_dir / f"{config.name}-{config.port}.log"
    if config.ssh_connection:
        run = ssh_runner(config.ssh_connection)
        rc, out = run(f"mkdir -p {shlex.quote(str(log_dir))} && nohup sh -c {shlex.quote(cmd)} > {shlex.quote(str(log_path))} 2>&1 & echo $!")
        if rc != 0:
            raise RuntimeError(f"remote launch failed: {out}")
        pid, alive = int(out.split()[-1]), None
    else:
        logf = open(log_path, "w")
        proc = subprocess.Popen(cmd, shell=True, stdout=logf, stderr=subprocess.STDOUT, start_new_session=True)
        pid, alive = proc.pid, (lambda: proc.poll() is None)
    if wait and not wait_until_healthy(config.url, timeout, alive):
        if config.ssh_connection:
            tail = ssh_runner(config.ssh_connection)(f"tail -c 2000 {shlex.quote(str(log_path))}")[1]
        else:
            tail = log_path.read_text()[-2000:] if log_path.exists() else ""
        raise RuntimeError(f"server did not become healthy at {config.url}\n--- log tail ---\n{tail}")
    return ServerInfo(config.url, pid, str(log_path), cmd)
