"""Run an experiment on a rented (or given) machine from start to finish, and many of them side by side.

One deployment is the sequence the reference repeats in every ``dev/*/deploy.py`` (dev/outlier-features/deploy.py:153-660,
dev/corpus-proximity/deploy.py, dev/integration_training/deploy.py): find a machine with enough memory, wait for ssh,
ship the repository's commit, start the run detached, poll it (job state plus optional marker files the run writes),
bring the result files back, and give the machine back unless asked to keep it. Here it is one function over the
package's own pieces (``broker.GPUClient``, ``bifrost.RemoteClient``), described by a ``DeployJob`` value that a config
file exports as ``job``.

A sweep starts one deployment per config file, each as its own child process with its own log, staggered so that the
providers' APIs are not hit at once, and ``sweep_status`` shows the state and last log lines of each
(dev/outlier-features/deploy_sweep.py:31-324).

    python -m research_b200.infra.experiment_deploy run configs/01_small.py --ssh user@host
    python -m research_b200.infra.experiment_deploy sweep configs/ --only 01 03 --dry-run
    python -m research_b200.infra.experiment_deploy status sweep_logs/
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable

from .bifrost import GPUQuery, ProcessSpec, RemoteClient, acquire_node, generate_job_name, subprocess_transport


@dataclass(frozen=True)
class DeployJob:
    name: str
    command: str                                    # run inside the pushed checkout
    repo: str = "."
    dest: str = ""                                  # remote directory; default ~/experiments/<name>
    env: dict[str, str] = field(default_factory=dict)
    bootstrap: str | None = "auto"                  # dependency set-up after the push ("auto": detected from the checkout)
    results: tuple[str, ...] = ()                   # paths under ``dest`` to bring back
    local_results: str = "remote_results"
    gpu: GPUQuery | None = None                     # what to rent when no machine is given
    success_marker: str | None = None               # files (under ``dest``) the run itself writes when it is done
    failure_marker: str | None = None
    timeout_s: float = 6 * 3600.0
    poll_s: float = 30.0
    keep_running: bool = False

    def remote_dir(self) -> str:
        return self.dest or f"~/experiments/{self.name}"


@dataclass
class DeployOutcome:
    name: str
    ok: bool
    stage: str                                      # the last stage reached: provision | push | start | wait | sync | done
    commit: str | None = None
    instance_id: str | None = None
    exit_code: int | None = None
    fetched: dict[str, int] = field(default_factory=dict)      # result path -> files brought back
    not_shipped: list[str] = field(default_factory=list)
    log_tail: str = ""
    error: str | None = None
    seconds: float = 0.0
    terminated: bool = False


def load_job(path: str | Path) -> DeployJob:
    """A config file is Python that leaves a ``DeployJob`` in ``job`` (or a function ``make_job()`` that returns one)."""
    path = Path(path)
    scope: dict[str, Any] = {"__file__": str(path), "__name__": f"deploy_config_{path.stem}"}
    exec(compile(path.read_text(), str(path), "exec"), scope)       # noqa: S102 - the user's own config file
    job = scope.get("job") or (scope["make_job"]() if callable(scope.get("make_job")) else None)
    if not isinstance(job, DeployJob):
        raise ValueError(f"{path} defines neither `job` nor `make_job()` giving a DeployJob")
    return job


def deploy_experiment(job: DeployJob, ssh: str | None = None, gpu_client: Any = None, key: str | None = None,
                      transport=subprocess_transport, log: Callable[[str], None] = print,
                      sleep: Callable[[float], None] = time.sleep) -> DeployOutcome:
    """The whole life of one remote run. Every failure is reported in the outcome (with the stage it happened at) rather
    than raised, and a machine that this call rented is given back on every path unless ``keep_running``."""
    t0 = time.monotonic()
    out = DeployOutcome(job.name, False, "provision")
    client: RemoteClient | None = None
    inst = None
    try:
        if ssh is not None:
            client, inst = acquire_node(ssh=ssh, key=key, transport=transport, ssh_timeout=60.0, poll=1.0)
        else:
            if gpu_client is None or job.gpu is None:
                raise ValueError("give an ssh target, or a gpu_client together with job.gpu")
            log(f"[{job.name}] looking for {job.gpu.count}x {job.gpu.type}" + (f" with >= {job.gpu.min_vram_gb} GB" if job.gpu.min_vram_gb else ""))
            client, inst = acquire_node(provision=job.gpu, gpu_client=gpu_client, key=key, transport=transport)
            out.instance_id = inst.instance_id
            log(f"[{job.name}] instance {inst.instance_id} answers on {inst.ssh_connection}")
        dest = job.remote_dir()

        out.stage = "push"
        out.commit = client.push(job.repo, dest, bootstrap=job.bootstrap, warn=lambda m: log(f"[{job.name}] warning: {m}"))
        out.not_shipped = list(getattr(client, "not_shipped", []))
        log(f"[{job.name}] commit {out.commit[:10]} is at {dest}")

        out.stage = "start"
        run_name = generate_job_name(job.name.replace("_", "-").replace(".", "-")[:24] or "run")
        import shlex

        markers = " ".join(shlex.quote(m) for m in (job.success_marker, job.failure_marker) if m)    # relative to the checkout, the job's cwd
        command = (f"rm -f {markers}; " if markers else "") + job.command
        client.start_job(ProcessSpec(command, cwd=client.expand_path(dest), env=dict(job.env), name=run_name))
        log(f"[{job.name}] started as job {run_name}")

        out.stage = "wait"
        deadline = time.monotonic() + job.timeout_s
        finished = False
        while True:
            info = client.job_status(run_name)
            if job.failure_marker and client.path_exists(f"{dest}/{job.failure_marker}"):
                out.error, finished = f"the run wrote {job.failure_marker}", True
            elif job.success_marker and client.path_exists(f"{dest}/{job.success_marker}"):
                finished = True
            elif info.status != "running":
                out.exit_code, finished = info.exit_code, True
                if info.exit_code != 0:
                    out.error = f"the run exited with code {info.exit_code}" if info.exit_code is not None else "the run disappeared without an exit code"
                elif job.success_marker:
                    out.error = f"the run exited without writing {job.success_marker}"
            if finished:
                break
            if time.monotonic() > deadline:
                out.error = f"still running after {job.timeout_s:.0f}s"
                client.stop_job(run_name)
                break
            sleep(job.poll_s)
        out.log_tail = client.job_logs(run_name, tail=40)

        out.stage = "sync"                           # also after a failure: partial results and logs are worth having
        local_root = Path(job.local_results) / job.name
        for rel in job.results:
            remote = f"{dest}/{rel}"
            if not client.path_exists(remote):
                log(f"[{job.name}] no {rel} on the machine")
                continue
            local_root.mkdir(parents=True, exist_ok=True)
            out.fetched[rel] = client.download(remote, local_root / Path(rel).name)
        if out.log_tail:
            local_root.mkdir(parents=True, exist_ok=True)
            (local_root / "run.log.tail").write_text(out.log_tail)

        if out.error is None:
            out.ok, out.stage = True, "done"
    except Exception as e:  # noqa: BLE001 - reported with its stage; the machine is released below
        out.error = f"{type(e).__name__}: {e}"
    finally:
        if inst is not None and ssh is None and gpu_client is not None:
            if job.keep_running:
                log(f"[{job.name}] instance {inst.instance_id} left running ({inst.ssh_connection})")
            else:
                try:
                    out.terminated = bool(gpu_client.terminate(inst.instance_id))
                except Exception as e:  # noqa: BLE001
                    log(f"[{job.name}] could NOT terminate {inst.instance_id}: {e} - terminate it by hand")
        out.seconds = time.monotonic() - t0
    log(f"[{job.name}] {'ok' if out.ok else 'FAILED at ' + out.stage + ': ' + str(out.error)} after {out.seconds:.0f}s")
    return out


# ------------------------------------------------------------------------------------------------- sweeps
def discover_configs(config_dir: str | Path, only: list[str] | None = None) -> list[Path]:
    """The ``*.py`` files of a directory in name order; ``only`` keeps those whose name starts with one of the prefixes
    (configs are numbered ``01_...``, ``02_...`` so that ``--only 01 03`` picks two of them)."""
    found = sorted(p for p in Path(config_dir).glob("*.py") if not p.name.startswith("_"))
    if only:
        found = [p for p in found if any(p.name.startswith(prefix) for prefix in only)]
    return found


def display_name(config: Path) -> str:
    stem = config.stem
    head, _, rest = stem.partition("_")
    return (rest if head.isdigit() and rest else stem).replace("_", "-")


def launch_sweep(configs: list[Path], log_dir: str | Path, extra_args: list[str] | None = None, stagger_s: float = 5.0,
                 dry_run: bool = False, python: str | None = None, sleep: Callable[[float], None] = time.sleep) -> dict[str, Any]:
    """One child process per config (``... experiment_deploy run <config>``), output to ``<log_dir>/<stem>.log``; the
    process ids are written to ``<log_dir>/sweep.json`` for ``sweep_status``. The children are not waited for: a sweep
    runs for hours and outlives this call."""
    log_dir = Path(log_dir)
    plan = [{"config": str(c), "name": display_name(c), "log": str(log_dir / f"{c.stem}.log"), "outcome": str(log_dir / f"{c.stem}.outcome.json")}
            for c in configs]
    if dry_run:
        return {"started_at": None, "runs": plan}
    log_dir.mkdir(parents=True, exist_ok=True)
    for i, run in enumerate(plan):
        argv = [python or sys.executable, "-m", "research_b200.infra.experiment_deploy", "run", run["config"], "--outcome", run["outcome"],
                *(extra_args or [])]
        with open(run["log"], "w") as f:
            proc = subprocess.Popen(argv, stdout=f, stderr=subprocess.STDOUT, start_new_session=True)
        run["pid"] = proc.pid
        if i + 1 < len(plan):
            sleep(stagger_s)
    record = {"started_at": time.time(), "runs": plan}
    (log_dir / "sweep.json").write_text(json.dumps(record, indent=2))
    return record


def _alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    try:                                            # a finished child that nobody reaped yet still answers signal 0
        with open(f"/proc/{pid}/stat") as f:
            return f.read().rsplit(")", 1)[1].split()[0] != "Z"
    except OSError:
        return True


def sweep_status(log_dir: str | Path, lines: int = 5) -> list[dict[str, Any]]:
    """State of every run of a sweep: ``running`` / ``ok`` / ``failed`` / ``died`` (the process is gone and left no
    outcome), with the last lines of its log."""
    log_dir = Path(log_dir)
    record = json.loads((log_dir / "sweep.json").read_text())
    rows = []
    for run in record["runs"]:
        outcome_path, log_path = Path(run["outcome"]), Path(run["log"])
        outcome = json.loads(outcome_path.read_text()) if outcome_path.exists() else None
        if outcome is not None:
            state = "ok" if outcome.get("ok") else "failed"
        else:
            state = "running" if _alive(int(run.get("pid", -1))) else "died"
        tail = log_path.read_text(errors="replace").splitlines()[-lines:] if log_path.exists() else []
        rows.append({"name": run["name"], "state": state, "pid": run.get("pid"), "stage": (outcome or {}).get("stage"),
                     "error": (outcome or {}).get("error"), "tail": tail})
    return rows


def format_status(rows: list[dict[str, Any]]) -> str:
    out = []
    for r in rows:
        out.append(f"{r['name']:<28} {r['state']:<8} " + (f"{r['stage']}: {r['error']}" if r["state"] == "failed" else ""))
        out.extend(f"    {line}" for line in r["tail"])
    counts = {s: sum(r["state"] == s for r in rows) for s in ("running", "ok", "failed", "died")}
    out.append("  ".join(f"{n} {s}" for s, n in counts.items() if n))
    return "\n".join(out)


# ------------------------------------------------------------------------------------------------- command line
def _gpu_client():
    from .broker import GPUClient
    from .broker_providers import providers_from_env

    return GPUClient(providers_from_env(), registry=os.path.expanduser("~/.research_b200/instances.json"))


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="experiment_deploy", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    run = sub.add_parser("run", help="one config, start to finish")
    run.add_argument("config")
    run.add_argument("--ssh", help="use this machine instead of renting one")
    run.add_argument("--key")
    run.add_argument("--keep-running", action="store_true")
    run.add_argument("--outcome", help="write the outcome as JSON here")
    sw = sub.add_parser("sweep", help="one deployment per config file of a directory, side by side")
    sw.add_argument("config_dir")
    sw.add_argument("--only", nargs="*", help="name prefixes to keep (01 03 ...)")
    sw.add_argument("--log-dir", default="sweep_logs")
    sw.add_argument("--stagger", type=float, default=5.0)
    sw.add_argument("--dry-run", action="store_true")
    sw.add_argument("--ssh")
    sw.add_argument("--keep-running", action="store_true")
    st = sub.add_parser("status", help="state and last log lines of a sweep's runs")
    st.add_argument("log_dir")
    st.add_argument("--lines", type=int, default=5)
    args = ap.parse_args(argv)

    if args.cmd == "run":
        job = load_job(args.config)
        if args.keep_running:
            from dataclasses import replace

            job = replace(job, keep_running=True)
        outcome = deploy_experiment(job, ssh=args.ssh, gpu_client=None if args.ssh else _gpu_client(), key=args.key)
        if args.outcome:
            Path(args.outcome).write_text(json.dumps(asdict(outcome), indent=2))
        return 0 if outcome.ok else 1
    if args.cmd == "sweep":
        configs = discover_configs(args.config_dir, args.only)
        if not configs:
            print(f"no configs in {args.config_dir}")
            return 1
        extra = (["--ssh", args.ssh] if args.ssh else []) + (["--keep-running"] if args.keep_running else [])
        record = launch_sweep(configs, args.log_dir, extra_args=extra, stagger_s=args.stagger, dry_run=args.dry_run)
        for r in record["runs"]:
            print(f"{'would start' if args.dry_run else 'started'} {r['name']:<28} {r['config']}" + (f"  pid {r['pid']}" if "pid" in r else ""))
        if not args.dry_run:
            print(f"logs in {args.log_dir}; `experiment_deploy status {args.log_dir}` shows progress")
        return 0
    print(format_status(sweep_status(args.log_dir, args.lines)))
    return 0


if __name__ == "__main__":
    # run through the importable module: a config file's ``DeployJob`` is that module's class, not ``__main__``'s copy
    from research_b200.infra.experiment_deploy import main as _main

    sys.exit(_main())
