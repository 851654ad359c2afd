"""Dataset evaluation: run an agent per sample with bounded concurrency and sample-level retry, score the trajectory,
write a report that can be resumed (rollouts/evaluation.py:130-994).

What a run leaves in ``<output_dir>/<eval_name>/``: ``report.json`` (summary metrics, configuration with API keys
redacted, the ids of the samples), ``samples/<id>.json`` and ``trajectories/<id>.jsonl`` per sample, and
``samples.jsonl`` with everything in one file. ``evaluate(..., resume=True)`` reads the per-sample files back and
runs only the samples that are missing or ended in a provider error.

A sample ends in one of three states (``metadata["status"]``): ``success`` (the agent ran and was scored),
``failed`` (the agent, the environment or the scorer raised) and ``provider_error`` (the model endpoint kept failing:
rate limits, time-outs). Provider errors are not the model's fault, so ``success_rate`` leaves them out of its
denominator while ``completion_rate`` counts them as failures (rollouts/evaluation.py:763-869)."""

from __future__ import annotations

import asyncio
import json
import statistics
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterable, Iterator

from .agents import run_agent
from .dtypes import Actor, AgentState, EvalConfig, Message, Score, Trajectory
from .fingerprint import fingerprint_eval, warn_if_changed
from .providers.base import NonRetryableError, ProviderError


@dataclass
class EvalSample:
    sample_id: str
    input: dict[str, Any]
    trajectory: Trajectory
    score: Score
    stop_reason: str | None = None
    error: str | None = None
    attempts: int = 1
    duration_s: float = 0.0
    metadata: dict[str, Any] = field(default_factory=dict)

    @property
    def id(self) -> str:
        return self.sample_id

    @property
    def status(self) -> str:
        return self.metadata.get("status", "failed" if self.error else "success")

    def to_dict(self) -> dict[str, Any]:
        return {"sample_id": self.sample_id, "input": self.input, "trajectory": self.trajectory.to_dict(),
                "score": self.score.to_dict(), "stop_reason": self.stop_reason, "error": self.error,
                "attempts": self.attempts, "duration_s": self.duration_s, "metadata": self.metadata}

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "EvalSample":
        from .dtypes import Metric

        metrics = tuple(Metric(m["name"], float(m["value"]), float(m.get("weight", 0.0))) for m in d.get("score", {}).get("metrics", []))
        return EvalSample(str(d["sample_id"]), d.get("input", {}), Trajectory.from_dict(d.get("trajectory", {})), Score(metrics),
                          d.get("stop_reason"), d.get("error"), int(d.get("attempts", 1)), float(d.get("duration_s", 0.0)),
                          dict(d.get("metadata", {})))


_SECRET_KEYS = ("api_key", "apikey", "authorization", "token", "secret", "password")


def sanitize_api_keys(data: Any) -> Any:
    """Copy of a JSON-like structure with credentials blanked: any string under a key that names a credential
    (``api_key``, ``authorization``, ``token`` ...), and any string value that looks like a provider key (``sk-...``)."""
    if isinstance(data, dict):
        out = {}
        for k, v in data.items():
            if isinstance(v, str) and v and any(s in str(k).lower() for s in _SECRET_KEYS):
                out[k] = "***REDACTED***"
            else:
                out[k] = sanitize_api_keys(v)
        return out
    if isinstance(data, (list, tuple)):
        return [sanitize_api_keys(v) for v in data]
    if isinstance(data, str) and data.startswith("sk-") and len(data) > 12:
        return "***REDACTED***"
    return data


@dataclass
class EvalReport:
    eval_name: str
    samples: list[EvalSample]
    summary: dict[str, Any]
    config: dict[str, Any] = field(default_factory=dict)
    timestamp: float = field(default_factory=time.time)
    dataset_path: str = ""

    # names the reference's report uses
    @property
    def sample_results(self) -> list[EvalSample]:
        return self.samples

    @property
    def summary_metrics(self) -> dict[str, Any]:
        return self.summary

    @property
    def total_samples(self) -> int:
        return len(self.samples)

    def save(self, output_dir: str | Path) -> Path:
        d = Path(output_dir) / self.eval_name
        (d / "samples").mkdir(parents=True, exist_ok=True)
        (d / "trajectories").mkdir(exist_ok=True)
        (d / "report.json").write_text(json.dumps(sanitize_api_keys(
            {"eval_name": self.eval_name, "dataset_path": self.dataset_path, "summary": self.summary, "config": self.config,
             "timestamp": self.timestamp, "num_samples": len(self.samples), "sample_ids": [s.sample_id for s in self.samples]}),
            indent=2, default=str))
        with open(d / "samples.jsonl", "w") as f:
            for s in self.samples:
                row = sanitize_api_keys(s.to_dict())
                f.write(json.dumps(row, default=str) + "\n")
                name = _safe_name(s.sample_id)
                (d / "samples" / f"{name}.json").write_text(json.dumps(row, indent=2, default=str))
                Trajectory.save_jsonl([s.trajectory], d / "trajectories" / f"{name}.jsonl")
        Trajectory.save_jsonl([s.trajectory for s in self.samples], d / "trajectories.jsonl")
        return d

    @staticmethod
    def load(run_dir: str | Path) -> "EvalReport":
        """Read a saved run back (``run_dir`` is the folder that holds ``report.json``)."""
        d = Path(run_dir)
        meta = json.loads((d / "report.json").read_text())
        samples = load_saved_samples(d)
        order = {sid: i for i, sid in enumerate(meta.get("sample_ids", []))}
        samples.sort(key=lambda s: order.get(s.sample_id, len(order)))
        return EvalReport(meta["eval_name"], samples, meta.get("summary", {}), meta.get("config", {}), meta.get("timestamp", 0.0),
                          meta.get("dataset_path", ""))


def _safe_name(sample_id: str) -> str:
    return "".join(c if c.isalnum() or c in "-_." else "_" for c in str(sample_id)) or "sample"


def load_saved_samples(run_dir: str | Path) -> list[EvalSample]:
    d = Path(run_dir) / "samples"
    if not d.is_dir():
        return []
    out = []
    for f in sorted(d.glob("*.json")):
        try:
            out.append(EvalSample.from_dict(json.loads(f.read_text())))
        except (ValueError, KeyError):
            continue            # a file cut short by an interrupted run: the sample runs again
    return out


def _std(vals: list[float]) -> float:
    m = sum(vals) / len(vals)
    return (sum((v - m) ** 2 for v in vals) / len(vals)) ** 0.5


def compute_summary_metrics(samples: list[EvalSample]) -> dict[str, Any]:
    """mean / min / max / std of the reward and of every named metric, turn and token averages, the three outcome
    counts, ``success_rate`` (provider errors left out of the denominator), ``completion_rate`` (not left out), and the
    failures broken down by exception type and the provider errors by provider."""
    if not samples:
        return {"num_samples": 0.0}
    n = len(samples)
    rewards = [s.score.reward for s in samples]
    out: dict[str, Any] = {"num_samples": float(n), "total_samples": n, "mean_reward": statistics.fmean(rewards), "min_reward": min(rewards),
                           "max_reward": max(rewards), "std_reward": _std(rewards),
                           "mean_duration_s": statistics.fmean(s.duration_s for s in samples)}
    for name in sorted({m.name for s in samples for m in s.score.metrics}):
        vals = [m.value for s in samples for m in s.score.metrics if m.name == name]
        out[f"mean_{name}"], out[f"min_{name}"], out[f"max_{name}"], out[f"std_{name}"] = statistics.fmean(vals), min(vals), max(vals), _std(vals)
    out["avg_turns"] = sum(s.metadata.get("turns_used", 0) for s in samples) / n
    out["avg_tokens"] = sum(s.metadata.get("total_tokens", 0) for s in samples) / n
    provider = [s for s in samples if s.status == "provider_error"]
    failed = [s for s in samples if s.status == "failed"]
    ok = [s for s in samples if s.status == "success"]
    out["provider_errors"], out["failed_samples"], out["successful_samples"] = len(provider), len(failed), len(ok)
    out["error_rate"] = (len(provider) + len(failed)) / n
    out["success_rate"] = len(ok) / (n - len(provider)) if n > len(provider) else 0.0
    out["completion_rate"] = len(ok) / n
    kinds: dict[str, int] = {}
    for s in failed:
        kind = (s.error or "Unknown error").split(":")[0]
        kinds[kind] = kinds.get(kind, 0) + 1
    if kinds:
        out["error_breakdown"] = kinds
    by_provider: dict[str, int] = {}
    for s in provider:
        p = s.metadata.get("provider") or "unknown"
        by_provider[p] = by_provider.get(p, 0) + 1
    if by_provider:
        out["provider_error_breakdown"] = by_provider
    return out


class _SampleTimeout(Exception):
    pass


def _progress_status(event: Any) -> str | None:
    """What a sample is doing right now, from a stream event (shown beside its line of the progress display)."""
    t = getattr(event, "type", "")
    if t == "llm_call_start":
        return "waiting for the model"
    if t in ("text_delta", "thinking_delta"):
        return "streaming"
    if t == "tool_execution_start":
        return f"running {getattr(event, 'tool_name', 'tool')}"
    if t == "tool_result":
        return "tool done"
    return None


async def evaluate_sample(row: dict[str, Any], sample_id: str, config: EvalConfig, run_config: Any = None) -> EvalSample:
    """One agent run + scoring. Transient provider errors are retried with the configured delays; what is left after
    the last attempt is a ``provider_error`` sample. Any other exception makes a ``failed`` sample at once."""
    t0 = time.time()
    last_err: str | None = None
    status = "provider_error"
    attempts = 0
    failing_provider = ""
    for attempt in range(config.n_retries + 1):
        attempts = attempt + 1
        try:
            msgs = config.prepare_messages(row) if config.prepare_messages else [Message("user", str(row.get("prompt", row.get("question", ""))))]
            env = config.environment_factory(row) if config.environment_factory else None
            if asyncio.iscoroutine(env):
                env = await env
            state = AgentState(Actor(Trajectory(tuple(msgs)), config.endpoint), env, max_turns=config.max_turns)
            run = run_agent(state, run_config or config.run_config)
            try:
                states = await (asyncio.wait_for(run, config.sample_timeout_s) if config.sample_timeout_s else run)
            except asyncio.TimeoutError:
                if config.sample_timeout_s:          # the sample's own limit, not a provider's: no retry
                    raise _SampleTimeout(f"no result after {config.sample_timeout_s:g} s") from None
                raise
            final = states[-1]
            score = config.score_fn(final.actor.trajectory, row)
            if asyncio.iscoroutine(score):
                score = await score
            if not isinstance(score, Score):
                from .dtypes import Metric

                score = Score((Metric("reward", float(score), 1.0),))
            traj = final.actor.trajectory
            meta = {"status": "success", "turns_used": getattr(final, "turn_idx", len(traj.completions)),
                    "total_tokens": sum(c.usage.total_tokens for c in traj.completions)}
            return EvalSample(sample_id, row, traj, score, final.stop.value if final.stop else None, None, attempts,
                              time.time() - t0, meta)
        except NonRetryableError as e:
            last_err = f"{type(e).__name__}: {e}"
            break
        except _SampleTimeout as e:
            last_err, status = f"timeout: {e}", "failed"
            break
        except (ProviderError, asyncio.TimeoutError, ConnectionError) as e:
            last_err = f"{type(e).__name__}: {e}"
            failing_provider = getattr(e, "provider", "") or failing_provider
            if attempt < config.n_retries:
                await asyncio.sleep(config.retry_delays[min(attempt, len(config.retry_delays) - 1)])
        except Exception as e:   # noqa: BLE001 - a broken environment or scorer fails this sample, not the run
            last_err, status = f"{type(e).__name__}: {e}", "failed"
            break
    provider = failing_provider or getattr(config.endpoint, "provider", None)
    return EvalSample(sample_id, row, Trajectory(), Score(), None, last_err, attempts, time.time() - t0,
                      {"status": status, "provider": provider, "turns_used": 0, "total_tokens": 0})


def _fingerprint(config: EvalConfig, dataset_path: str) -> dict[str, Any] | None:
    """The run's fingerprint for the report (never a reason to fail a run: a dirty tree is recorded, and a scoring lambda,
    whose name identifies nothing, leaves the report without one)."""
    try:
        return fingerprint_eval(config, dataset_path=dataset_path or None, allow_dirty=True)
    except ValueError:
        return None


async def evaluate(dataset: Iterable[dict[str, Any]], config: EvalConfig, *, resume: bool = False,
                   on_sample_done: Callable[[EvalSample, int, int], None] | None = None, dataset_path: str = "") -> EvalReport:
    """Evaluate every row (``config.max_samples`` first rows) with at most ``config.max_concurrent`` agents in flight.

    ``resume``: samples already saved under ``config.output_dir`` are taken from disk unless they ended in a provider
    error. ``on_sample_done(sample, done, total)`` is called as samples finish (progress display, logging)."""
    rows = list(dataset)
    if config.max_samples is not None:
        rows = rows[:config.max_samples]
    ids = [str(r.get("id", i)) for i, r in enumerate(rows)]
    have: dict[str, EvalSample] = {}
    fp = _fingerprint(config, dataset_path)
    if resume and config.output_dir:
        run_dir = Path(config.output_dir) / config.eval_name
        have = {s.sample_id: s for s in load_saved_samples(run_dir) if s.status != "provider_error"}
        if fp is not None and (run_dir / "report.json").is_file():
            try:
                saved = json.loads((run_dir / "report.json").read_text()).get("config", {}).get("fingerprint")
            except (OSError, ValueError):
                saved = None
            warn_if_changed(saved, fp, context=f"the saved run {run_dir}")
    sem = asyncio.Semaphore(config.max_concurrent)
    done = 0
    finished: dict[str, EvalSample] = {}
    progress = None
    if config.show_progress:
        from .progress import MultiProgress

        progress = MultiProgress()
        progress.add_task(config.eval_name, total=len(rows))

    def sample_run_config(sid: str):
        """The run's ``RunConfig`` with the sample's status line fed from its stream events (the caller's own ``on_chunk`` still runs)."""
        if progress is None:
            return None
        from dataclasses import replace as _replace

        inner = config.run_config.on_chunk

        async def on_chunk(ev: Any) -> None:
            status = _progress_status(ev)
            if status and sid in progress.tasks:
                progress.update(sid, advance=0, message=status)
            if inner is not None:
                await inner(ev)

        return _replace(config.run_config, on_chunk=on_chunk)

    async def one(sid: str, row: dict[str, Any]) -> EvalSample:
        nonlocal done
        if sid in have:
            s = have[sid]
        else:
            async with sem:
                if progress is not None:
                    progress.add_task(sid)
                s = await evaluate_sample(row, sid, config, sample_run_config(sid))
                if progress is not None:
                    progress.finish(sid, "done" if s.status == "success" else "failed", s.error or f"reward {s.score.reward:.3g}")
                    progress.tasks.pop(sid, None)               # finished samples leave the display; the overall bar counts them
        finished[sid] = s
        done += 1
        if progress is not None:
            progress.update(config.eval_name, message=f"mean reward {sum(x.score.reward for x in finished.values()) / len(finished):.3f}")
        if on_sample_done is not None:
            on_sample_done(s, done, len(rows))
        return s

    def report_of(samples: list[EvalSample], interrupted: bool) -> EvalReport:
        cfg = {"endpoint": config.endpoint.to_dict(), "max_turns": config.max_turns, "max_concurrent": config.max_concurrent,
               "n_retries": config.n_retries, "resumed_samples": len(have), "fingerprint": fp}
        if interrupted:
            cfg.update(interrupted=True, planned_samples=len(rows))
        r = EvalReport(config.eval_name, samples, compute_summary_metrics(samples) if samples else {}, cfg, dataset_path=dataset_path)
        if config.output_dir:
            r.save(config.output_dir)
        return r

    tasks = [asyncio.ensure_future(one(sid, r)) for sid, r in zip(ids, rows)]
    try:
        samples = list(await asyncio.gather(*tasks))
    except (asyncio.CancelledError, KeyboardInterrupt):
        # interrupted: stop what is in flight, keep what finished (``resume=True`` picks the run up from there)
        for t in tasks:
            t.cancel()
        await asyncio.gather(*tasks, return_exceptions=True)
        report_of([finished[sid] for sid in ids if sid in finished], interrupted=True)
        raise
    finally:
        if progress is not None:
            progress.__exit__(None, None, None)
    return report_of(samples, interrupted=False)


def load_jsonl(path: str | Path) -> Iterator[dict[str, Any]]:
    with open(path) as f:
        for line in f:
            if line.strip():
                yield json.loads(line)


def load_csv(path: str | Path) -> Iterator[dict[str, Any]]:
    import csv

    with open(path, newline="") as f:
        for row in csv.DictReader(f):
            yield dict(row)


async def simple_evaluate(dataset_path: str | Path, config: EvalConfig, **kw) -> EvalReport:
    """``evaluate`` on a ``.jsonl`` / ``.json`` / ``.csv`` file (rollouts/evaluation.py:891-926)."""
    p = Path(dataset_path)
    if p.suffix == ".jsonl":
        rows: Iterable[dict[str, Any]] = load_jsonl(p)
    elif p.suffix == ".csv":
        rows = load_csv(p)
    elif p.suffix == ".json":
        rows = json.loads(p.read_text())
    else:
        raise ValueError(f"unsupported dataset format: {p.suffix}")
    return await evaluate(rows, config, dataset_path=str(p), **kw)


def group_by(samples: list[EvalSample], key: Callable[[EvalSample], Any]) -> dict[Any, list[EvalSample]]:
    out: dict[Any, list[EvalSample]] = {}
    for s in samples:
        out.setdefault(key(s), []).append(s)
    return out


def summarize(groups):
    """For a dict of groups (``group_by``): the summary metrics of each group. For a plain list of samples: mean, std,
    min, max and n of the reward (rollouts/evaluation.py:957-994)."""
    if isinstance(groups, dict):
        return {k: compute_summary_metrics(v) for k, v in groups.items()}
    rewards = [s.score.reward for s in groups]
    if not rewards:
        return {"mean": 0.0, "std": 0.0, "min": 0.0, "max": 0.0, "n": 0}
    return {"mean": statistics.fmean(rewards), "std": _std(rewards), "min": min(rewards), "max": max(rewards), "n": len(rewards)}


_ = asdict
