"""A local experiment tracker: ``log()`` calls append to a run's ``metrics.jsonl``, a viewer draws the runs of a
directory as braille line charts in the terminal and compares their latest values.

The design is the one the reference writes down for its "wandb at home" (rollouts/docs/EXPERIMENT_TRACKER.md:16-135):
a run is a directory ``<dir>/<run id>/`` with ``meta.json`` (name, config, git commit, start and end time) and an
append-only ``metrics.jsonl`` whose records carry ``_step`` and ``_timestamp``; optional ``system.jsonl`` records hold
machine readings. The viewer here is a function from files to text (``render``), which ``watch`` repeats; selection is
by arguments rather than by keys, so it works in a pipe and under test.

``Tracker`` has the ``log(metrics, step)`` / ``finish()`` surface of the training loops' metric sinks, so it can be passed
wherever a ``training.metrics.MetricsLogger`` is expected.

    tracker = Tracker("my-experiment", config={"lr": 3e-4})
    tracker.log({"loss": 2.3})
    tracker.finish()
    python -m research_b200.utils.tracker runs/ --metric loss
"""

from __future__ import annotations

import argparse
import json
import math
import os
import secrets
import subprocess
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable


def _git_commit() -> str | None:
    try:
        out = subprocess.run(["git", "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5)
        return out.stdout.strip() or None if out.returncode == 0 else None
    except (OSError, subprocess.SubprocessError):
        return None


class Tracker:
    def __init__(self, name: str, config: dict[str, Any] | None = None, dir: str | Path = "./runs", run_id: str | None = None,
                 clock: Callable[[], float] = time.time):
        self.clock = clock
        self.run_id = run_id or f"run-{time.strftime('%Y%m%d-%H%M%S', time.gmtime(clock()))}-{secrets.token_hex(3)}"
        self.path = Path(dir) / self.run_id
        self.path.mkdir(parents=True, exist_ok=True)
        self._step = -1
        self.meta = {"name": name, "run_id": self.run_id, "config": config or {}, "git_hash": _git_commit(),
                     "started_at": clock(), "finished_at": None, "status": "running"}
        self._write_meta()
        self._metrics = open(self.path / "metrics.jsonl", "a", buffering=1)      # line-buffered: a viewer sees every record at once

    def _write_meta(self) -> None:
        tmp = self.path / "meta.json.tmp"
        tmp.write_text(json.dumps(self.meta, indent=2, default=str))
        os.replace(tmp, self.path / "meta.json")

    def log(self, data: dict[str, Any], step: int | None = None) -> int:
        """Append one record; without ``step`` the run's counter advances by one. Values that JSON cannot hold (tensors,
        numpy scalars) are converted with ``float`` where that works, else ``str``."""
        self._step = self._step + 1 if step is None else int(step)
        rec: dict[str, Any] = {"_step": self._step, "_timestamp": self.clock()}
        for k, v in data.items():
            if isinstance(v, (bool, int, float, str)) or v is None:
                rec[k] = v
            else:
                try:
                    rec[k] = float(v)
                except (TypeError, ValueError):
                    rec[k] = str(v)
        self._metrics.write(json.dumps(rec) + "\n")
        return self._step

    def log_system(self, readings: dict[str, Any] | None = None) -> dict[str, Any]:
        """Machine readings beside the metrics: given ones, else load average and resident memory of this process."""
        if readings is None:
            readings = {"load_1m": os.getloadavg()[0]}
            try:
                with open("/proc/self/statm") as f:
                    readings["rss_mb"] = int(f.read().split()[1]) * os.sysconf("SC_PAGE_SIZE") / 2**20
            except (OSError, ValueError, IndexError):
                pass
        rec = {"_step": self._step, "_timestamp": self.clock(), **readings}
        with open(self.path / "system.jsonl", "a") as f:
            f.write(json.dumps(rec) + "\n")
        return rec

    def finish(self, status: str = "finished") -> None:
        if not self._metrics.closed:
            self._metrics.close()
        self.meta.update(finished_at=self.clock(), status=status)
        self._write_meta()

    def __enter__(self) -> "Tracker":
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        self.finish("failed" if exc_type is not None else "finished")


# ------------------------------------------------------------------------------------------------- reading
@dataclass
class Run:
    run_id: str
    path: Path
    meta: dict[str, Any]
    records: list[dict[str, Any]] = field(default_factory=list)

    def series(self, metric: str) -> tuple[list[float], list[float]]:
        """(steps, values) of the records that carry a finite number under ``metric``."""
        xs, ys = [], []
        for r in self.records:
            v = r.get(metric)
            if isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(v):
                xs.append(float(r.get("_step", len(xs))))
                ys.append(float(v))
        return xs, ys

    def metrics(self) -> list[str]:
        seen: dict[str, None] = {}
        for r in self.records:
            for k, v in r.items():
                if not k.startswith("_") and isinstance(v, (int, float)) and not isinstance(v, bool):
                    seen.setdefault(k)
        return list(seen)

    def latest(self, metric: str) -> float | None:
        ys = self.series(metric)[1]
        return ys[-1] if ys else None


def load_run(path: str | Path) -> Run:
    path = Path(path)
    meta_file = path / "meta.json"
    meta = json.loads(meta_file.read_text()) if meta_file.exists() else {"name": path.name, "run_id": path.name}
    records = []
    metrics_file = path / "metrics.jsonl"
    if metrics_file.exists():
        for line in metrics_file.read_text().splitlines():
            try:
                records.append(json.loads(line))
            except json.JSONDecodeError:
                continue                                   # a line that is being written right now
    return Run(meta.get("run_id", path.name), path, meta, records)


def list_runs(directory: str | Path) -> list[Run]:
    """Runs of a directory, oldest first; the directory itself if it is a run."""
    directory = Path(directory)
    if (directory / "metrics.jsonl").exists():
        return [load_run(directory)]
    runs = [load_run(p) for p in sorted(directory.iterdir()) if p.is_dir() and (p / "metrics.jsonl").exists()] if directory.is_dir() else []
    return sorted(runs, key=lambda r: r.meta.get("started_at") or 0)


# ------------------------------------------------------------------------------------------------- drawing
_DOT = ((0x01, 0x08), (0x02, 0x10), (0x04, 0x20), (0x40, 0x80))      # braille dot bits by (row 0-3, column 0-1) of a cell
SERIES_COLOURS = ("\x1b[36m", "\x1b[33m", "\x1b[35m", "\x1b[32m", "\x1b[31m", "\x1b[34m")


def braille_chart(series: list[tuple[list[float], list[float]]], width: int = 60, height: int = 10, colour: bool = False) -> list[str]:
    """Line chart of one or more (xs, ys) series on a shared scale, ``height`` text rows of ``width`` braille cells
    (2 x 4 dots each), with the y range on the left of the first and last row. Consecutive points are joined by
    straight segments so that sparse series still read as lines."""
    pts = [(x, y) for xs, ys in series for x, y in zip(xs, ys)]
    if not pts:
        return ["(no data)"]
    x0, x1 = min(p[0] for p in pts), max(p[0] for p in pts)
    y0, y1 = min(p[1] for p in pts), max(p[1] for p in pts)
    if y1 == y0:
        y0, y1 = y0 - 0.5, y1 + 0.5
    w, h = width * 2, height * 4
    cells = [[0] * width for _ in range(height)]
    owner = [[-1] * width for _ in range(height)]

    def px(x: float, y: float) -> tuple[int, int]:
        cx = 0 if x1 == x0 else round((x - x0) / (x1 - x0) * (w - 1))
        return cx, round((y1 - y) / (y1 - y0) * (h - 1))

    def dot(cx: int, cy: int, who: int) -> None:
        cells[cy // 4][cx // 2] |= _DOT[cy % 4][cx % 2]
        owner[cy // 4][cx // 2] = who

    for who, (xs, ys) in enumerate(series):
        prev = None
        for x, y in zip(xs, ys):
            cx, cy = px(x, y)
            if prev is None:
                dot(cx, cy, who)
            else:
                n = max(abs(cx - prev[0]), abs(cy - prev[1]), 1)
                for i in range(1, n + 1):
                    dot(prev[0] + round((cx - prev[0]) * i / n), prev[1] + round((cy - prev[1]) * i / n), who)
            prev = (cx, cy)
    labels = [f"{y1:.4g}", f"{y0:.4g}"]
    pad = max(len(s) for s in labels)
    rows = []
    for r in range(height):
        label = labels[0] if r == 0 else labels[1] if r == height - 1 else ""
        if colour:
            body = "".join((SERIES_COLOURS[owner[r][c] % len(SERIES_COLOURS)] + chr(0x2800 + cells[r][c]) + "\x1b[0m") if cells[r][c] else " "
                           for c in range(width))
        else:
            body = "".join(chr(0x2800 + v) if v else " " for v in cells[r])
        rows.append(f"{label:>{pad}} |{body}")
    rows.append(f"{'':>{pad}} +{'-' * width}")
    rows.append(f"{'':>{pad}}  {x0:<.6g}{'step':^{max(width - 16, 4)}}{x1:>.6g}")
    return rows


def render(directory: str | Path, metrics: list[str] | None = None, run_filter: str | None = None, width: int = 60, height: int = 10,
           colour: bool = False, max_runs: int = 6) -> str:
    """Everything the viewer shows, as text: the run list (newest last, ``*`` = still running), a table of the latest
    value of every metric per run, and one chart per requested metric (default: the first three) with all runs overlaid."""
    runs = [r for r in list_runs(directory) if not run_filter or run_filter in r.run_id or run_filter in str(r.meta.get("name", ""))]
    if not runs:
        return f"no runs under {directory}"
    runs = runs[-max_runs:]
    names = list(dict.fromkeys(m for r in runs for m in r.metrics()))
    out = ["runs:"]
    for i, r in enumerate(runs):
        tag = SERIES_COLOURS[i % len(SERIES_COLOURS)] + "--" + "\x1b[0m" if colour else f"[{i}]"
        live = "*" if r.meta.get("finished_at") is None else " "
        out.append(f"  {tag} {live} {r.run_id}  {r.meta.get('name', '')}  {len(r.records)} records  {r.meta.get('status', '')}  "
                   f"{json.dumps(r.meta.get('config', {}))[:60]}")
    if names:
        head = f"{'metric':<24}" + "".join(f"{('[' + str(i) + ']'):>14}" for i in range(len(runs)))
        out += ["", "latest:", "  " + head]
        for m in names:
            vals = [r.latest(m) for r in runs]
            out.append("  " + f"{m:<24}" + "".join(f"{(f'{v:.5g}' if v is not None else '-'):>14}" for v in vals))
    for m in (metrics or names[:3]):
        if m not in names:
            out += ["", f"{m}: no run has it"]
            continue
        out += ["", m] + braille_chart([r.series(m) for r in runs], width, height, colour)
    return "\n".join(out)


def watch(directory: str | Path, interval: float = 2.0, out=None, iterations: int | None = None, sleep=time.sleep, **kw) -> None:
    """Redraw ``render`` until interrupted (or ``iterations`` times); only when some file of the runs changed."""
    out = out or sys.stdout
    last, n = None, 0
    while iterations is None or n < iterations:
        stamp = tuple(sorted((str(p), p.stat().st_mtime_ns) for p in Path(directory).rglob("*.json*")))
        if stamp != last:
            out.write("\x1b[2J\x1b[H" + render(directory, **kw) + "\n")
            out.flush()
            last = stamp
        n += 1
        if iterations is None or n < iterations:
            sleep(interval)


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="track", description="terminal view of the runs a Tracker wrote")
    ap.add_argument("path", nargs="?", default="./runs", help="a directory of runs, or one run")
    ap.add_argument("--metric", action="append", help="chart this metric (repeatable; default: the first three)")
    ap.add_argument("--run", help="only runs whose id or name contains this")
    ap.add_argument("--width", type=int, default=60)
    ap.add_argument("--height", type=int, default=10)
    ap.add_argument("--watch", action="store_true", help="keep redrawing as the files grow")
    ap.add_argument("--no-colour", action="store_true")
    args = ap.parse_args(argv)
    kw = dict(metrics=args.metric, run_filter=args.run, width=args.width, height=args.height, colour=sys.stdout.isatty() and not args.no_colour)
    if args.watch:
        try:
            watch(args.path, **kw)
        except KeyboardInterrupt:
            pass
        return 0
    print(render(args.path, **kw))
    return 0


if __name__ == "__main__":
    sys.exit(main())
