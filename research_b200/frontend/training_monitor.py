"""Multi-pane terminal monitor for a training run (rollouts/rollouts/tui/monitor.py:91-877): a unified JSONL log stream
(one JSON object per line, as ``utils/logging_config.JSONFormatter`` writes them; plain text lines are accepted too) is
routed by logger name into panes, numeric fields are collected into series for a sparkline pane, and vim-style keys
move around:

    1 / 2 / 3 / 4   training | engine | metrics | all      j / k   scroll (metrics pane: next / previous chart)
    g / G           top / bottom (G re-enables follow)     h / l   scroll sideways        q   quit

    tail -f run/training.jsonl | python -m research_b200.frontend.training_monitor
    python -m research_b200.frontend.training_monitor --replay results/rl/grpo_20250101-120000

``--replay`` reads a finished run's directory (``training.log`` / ``*.jsonl`` / ``metrics.jsonl``) instead of stdin.
Rendering is a pure function of the monitor state (``render(width, height) -> list[str]``), so it is testable
without a terminal; ``run`` adds the raw-mode input loop on a tty.
"""

from __future__ import annotations

import argparse
import json
import os
import select
import sys
from collections import deque
from dataclasses import dataclass, field
from pathlib import Path
from typing import Iterable

from ..utils.monitor import sparkline

DIM, CYAN, GREEN, YELLOW, RED, BOLD, RESET, INVERSE = "\x1b[90m", "\x1b[36m", "\x1b[32m", "\x1b[33m", "\x1b[31m", "\x1b[1m", "\x1b[0m", "\x1b[7m"
LEVEL_COLOR = {"DEBUG": DIM, "INFO": "", "WARNING": YELLOW, "ERROR": RED, "CRITICAL": RED + BOLD}
_STANDARD = {"timestamp", "level", "logger", "message", "exception", "step"}


@dataclass(frozen=True)
class LogLine:
    logger: str
    level: str
    message: str
    extra: dict = field(default_factory=dict)
    timestamp: str = ""


@dataclass
class Pane:
    name: str
    prefixes: tuple[str, ...]                    # logger-name prefixes routed here ("" matches everything)
    lines: deque = field(default_factory=lambda: deque(maxlen=20000))
    scroll: int = 0                              # index of the first visible line
    hscroll: int = 0
    follow: bool = True

    def add(self, line: LogLine) -> None:
        self.lines.append(line)

    def visible(self, height: int) -> list[LogLine]:
        if self.follow:
            self.scroll = max(0, len(self.lines) - height)
        self.scroll = max(0, min(self.scroll, max(0, len(self.lines) - 1)))
        return list(self.lines)[self.scroll:self.scroll + height]

    def scroll_by(self, n: int, height: int) -> None:
        self.follow = False
        self.scroll = max(0, min(self.scroll + n, max(0, len(self.lines) - height)))
        if n > 0 and self.scroll >= len(self.lines) - height:
            self.follow = True


class TrainingMonitor:
    PANES = (("training", ("research_b200.training", "training", "grpo", "sft", "pretrain", "__main__")),
             ("engine", ("research_b200.inference", "engine", "sglang", "vllm", "server")),
             ("metrics", ("metrics",)),
             ("all", ("",)))

    def __init__(self, max_points: int = 2000):
        self.panes = [Pane(n, p) for n, p in self.PANES]
        self.active = 0
        self.series: dict[str, deque] = {}
        self.max_points = max_points
        self.chart = 0                           # first chart shown on the metrics pane
        self.last_step: int | None = None
        self.errors = 0
        self.running = True
        self.needs_redraw = True

    # ------------------------------------------------------------------ input side
    def parse_line(self, raw: str) -> LogLine | None:
        raw = raw.rstrip("\n")
        if not raw.strip():
            return None
        if raw.lstrip().startswith("{"):
            try:
                d = json.loads(raw)
            except json.JSONDecodeError:
                d = None
            if isinstance(d, dict):
                extra = {k: v for k, v in d.items() if k not in _STANDARD}
                if "step" in d:
                    extra["step"] = d["step"]
                is_metrics = "message" not in d and any(isinstance(v, (int, float)) for v in d.values())
                logger = str(d.get("logger", "metrics" if is_metrics else "log"))
                msg = str(d.get("message", "")) or " ".join(f"{k}={_fmt(v)}" for k, v in d.items() if k not in ("logger", "level", "timestamp"))
                if d.get("exception"):
                    msg += "\n" + str(d["exception"])
                return LogLine(logger, str(d.get("level", "INFO")).upper(), msg, extra, str(d.get("timestamp", "")))
        level = next((lv for lv in ("ERROR", "WARNING", "CRITICAL", "DEBUG") if lv in raw[:40].upper()), "INFO")
        return LogLine("log", level, raw)

    def route(self, line: LogLine) -> str:
        for pane in self.panes[:-1]:
            if any(line.logger == p or line.logger.startswith(p + ".") or (p and line.logger.startswith(p)) for p in pane.prefixes):
                return pane.name
        return "training" if line.logger == "log" else "all"

    def feed_line(self, raw: str) -> None:
        line = self.parse_line(raw)
        if line is None:
            return
        target = self.route(line)
        for pane in self.panes:
            if pane.name == target or pane.name == "all":
                pane.add(line)
        if line.level in ("ERROR", "CRITICAL"):
            self.errors += 1
        step = line.extra.get("step")
        if isinstance(step, (int, float)):
            self.last_step = int(step)
        for k, v in line.extra.items():
            if isinstance(v, (int, float)) and not isinstance(v, bool) and k != "step":
                self.series.setdefault(k, deque(maxlen=self.max_points)).append(float(v))
        self.needs_redraw = True

    def feed(self, lines: Iterable[str]) -> None:
        for raw in lines:
            self.feed_line(raw)

    def handle_key(self, key: str, height: int = 20) -> None:
        pane = self.panes[self.active]
        body = max(1, height - 3)
        on_metrics = pane.name == "metrics"
        if key in "1234":
            self.active = int(key) - 1
        elif key == "q":
            self.running = False
        elif key == "j":
            if on_metrics:
                self.chart = min(self.chart + 1, max(0, len(self.series) - 1))
            else:
                pane.scroll_by(1, body)
        elif key == "k":
            if on_metrics:
                self.chart = max(self.chart - 1, 0)
            else:
                pane.scroll_by(-1, body)
        elif key == "g":
            pane.follow, pane.scroll = False, 0
        elif key == "G":
            pane.follow = True
        elif key == "l":
            pane.hscroll += 10
        elif key == "h":
            pane.hscroll = max(0, pane.hscroll - 10)
        elif key in ("\x04", " "):               # ctrl-d / space: page down
            pane.scroll_by(body, body)
        elif key == "\x15":                      # ctrl-u: page up
            pane.scroll_by(-body, body)
        self.needs_redraw = True

    # ------------------------------------------------------------------ output side
    def render(self, width: int = 100, height: int = 30, color: bool = True) -> list[str]:
        c = (lambda code, s: f"{code}{s}{RESET}" if code else s) if color else (lambda code, s: s)
        tabs = "  ".join(c(INVERSE, f" {i + 1}:{p.name} ") if i == self.active else f" {i + 1}:{p.name} " for i, p in enumerate(self.panes))
        out = [tabs]
        body = max(1, height - 3)
        pane = self.panes[self.active]
        if pane.name == "metrics":
            rows = self._render_charts(width, body)
        else:
            rows = []
            for ln in pane.visible(body):
                first, *rest = ln.message.split("\n")
                text = f"{ln.timestamp[11:19] + ' ' if ln.timestamp else ''}{ln.level[:4]:<4} {ln.logger.split('.')[-1][:14]:<14} {first}"
                rows.append(c(LEVEL_COLOR.get(ln.level, ""), text[pane.hscroll:pane.hscroll + width]))
                rows += [c(DIM, ("     " + r)[pane.hscroll:pane.hscroll + width]) for r in rest]
            rows = rows[-body:] if pane.follow else rows[:body]      # continuation lines may overflow the window
        out += rows + [""] * (body - len(rows))
        step = f"step {self.last_step}" if self.last_step is not None else "no step yet"
        pos = f"{pane.scroll + 1}-{min(pane.scroll + body, len(pane.lines))}/{len(pane.lines)}" if pane.name != "metrics" else f"{len(self.series)} series"
        err = c(RED, f"  {self.errors} errors") if self.errors else ""
        out.append(c(DIM, f"{step}  {pos}  {'follow' if pane.follow else 'paused'}") + err)
        out.append(c(DIM, "1-4 pane  j/k scroll  g/G top/bottom  h/l sideways  q quit"))
        return out

    def _render_charts(self, width: int, height: int) -> list[str]:
        names = sorted(self.series)[self.chart:]
        rows = []
        w = max(10, width - 52)
        for name in names[:height]:
            v = list(self.series[name])
            rows.append(f"{name[:22]:<22}{v[-1]:>12.5g}  min {min(v):<9.3g}max {max(v):<9.3g}{sparkline(v, w)}")
        return rows or ["(no numeric fields seen yet)"]

    # ------------------------------------------------------------------ terminal loop
    def run(self, stream=None, interval: float = 0.05) -> None:
        """Read ``stream`` (default stdin) until it ends or ``q``; keys come from the controlling terminal."""
        stream = stream or sys.stdin
        tty = None
        restore = None
        if sys.stdout.isatty():
            try:
                import termios
                import tty as ttymod

                tty = open("/dev/tty", "rb", buffering=0)  # noqa: SIM115 - closed in finally
                restore = termios.tcgetattr(tty.fileno())
                ttymod.setcbreak(tty.fileno())
                sys.stdout.write("\x1b[?1049h\x1b[?25l")
            except (OSError, ImportError):
                tty = None
        eof = False
        try:
            stream.fileno()
        except (AttributeError, OSError, ValueError):      # an in-memory stream: take it whole, then only keys remain
            self.feed(stream)
            eof = True
        try:
            while self.running and not (eof and tty is None):
                ready = [f for f in ([] if eof else [stream]) + ([tty] if tty else [])]
                r, _, _ = select.select(ready, [], [], interval) if ready else ([], [], [])
                if stream in r:
                    raw = stream.readline()
                    if raw == "":
                        eof = True
                    else:
                        self.feed_line(raw)
                if tty is not None and tty in r:
                    for ch in os.read(tty.fileno(), 32).decode(errors="ignore"):
                        size = os.get_terminal_size()
                        self.handle_key(ch, size.lines)
                if self.needs_redraw and tty is not None:
                    size = os.get_terminal_size()
                    sys.stdout.write("\x1b[H" + "\n".join(line + "\x1b[K" for line in self.render(size.columns, size.lines)) + "\x1b[J")
                    sys.stdout.flush()
                    self.needs_redraw = False
        finally:
            if tty is not None:
                import termios

                termios.tcsetattr(tty.fileno(), termios.TCSADRAIN, restore)
                sys.stdout.write("\x1b[?25h\x1b[?1049l")
                tty.close()
        if tty is None:                          # not a terminal: print the final screen once
            print("\n".join(self.render(120, 40, color=False)))


def _fmt(v) -> str:
    return f"{v:.5g}" if isinstance(v, float) else str(v)


def replay_lines(run_dir: str | Path) -> list[str]:
    """Every log line of a finished run's directory, in a stable order: training.log, other .log / .jsonl files, and
    metrics.jsonl (tagged so they land in the metrics pane)."""
    d = Path(run_dir)
    files = sorted(p for p in d.rglob("*") if p.is_file() and p.suffix in (".log", ".jsonl") and "rollouts" not in p.name)
    files.sort(key=lambda p: (p.name != "training.log", p.name == "metrics.jsonl", str(p)))
    out: list[str] = []
    for p in files:
        for raw in p.read_text(errors="replace").splitlines():
            if p.name == "metrics.jsonl" and raw.startswith("{") and '"logger"' not in raw:
                raw = '{"logger": "metrics", ' + raw.lstrip()[1:]
            out.append(raw)
    return out


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Multi-pane monitor for a JSONL training log")
    ap.add_argument("--replay", default="", help="results directory of a finished run")
    ap.add_argument("--once", action="store_true", help="render one screen to stdout and exit")
    a = ap.parse_args(argv)
    mon = TrainingMonitor()
    if a.replay:
        mon.feed(replay_lines(a.replay))
        if a.once or not sys.stdout.isatty():
            print("\n".join(mon.render(120, 40, color=False)))
            return 0
        import io

        mon.run(io.StringIO(""))
        return 0
    if a.once:
        mon.feed(sys.stdin)
        print("\n".join(mon.render(120, 40, color=False)))
        return 0
    mon.run()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
