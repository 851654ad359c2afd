"""Terminal progress: a multi-task board and a small tqdm-compatible bar (rollouts/progress.py:49-502).

Both write carriage-return lines to a stream (stderr by default), degrade to plain log lines when
the stream is not a terminal, and never need a curses / rich dependency.
"""

from __future__ import annotations

import sys
import time
from dataclasses import dataclass, field
from typing import Generic, Iterable, Iterator, TextIO, TypeVar

T = TypeVar("T")


def format_time(seconds: float) -> str:
    seconds = max(0, int(seconds))
    h, rem = divmod(seconds, 3600)
    m, s = divmod(rem, 60)
    return f"{h}:{m:02d}:{s:02d}" if h else f"{m:02d}:{s:02d}"


def format_bar(progress: float, width: int) -> str:
    progress = min(max(progress, 0.0), 1.0)
    full = int(progress * width)
    part = int((progress * width - full) * 8)
    bar = "█" * full + (" ▏▎▍▌▋▊▉"[part] if full < width and part else "")
    return bar.ljust(width)


@dataclass
class TaskState:
    name: str
    total: int | None = None
    done: int = 0
    status: str = "running"            # running | done | failed
    message: str = ""
    started: float = field(default_factory=time.monotonic)
    finished: float | None = None

    @property
    def elapsed(self) -> float:
        return (self.finished or time.monotonic()) - self.started


class MultiProgress:
    """Several named tasks rendered as one block that is redrawn in place."""

    def __init__(self, stream: TextIO | None = None, width: int = 24, min_interval: float = 0.1):
        self.stream = stream or sys.stderr
        self.width, self.min_interval = width, min_interval
        self.tasks: dict[str, TaskState] = {}
        self._drawn, self._last = 0, 0.0
        self.tty = hasattr(self.stream, "isatty") and self.stream.isatty()

    def add_task(self, name: str, total: int | None = None) -> TaskState:
        self.tasks[name] = TaskState(name, total)
        self.refresh(force=True)
        return self.tasks[name]

    def update(self, name: str, advance: int = 1, message: str | None = None) -> None:
        t = self.tasks[name]
        t.done += advance
        if message is not None:
            t.message = message
        self.refresh()

    def finish(self, name: str, status: str = "done", message: str | None = None) -> None:
        t = self.tasks[name]
        t.status, t.finished = status, time.monotonic()
        if message is not None:
            t.message = message
        self.refresh(force=True)

    def render_lines(self) -> list[str]:
        lines = []
        for t in self.tasks.values():
            mark = {"running": "…", "done": "✓", "failed": "✗"}.get(t.status, "?")
            if t.total:
                frac = t.done / t.total
                rate = t.done / t.elapsed if t.elapsed > 0 else 0.0
                eta = f" eta {format_time((t.total - t.done) / rate)}" if rate > 0 and t.status == "running" else ""
                body = f"|{format_bar(frac, self.width)}| {t.done}/{t.total} [{format_time(t.elapsed)}{eta}]"
            else:
                body = f"{t.done} [{format_time(t.elapsed)}]"
            lines.append(f"{mark} {t.name:<20.20} {body} {t.message}".rstrip())
        return lines

    def refresh(self, force: bool = False) -> None:
        now = time.monotonic()
        if not force and now - self._last < self.min_interval:
            return
        self._last = now
        lines = self.render_lines()
        if self.tty:
            if self._drawn:
                self.stream.write(f"\x1b[{self._drawn}F")
            self.stream.write("".join(f"\x1b[2K{line}\n" for line in lines))
            self._drawn = len(lines)
        elif force and lines:
            self.stream.write(lines[-1] + "\n")
        self.stream.flush()

    def __enter__(self) -> "MultiProgress":
        return self

    def __exit__(self, *exc) -> None:
        for t in self.tasks.values():
            if t.status == "running":
                t.status, t.finished = ("failed" if exc[0] else "done"), time.monotonic()
        self.refresh(force=True)


class tqdm(Generic[T]):
    """The subset of the tqdm interface the loops use: iteration, ``update``, ``set_postfix``, ``close``."""

    def __init__(self, iterable: Iterable[T] | None = None, total: int | None = None, desc: str = "", file: TextIO | None = None,
                 disable: bool = False, width: int = 24, mininterval: float = 0.1):
        self.iterable, self.desc, self.file, self.disable = iterable, desc, file or sys.stderr, disable
        self.total = total if total is not None else (len(iterable) if hasattr(iterable, "__len__") else None)
        self.n, self.width, self.mininterval = 0, width, mininterval
        self.postfix = ""
        self._t0 = self._last = time.monotonic()

    def __iter__(self) -> Iterator[T]:
        assert self.iterable is not None
        for x in self.iterable:
            yield x
            self.update(1)
        self.close()

    def __len__(self) -> int:
        return self.total or 0

    def set_postfix(self, **kw) -> None:
        self.postfix = ", ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in kw.items())

    def set_description(self, desc: str) -> None:
        self.desc = desc

    def format_line(self) -> str:
        el = time.monotonic() - self._t0
        rate = self.n / el if el > 0 else 0.0
        if self.total:
            eta = format_time((self.total - self.n) / rate) if rate > 0 else "?"
            s = f"{self.desc}: {100 * self.n // self.total:3d}%|{format_bar(self.n / self.total, self.width)}| {self.n}/{self.total} [{format_time(el)}<{eta}, {rate:.2f}it/s]"
        else:
            s = f"{self.desc}: {self.n}it [{format_time(el)}, {rate:.2f}it/s]"
        return s + (f" {self.postfix}" if self.postfix else "")

    def update(self, n: int = 1) -> None:
        self.n += n
        now = time.monotonic()
        if self.disable or (now - self._last < self.mininterval and self.n != self.total):
            return
        self._last = now
        self.file.write("\r" + self.format_line())
        self.file.flush()

    def close(self) -> None:
        if not self.disable:
            self.file.write("\r" + self.format_line() + "\n")
            self.file.flush()

    def __enter__(self) -> "tqdm[T]":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
