"""Run a training command and merge everything it produces into ONE stream of JSON lines on standard output
(rollouts/rollouts/tui/remote_runner.py:28-143): the command's own output (made to log JSON), plus any number of side
files (an inference server's log, a metrics JSONL) tailed as ``{"logger": <name>, "message": <line>}`` records. The
stream is what ``frontend.training_monitor`` and ``frontend.trace_browser --follow`` read, locally or through ssh:

    ssh node "python -m research_b200.frontend.remote_runner --training-cmd 'python train.py cfg.py' \\
              --tail engine=/tmp/engine.log --tail metrics=results/run/metrics.jsonl" | python -m research_b200.frontend.training_monitor
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path
from typing import Callable, TextIO

_print_lock = threading.Lock()


def emit(record: dict, out: TextIO | None = None) -> None:
    with _print_lock:
        (out or sys.stdout).write(json.dumps(record) + "\n")
        (out or sys.stdout).flush()


def tail_file_as_jsonl(file_path: str | Path, logger_name: str, stop_event: threading.Event, out: TextIO | None = None,
                       from_start: bool = False, poll_s: float = 0.1) -> int:
    """Follow ``file_path`` (waiting for it to appear) and emit each new line as a JSON record under ``logger_name``
    until ``stop_event`` is set; lines that are JSON objects already only get the logger name added. Returns the
    number of lines emitted."""
    path = Path(file_path)
    while not path.exists():
        if stop_event.wait(0.2):
            return 0
    n = 0
    with open(path, errors="replace") as f:
        if not from_start:
            f.seek(0, 2)
        while True:
            line = f.readline()
            if line:
                if not line.endswith("\n") and not stop_event.is_set():
                    # a partially written line: wait for the rest
                    time.sleep(poll_s)
                    line += f.readline()
                text = line.rstrip("\n")
                rec = None
                if text.startswith("{"):
                    try:
                        obj = json.loads(text)
                        if isinstance(obj, dict):
                            rec = {"logger": logger_name, **obj}
                    except json.JSONDecodeError:
                        rec = None
                emit(rec if rec is not None else {"logger": logger_name, "message": text}, out)
                n += 1
            elif stop_event.is_set():
                return n
            else:
                time.sleep(poll_s)


def run_training_with_json_logging(cmd: str, stop_event: threading.Event, out: TextIO | None = None,
                                   on_line: Callable[[str], None] | None = None) -> int:
    """Run ``cmd`` through the shell with JSON logging switched on (``LOG_JSON=true``, unbuffered Python) and pass its
    merged stdout / stderr through: JSON lines untouched, anything else wrapped as a ``training`` record. Sets
    ``stop_event`` when the command ends; returns its exit code."""
    env = dict(os.environ, LOG_JSON="true", PYTHONUNBUFFERED="1")
    proc = subprocess.Popen(cmd, shell=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, text=True)
    assert proc.stdout is not None
    for line in proc.stdout:
        text = line.rstrip("\n")
        if on_line is not None:
            on_line(text)
        if text.startswith("{"):
            with _print_lock:
                (out or sys.stdout).write(text + "\n")
                (out or sys.stdout).flush()
        elif text:
            emit({"logger": "training", "message": text}, out)
    proc.wait()
    stop_event.set()
    return proc.returncode


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Run a training command with one merged JSONL output stream")
    ap.add_argument("--training-cmd", required=True)
    ap.add_argument("--tail", action="append", default=[], metavar="NAME=PATH", help="file to follow as records of logger NAME")
    ap.add_argument("--sglang-log", help="same as --tail sglang=PATH")
    ap.add_argument("--metrics-log", help="same as --tail metrics=PATH")
    a = ap.parse_args(argv)
    tails = [t.split("=", 1) for t in a.tail]
    if a.sglang_log:
        tails.append(["sglang", a.sglang_log])
    if a.metrics_log:
        tails.append(["metrics", a.metrics_log])
    stop = threading.Event()
    threads = [threading.Thread(target=tail_file_as_jsonl, args=(path, name, stop), daemon=True) for name, path in tails]
    for t in threads:
        t.start()
    rc = run_training_with_json_logging(a.training_cmd, stop)
    for t in threads:
        t.join(timeout=2.0)
    return rc


if __name__ == "__main__":
    raise SystemExit(main())
