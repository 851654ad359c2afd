"""Logging set-up: coloured or JSON console, rotating JSONL file, queue handler
(rollouts/_logging/logging_config.py:11-180, json_formatter.py:38-81). ``extra=`` fields are
emitted as top-level JSON keys, which is what the training monitor routes on."""

from __future__ import annotations

import json
import logging
import logging.handlers
import os
import queue
import time
from pathlib import Path

_RESERVED = set(logging.LogRecord("", 0, "", 0, "", (), None).__dict__) | {"message", "asctime"}


class JSONFormatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        d = {"timestamp": time.strftime("%Y-%m-%dT%H:%M:%S", time.gmtime(record.created)) + f".{int(record.msecs):03d}Z",
             "level": record.levelname, "logger": record.name, "message": record.getMessage()}
        for k, v in record.__dict__.items():
            if k not in _RESERVED and not k.startswith("_"):
                try:
                    json.dumps(v)
                    d[k] = v
                except (TypeError, ValueError):
                    d[k] = repr(v)
        if record.exc_info:
            d["exception"] = self.formatException(record.exc_info)
        return json.dumps(d)


class ColorFormatter(logging.Formatter):
    COLORS = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m", "CRITICAL": "\033[35m"}

    def format(self, record: logging.LogRecord) -> str:
        c = self.COLORS.get(record.levelname, "")
        return f"{c}{record.levelname[:4]}\033[0m {record.name}: {record.getMessage()}"


def setup_logging(level: str | None = None, log_file: str | Path | None = None, json_console: bool | None = None,
                  use_queue: bool = False, max_bytes: int = 50 << 20, backup_count: int = 3) -> logging.Logger:
    """Configure the root logger. ``LOG_LEVEL`` and ``LOG_JSON`` (or ``ROLLOUTS_JSON_LOGS``) override the arguments."""
    level = (os.environ.get("LOG_LEVEL") or level or "INFO").upper()
    if json_console is None:
        json_console = os.environ.get("LOG_JSON", os.environ.get("ROLLOUTS_JSON_LOGS", "")).lower() in ("1", "true", "yes")
    root = logging.getLogger()
    for h in list(root.handlers):
        root.removeHandler(h)
    root.setLevel(level)
    handlers: list[logging.Handler] = []
    console = logging.StreamHandler()
    console.setFormatter(JSONFormatter() if json_console else ColorFormatter())
    handlers.append(console)
    if log_file is not None:
        Path(log_file).parent.mkdir(parents=True, exist_ok=True)
        fh = logging.handlers.RotatingFileHandler(log_file, maxBytes=max_bytes, backupCount=backup_count)
        fh.setFormatter(JSONFormatter())
        handlers.append(fh)
    if use_queue:
        q: queue.Queue = queue.Queue(-1)
        listener = logging.handlers.QueueListener(q, *handlers, respect_handler_level=True)
        listener.start()
        root.addHandler(logging.handlers.QueueHandler(q))
        root._rb_listener = listener  # type: ignore[attr-defined]
    else:
        for h in handlers:
            root.addHandler(h)
    return root


# chatty libraries that say nothing useful below WARNING during an agent run
QUIET_LOGGERS = ("httpx", "httpcore", "httpcore.http11", "httpcore.http2", "openai", "anthropic", "paramiko", "paramiko.transport",
                 "urllib3", "asyncio")


def init_run_logging(experiment_name: str, results_base_dir: str | Path = "results", log_level: str = "INFO",
                     logger_levels: dict[str, str] | None = None, now: float | None = None) -> Path:
    """A results folder ``<base>/<experiment>_<UTC timestamp>/`` with the run's JSONL log (``error_log.jsonl``) in it,
    console logging set up, and HTTP / SSH client libraries held at WARNING unless ``logger_levels`` says otherwise
    (rollouts/logging_utils.py:13-80). Returns the folder: a run writes its other outputs there."""
    stamp = time.strftime("%Y%m%d-%H%M%S", time.gmtime(now if now is not None else time.time()))
    result_dir = Path(results_base_dir) / f"{experiment_name}_{stamp}"
    result_dir.mkdir(parents=True, exist_ok=True)
    setup_logging(level=log_level, log_file=result_dir / "error_log.jsonl")
    for name, lvl in {**{n: "WARNING" for n in QUIET_LOGGERS}, **(logger_levels or {})}.items():
        logging.getLogger(name).setLevel(lvl.upper())
    logging.getLogger(__name__).info("results directory: %s", result_dir)
    return result_dir


def get_logger(name: str) -> logging.Logger:
    return logging.getLogger(name)
