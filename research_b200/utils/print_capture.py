"""Route ``print`` output of noisy third-party code into ``logging`` for the length of a ``with`` block
(shared/shared/print_interceptor.py:131). Lines are forwarded whole: partial writes are held until their newline."""

from __future__ import annotations

import logging
import sys
from contextlib import contextmanager
from typing import Iterator, TextIO


class _LineToLogger:
    def __init__(self, logger: logging.Logger, level: int, tee: TextIO | None):
        self.logger, self.level, self.tee = logger, level, tee
        self._held = ""

    def write(self, text: str) -> int:
        if self.tee is not None:
            self.tee.write(text)
        self._held += text
        *lines, self._held = self._held.split("\n")
        for ln in lines:
            if ln.strip():
                self.logger.log(self.level, ln.rstrip())
        return len(text)

    def flush(self) -> None:
        if self.tee is not None:
            self.tee.flush()

    def finish(self) -> None:
        if self._held.strip():
            self.logger.log(self.level, self._held.rstrip())
        self._held = ""

    def isatty(self) -> bool:
        return False


@contextmanager
def intercept_prints(logger: logging.Logger | None = None, level: int = logging.INFO, intercept_stdout: bool = True,
                     intercept_stderr: bool = False, also_print: bool = False) -> Iterator[None]:
    """Inside the block ``sys.stdout`` (and optionally ``sys.stderr``, logged at ERROR) feed ``logger``;
    ``also_print`` keeps writing to the real stream as well. The streams are always restored."""
    logger = logger or logging.getLogger()
    old_out, old_err = sys.stdout, sys.stderr
    out = _LineToLogger(logger, level, old_out if also_print else None) if intercept_stdout else None
    err = _LineToLogger(logger, logging.ERROR, old_err if also_print else None) if intercept_stderr else None
    try:
        if out is not None:
            sys.stdout = out  # type: ignore[assignment]
        if err is not None:
            sys.stderr = err  # type: ignore[assignment]
        yield
    finally:
        sys.stdout, sys.stderr = old_out, old_err
        for w in (out, err):
            if w is not None:
                w.finish()
