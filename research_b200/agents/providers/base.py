"""Provider errors, retry with back-off and jitter, and rate limiting
(rollouts/providers/base.py:13-94, _retry.py:92-270, _rate_limit.py:22-147)."""

from __future__ import annotations

import asyncio
import functools
import random
import time
from typing import Any, Awaitable, Callable


class ProviderError(Exception):
    """Transient failure: worth retrying (timeouts, 429, 5xx)."""

    def __init__(self, message: str, status: int | None = None, provider: str = ""):
        super().__init__(message)
        self.status, self.provider = status, provider


class NonRetryableError(ProviderError):
    """Permanent failure: bad request, auth, context overflow."""


class ContextTooLongError(NonRetryableError):
    pass


def classify_http_status(status: int, body: str = "", provider: str = "") -> ProviderError:
    if status in (408, 409, 425, 429) or status >= 500:
        return ProviderError(f"HTTP {status}: {body[:200]}", status, provider)
    if status == 400 and "context" in body.lower() and "length" in body.lower():
        return ContextTooLongError(f"HTTP 400: {body[:200]}", status, provider)
    return NonRetryableError(f"HTTP {status}: {body[:200]}", status, provider)


def backoff_delay(attempt: int, base: float = 1.0, factor: float = 2.0, max_delay: float = 60.0, jitter: float = 0.25,
                  rng: random.Random | None = None) -> float:
    d = min(max_delay, base * factor ** attempt)
    r = (rng or random).uniform(-jitter, jitter)
    return max(0.0, d * (1 + r))


def async_retry(max_attempts: int = 3, base: float = 1.0, factor: float = 2.0, max_delay: float = 60.0,
                retry_on: tuple[type[BaseException], ...] = (ProviderError, asyncio.TimeoutError, ConnectionError),
                sleep: Callable[[float], Awaitable[None]] = asyncio.sleep):
    def deco(fn):
        @functools.wraps(fn)
        async def wrapper(*a: Any, **k: Any):
            last: BaseException | None = None
            for attempt in range(max_attempts):
                try:
                    return await fn(*a, **k)
                except NonRetryableError:
                    raise
                except retry_on as e:  # type: ignore[misc]
                    last = e
                    if attempt + 1 < max_attempts:
                        await sleep(backoff_delay(attempt, base, factor, max_delay))
            assert last is not None
            raise last

        return wrapper

    return deco


def retry(max_attempts: int = 3, base: float = 0.5, retry_on: tuple[type[BaseException], ...] = (Exception,)):
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a: Any, **k: Any):
            for attempt in range(max_attempts):
                try:
                    return fn(*a, **k)
                except retry_on:
                    if attempt + 1 == max_attempts:
                        raise
                    time.sleep(backoff_delay(attempt, base))

        return wrapper

    return deco


class RateLimiter:
    """Bounded concurrency plus a token bucket of requests per second; use as ``async with``."""

    def __init__(self, max_concurrent: int = 8, requests_per_second: float | None = None):
        self._sem = asyncio.Semaphore(max_concurrent)
        self.rps = requests_per_second
        self._next = 0.0
        self._lock = asyncio.Lock()
        self.in_flight = 0
        self.total = 0

    async def __aenter__(self) -> "RateLimiter":
        await self._sem.acquire()
        if self.rps:
            async with self._lock:
                now = time.monotonic()
                wait = self._next - now
                self._next = max(now, self._next) + 1.0 / self.rps
            if wait > 0:
                await asyncio.sleep(wait)
        self.in_flight += 1
        self.total += 1
        return self

    async def __aexit__(self, *exc: Any) -> None:
        self.in_flight -= 1
        self._sem.release()
