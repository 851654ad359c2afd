"""Rate-limit stress run for a provider call (rollouts/scripts/stress_test_rate_limits.py): fire many requests through a
``RateLimiter`` + retry policy and report what came back: achieved request rate, how many calls hit a retryable error
(HTTP 429 and friends), how many retries were spent, how many failed for good, and latency percentiles. The call under
test is any ``async () -> Any``; ``simulated_provider`` is a stand-in with a sliding-window quota for dry runs.

    python -m research_b200.agents.providers.stress --requests 200 --concurrency 16 --rps 20 --quota 10
"""

from __future__ import annotations

import argparse
import asyncio
import statistics
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Any, Awaitable, Callable, Sequence

from .base import NonRetryableError, ProviderError, RateLimiter, backoff_delay


@dataclass
class StressReport:
    requests: int
    succeeded: int = 0
    failed: int = 0
    rate_limited_calls: int = 0        # calls that saw at least one retryable error
    retries: int = 0
    non_retryable: int = 0
    seconds: float = 0.0
    latencies: list[float] = field(default_factory=list, repr=False)
    peak_in_flight: int = 0

    @property
    def achieved_rps(self) -> float:
        return self.succeeded / self.seconds if self.seconds > 0 else 0.0

    def percentile(self, q: float) -> float:
        if not self.latencies:
            return 0.0
        xs = sorted(self.latencies)
        return xs[min(len(xs) - 1, int(q * len(xs)))]

    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        d.pop("latencies")
        d.update(achieved_rps=self.achieved_rps, p50_s=self.percentile(0.5), p95_s=self.percentile(0.95), p99_s=self.percentile(0.99),
                 mean_s=statistics.fmean(self.latencies) if self.latencies else 0.0)
        return d

    def summary(self) -> str:
        d = self.to_dict()
        return (f"{self.succeeded}/{self.requests} ok, {self.failed} failed ({self.non_retryable} non-retryable), "
                f"{self.rate_limited_calls} calls rate-limited, {self.retries} retries, {d['achieved_rps']:.1f} req/s, "
                f"latency p50 {d['p50_s'] * 1e3:.0f} ms p95 {d['p95_s'] * 1e3:.0f} ms, peak in flight {self.peak_in_flight}")


async def stress(call: Callable[[], Awaitable[Any]], requests: int = 100, max_concurrent: int = 8, requests_per_second: float | None = None,
                 max_attempts: int = 4, backoff_base: float = 0.5, max_delay: float = 30.0,
                 sleep: Callable[[float], Awaitable[None]] = asyncio.sleep) -> StressReport:
    limiter = RateLimiter(max_concurrent, requests_per_second)
    rep = StressReport(requests)

    async def one() -> None:
        t0 = time.monotonic()
        limited = False
        for attempt in range(max_attempts):
            try:
                async with limiter:
                    rep.peak_in_flight = max(rep.peak_in_flight, limiter.in_flight)
                    await call()
                rep.succeeded += 1
                rep.latencies.append(time.monotonic() - t0)
                break
            except NonRetryableError:
                rep.failed += 1
                rep.non_retryable += 1
                break
            except (ProviderError, asyncio.TimeoutError, ConnectionError):
                limited = True
                if attempt + 1 == max_attempts:
                    rep.failed += 1
                    break
                rep.retries += 1
                await sleep(backoff_delay(attempt, backoff_base, 2.0, max_delay))
        rep.rate_limited_calls += limited

    t0 = time.monotonic()
    await asyncio.gather(*(one() for _ in range(requests)))
    rep.seconds = time.monotonic() - t0
    return rep


def simulated_provider(quota: int = 10, window_s: float = 1.0, latency_s: float = 0.01, clock: Callable[[], float] = time.monotonic,
                       sleep: Callable[[float], Awaitable[None]] = asyncio.sleep) -> Callable[[], Awaitable[str]]:
    """A call that answers after ``latency_s`` unless more than ``quota`` calls arrived within the last ``window_s``
    seconds, in which case it raises the retryable error an HTTP 429 maps to."""
    seen: deque[float] = deque()

    async def call() -> str:
        now = clock()
        while seen and now - seen[0] > window_s:
            seen.popleft()
        if len(seen) >= quota:
            raise ProviderError("HTTP 429: quota exceeded", 429, "simulated")
        seen.append(now)
        await sleep(latency_s)
        return "ok"

    return call


def main(argv: Sequence[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--requests", type=int, default=100)
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--rps", type=float, default=0.0, help="client-side requests per second (0: unlimited)")
    ap.add_argument("--quota", type=int, default=10, help="simulated server quota per window")
    ap.add_argument("--window", type=float, default=1.0)
    ap.add_argument("--latency", type=float, default=0.01)
    ap.add_argument("--attempts", type=int, default=4)
    a = ap.parse_args(argv)
    rep = asyncio.run(stress(simulated_provider(a.quota, a.window, a.latency), a.requests, a.concurrency, a.rps or None, a.attempts, 0.1, 2.0))
    print(rep.summary())
    return 0 if rep.failed == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
