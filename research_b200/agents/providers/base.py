"""Provider errors, request hygiene (log sanitising, prompt-cache markers, cost), retry with back-off and jitter, and
rate limiting (rollouts/providers/base.py:13-270, _retry.py:92-270, _rate_limit.py:22-147)."""

from __future__ import annotations

import asyncio
import copy
import functools
import random
import re
import time
from dataclasses import replace
from typing import Any, Awaitable, Callable


class ProviderError(Exception):
    """Transient failure of the endpoint, not of the model: worth retrying (timeouts, 429, 5xx). Evaluation counts a
    sample that ends with one as ``provider_error`` and leaves it out of the accuracy. ``attempts`` and
    ``original_error`` are filled in by the retry wrapper when it gives up."""

    def __init__(self, message: str, status: int | None = None, provider: str = "", original_error: BaseException | None = None,
                 attempts: int = 0):
        super().__init__(message)
        self.status, self.provider, self.original_error, self.attempts = status, provider, original_error, attempts


class NonRetryableError(ProviderError):
    """Permanent failure: bad request, auth, context overflow."""


class ContextTooLongError(NonRetryableError):
    """The prompt does not fit the model's window. Recoverable by the caller (compact or slice the conversation);
    ``current_tokens`` / ``max_tokens`` are filled in when the server's message states them."""

    def __init__(self, message: str = "context too long", status: int | None = None, provider: str = "",
                 current_tokens: int | None = None, max_tokens: int | None = None):
        super().__init__(message, status, provider)
        self.current_tokens, self.max_tokens = current_tokens, max_tokens


_CTX_PATTERNS = (
    re.compile(r"maximum context length is (\d+) tokens.*?(?:requested|resulted in|have) (\d+)", re.I | re.S),
    re.compile(r"prompt is too long: (\d+) tokens > (\d+)", re.I),
    re.compile(r"input token count \(?(\d+)\)? exceeds the maximum.*?(\d+)", re.I | re.S),
)


def parse_context_overflow(body: str) -> tuple[int | None, int | None] | None:
    """``(current_tokens, max_tokens)`` out of a server's context-overflow message (OpenAI / vLLM / SGLang, Anthropic,
    Google wording), ``(None, None)`` if it is one without numbers, ``None`` if the body is about something else."""
    low = body.lower()
    for i, pat in enumerate(_CTX_PATTERNS):
        m = pat.search(body)
        if m:
            a, b = int(m.group(1)), int(m.group(2))
            return (b, a) if i == 0 else (a, b)
    if ("context" in low and ("length" in low or "window" in low)) or "prompt is too long" in low or "too many tokens" in low:
        return None, None
    return None


def classify_server_error(status: int, body: str) -> str:
    """``success`` | ``context_length`` | ``invalid_param`` | ``rate_limit`` | ``auth`` | ``server`` | ``http_error``
    for a response of an OpenAI-compatible server (vLLM / SGLang / this package's own)."""
    low = body.lower()
    if status == 200:
        return "success"
    if parse_context_overflow(body) is not None:
        return "context_length"
    if "not a valid parameter" in low or "unexpected keyword" in low or "extra inputs are not permitted" in low or "unknown parameter" in low:
        return "invalid_param"
    if status == 429:
        return "rate_limit"
    if status in (401, 403):
        return "auth"
    if status >= 500 or status in (408, 409, 425):
        return "server"
    return "http_error"


def explain_server_error(kind: str, *, max_tokens: int | None = None, param_keys: list[str] | None = None) -> str:
    """What a person should do about an error of this kind (shown once, when retries stop)."""
    if kind == "context_length":
        half = f" (try {max_tokens // 2})" if max_tokens else ""
        return ("the request does not fit the server's context window: the server itself is fine. Lower max_tokens" + half +
                ", shorten the conversation (slice / compact it), or start the server with a larger --max-model-len. Retrying cannot help.")
    if kind == "invalid_param":
        return (f"the server rejects one of the request parameters {sorted(param_keys or [])}: drop the optional ones "
                "(logprobs, echo, return_tokens_as_token_ids) or upgrade the server.")
    if kind == "rate_limit":
        return "rate limited: the retry wrapper backs off; lower max_concurrent if it keeps happening."
    if kind == "auth":
        return "the API key was rejected: check the environment variable the endpoint names."
    if kind == "server":
        return "server-side failure (5xx / timeout): retried with back-off."
    return "unexpected HTTP error: see the response body."


def classify_http_status(status: int, body: str = "", provider: str = "") -> ProviderError:
    kind = classify_server_error(status, body)
    if kind in ("rate_limit", "server"):
        return ProviderError(f"HTTP {status}: {body[:200]}", status, provider)
    if kind == "context_length":
        cur, mx = parse_context_overflow(body) or (None, None)
        return ContextTooLongError(f"HTTP {status}: {body[:200]}", status, provider, cur, mx)
    return NonRetryableError(f"HTTP {status}: {body[:200]}", status, provider)


def sanitize_request_for_logging(params: dict, max_text: int = 500) -> dict:
    """Copy of a request body that is safe to log: inline images (base64 data URLs or raw ``data`` fields, often
    100 KB and more) become ``<image: N bytes>`` and long texts are cut to ``max_text`` characters with their length."""
    def clip(text: str) -> str:
        if text.startswith("data:") and ";base64," in text[:64]:
            return f"<image: {len(text)} bytes>"
        return text if len(text) <= max_text else text[:max_text] + f"... ({len(text)} chars total)"

    def walk(x: Any, key: str = "") -> Any:
        if isinstance(x, dict):
            return {k: walk(v, k) for k, v in x.items()}
        if isinstance(x, list):
            return [walk(v, key) for v in x]
        if isinstance(x, str):
            if key == "data" and len(x) > max_text:       # a raw base64 payload
                return f"<image: {len(x)} bytes>"
            return clip(x)
        return x

    out = walk(copy.deepcopy(params))
    for k in list(out):
        if "key" in k.lower() or k.lower() == "authorization":
            out[k] = "***"
    return out


def add_cache_control_to_last_content(messages: list[dict], cache_control: dict | None = None, max_cache_controls: int = 4) -> list[dict]:
    """Anthropic prompt caching: mark the last content block of the last message as a cache break point, unless the
    request already carries ``max_cache_controls`` of them (the API allows four). Returns a copy."""
    cache_control = cache_control or {"type": "ephemeral"}
    if not messages:
        return messages
    out = copy.deepcopy(messages)

    def blocks(m):
        c = m.get("content")
        return c if isinstance(c, list) else [c]

    if sum(1 for m in out for b in blocks(m) if isinstance(b, dict) and "cache_control" in b) >= max_cache_controls:
        return out
    last = out[-1]
    c = last.get("content")
    if isinstance(c, str) and c:                       # a plain string cannot carry the marker: make it a text block
        last["content"] = [{"type": "text", "text": c, "cache_control": cache_control}]
    elif isinstance(c, list) and c and isinstance(c[-1], dict) and "type" in c[-1]:
        c[-1].setdefault("cache_control", cache_control)
    elif isinstance(c, dict):
        c.setdefault("cache_control", cache_control)
    return out


def prepare_messages_for_llm(messages: list) -> list:
    """Tool results carry ``metadata["details"]`` for the user interface (full diffs, long outputs); the model only
    gets ``content``. Returns the list with those details removed from tool messages (no message is dropped)."""
    out = []
    for m in messages:
        if m.role == "tool" and m.metadata and "details" in m.metadata:
            out.append(replace(m, metadata={k: v for k, v in m.metadata.items() if k != "details"}))
        else:
            out.append(m)
    return out


def calculate_cost_from_usage(usage, model) -> Any:
    """``Usage`` x a model's prices per million tokens (``providers.models.ModelInfo``; None = unknown model) -> ``Cost``
    in USD, cache reads and writes priced separately."""
    from ..dtypes import Cost

    if model is None:
        return Cost()
    return Cost(input=usage.input_tokens / 1e6 * model.input_per_mtok, output=usage.output_tokens / 1e6 * model.output_per_mtok,
                cache_read=usage.cache_read_tokens / 1e6 * getattr(model, "cache_read_per_mtok", 0.0),
                cache_write=usage.cache_write_tokens / 1e6 * getattr(model, "cache_write_per_mtok", 0.0))


def backoff_delay(attempt: int, base: float = 1.0, factor: float = 2.0, max_delay: float = 60.0, jitter: float = 0.25,
                  rng: random.Random | None = None) -> float:
    d = min(max_delay, base * factor ** attempt)
    r = (rng or random).uniform(-jitter, jitter)
    return max(0.0, d * (1 + r))


def async_retry(max_attempts: int = 3, base: float = 1.0, factor: float = 2.0, max_delay: float = 60.0,
                retry_on: tuple[type[BaseException], ...] = (ProviderError, asyncio.TimeoutError, ConnectionError),
                sleep: Callable[[float], Awaitable[None]] = asyncio.sleep, wrap_as_provider_error: str | None = None):
    """Retry ``fn`` on transient errors with exponential back-off and jitter. ``wrap_as_provider_error="anthropic"``:
    when the attempts run out, raise ``ProviderError`` naming that provider, the attempts made and the last error,
    whatever its type was (so that callers can tell infrastructure failures from model failures)."""
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
            if wrap_as_provider_error is not None:
                raise ProviderError(f"ProviderError[{wrap_as_provider_error}]: {type(last).__name__}: {last}",
                                    getattr(last, "status", None), wrap_as_provider_error, last, max_attempts) from last
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
