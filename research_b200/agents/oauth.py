"""Subscription log-in for hosted models: OAuth 2 authorization-code flow with PKCE, where the user opens a URL,
signs in, and pastes the code the provider shows back into the terminal (rollouts/frontends/tui/oauth.py:45-316).

The flow is generic. Which application it logs into is described by an ``OAuthApp`` (authorize / token URLs, client
id, redirect URI, scopes) that the user supplies in ``~/.research_b200/oauth/<name>.app.json`` or through
``RB_OAUTH_<NAME>_*`` environment variables; no provider's client id is built in. Tokens are kept in
``~/.research_b200/oauth/<name>.json`` readable by the owner only, treated as expired three minutes early so that no
request starts with a token that dies under it, refreshed on demand, and dropped when a refresh is refused (the
grant was revoked). HTTP goes through an injectable ``transport(url, json) -> (status, body)`` so that every path is
testable without a network.
"""

from __future__ import annotations

import asyncio
import base64
import hashlib
import json
import os
import secrets
import time
import urllib.error
import urllib.request
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Awaitable, Callable
from urllib.parse import urlencode

EXPIRY_MARGIN_S = 180.0
DEFAULT_DIR = Path.home() / ".research_b200" / "oauth"
Transport = Callable[[str, dict[str, Any]], Awaitable[tuple[int, Any]]]


class OAuthError(RuntimeError):
    pass


@dataclass(frozen=True)
class OAuthApp:
    name: str
    authorize_url: str
    token_url: str
    client_id: str
    redirect_uri: str
    scopes: str = ""
    extra_authorize_params: dict[str, str] = field(default_factory=dict)
    request_headers: dict[str, str] = field(default_factory=dict)     # sent with model requests that use the token

    @staticmethod
    def load(name: str, directory: Path = DEFAULT_DIR, env: dict[str, str] | None = None) -> "OAuthApp":
        """From ``<directory>/<name>.app.json``, overridden field by field by ``RB_OAUTH_<NAME>_<FIELD>``."""
        env = os.environ if env is None else env
        d: dict[str, Any] = {}
        f = directory / f"{name}.app.json"
        if f.is_file():
            d = json.loads(f.read_text())
        for key in ("authorize_url", "token_url", "client_id", "redirect_uri", "scopes"):
            v = env.get(f"RB_OAUTH_{name.upper()}_{key.upper()}")
            if v:
                d[key] = v
        missing = [k for k in ("authorize_url", "token_url", "client_id", "redirect_uri") if not d.get(k)]
        if missing:
            raise OAuthError(f"OAuth application {name!r} is not configured: {', '.join(missing)} missing (write {f} or set "
                             f"RB_OAUTH_{name.upper()}_{missing[0].upper()} ...)")
        d.pop("name", None)
        return OAuthApp(name=name, **d)


@dataclass
class OAuthTokens:
    access_token: str
    refresh_token: str
    expires_at: float                         # seconds since the epoch, margin already subtracted

    def is_expired(self, now: float | None = None) -> bool:
        return (time.time() if now is None else now) >= self.expires_at


class TokenStorage:
    def __init__(self, path: Path):
        self.path = Path(path)

    def save(self, tokens: OAuthTokens) -> None:
        self.path.parent.mkdir(parents=True, exist_ok=True, mode=0o700)
        tmp = self.path.with_suffix(".tmp")
        fd = os.open(tmp, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)      # never world-readable, not even briefly
        with os.fdopen(fd, "w") as f:
            json.dump(asdict(tokens), f)
        os.replace(tmp, self.path)

    def load(self) -> OAuthTokens | None:
        try:
            return OAuthTokens(**json.loads(self.path.read_text()))
        except (OSError, ValueError, TypeError):
            return None

    def delete(self) -> None:
        try:
            self.path.unlink()
        except FileNotFoundError:
            pass


def generate_pkce() -> tuple[str, str]:
    """``(verifier, challenge)``: 32 random bytes, and the unpadded URL-safe base64 of their SHA-256."""
    verifier = base64.urlsafe_b64encode(secrets.token_bytes(32)).rstrip(b"=").decode()
    challenge = base64.urlsafe_b64encode(hashlib.sha256(verifier.encode()).digest()).rstrip(b"=").decode()
    return verifier, challenge


async def urllib_transport(url: str, payload: dict[str, Any]) -> tuple[int, Any]:
    def post() -> tuple[int, Any]:
        req = urllib.request.Request(url, json.dumps(payload).encode(), {"Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(req, timeout=30) as r:
                return r.status, json.loads(r.read() or b"{}")
        except urllib.error.HTTPError as e:
            return e.code, e.read().decode(errors="replace")
        except (urllib.error.URLError, OSError) as e:
            raise OAuthError(f"cannot reach {url}: {e}") from e

    return await asyncio.to_thread(post)


class OAuthClient:
    def __init__(self, app: OAuthApp, storage: TokenStorage | None = None, transport: Transport = urllib_transport,
                 clock: Callable[[], float] = time.time):
        self.app, self.transport, self.clock = app, transport, clock
        self.storage = storage or TokenStorage(DEFAULT_DIR / f"{app.name}.json")
        self._tokens: OAuthTokens | None = None
        self._verifier: str | None = None
        self._state: str | None = None
        self._refreshing: asyncio.Lock | None = None

    @property
    def tokens(self) -> OAuthTokens | None:
        if self._tokens is None:
            self._tokens = self.storage.load()
        return self._tokens

    def is_logged_in(self) -> bool:
        return self.tokens is not None

    def get_authorize_url(self) -> str:
        """The URL to open. Keeps the PKCE verifier and a separate random ``state`` for ``exchange_code``."""
        self._verifier, challenge = generate_pkce()
        self._state = secrets.token_urlsafe(16)
        params = {"client_id": self.app.client_id, "response_type": "code", "redirect_uri": self.app.redirect_uri,
                  "scope": self.app.scopes, "code_challenge": challenge, "code_challenge_method": "S256", "state": self._state,
                  **self.app.extra_authorize_params}
        return f"{self.app.authorize_url}?{urlencode(params)}"

    def _take(self, data: Any, old_refresh: str | None = None) -> OAuthTokens:
        try:
            t = OAuthTokens(data["access_token"], data.get("refresh_token") or old_refresh or "",
                            self.clock() + float(data["expires_in"]) - EXPIRY_MARGIN_S)
        except (KeyError, TypeError, ValueError) as e:
            raise OAuthError(f"the token endpoint's answer lacks a field: {e}") from e
        self._tokens = t
        self.storage.save(t)
        return t

    async def exchange_code(self, pasted: str) -> OAuthTokens:
        """``pasted`` is what the provider showed: the code, possibly as ``code#state``. A state that is not the one
        this client sent means the code belongs to another log-in attempt and is refused."""
        if self._verifier is None:
            raise OAuthError("no log-in in progress: call get_authorize_url first")
        code, _, state = pasted.strip().partition("#")
        if not code:
            raise OAuthError("empty authorization code")
        if state and state != self._state:
            raise OAuthError("the pasted code belongs to a different log-in attempt (state mismatch): start again")
        status, body = await self.transport(self.app.token_url, {
            "grant_type": "authorization_code", "code": code, "state": state or self._state, "client_id": self.app.client_id,
            "redirect_uri": self.app.redirect_uri, "code_verifier": self._verifier})
        if status != 200:
            raise OAuthError(f"token exchange failed: {status} {str(body)[:200]}")
        self._verifier = self._state = None
        return self._take(body)

    async def refresh_tokens(self) -> OAuthTokens:
        old = self.tokens
        if old is None or not old.refresh_token:
            raise OAuthError("nothing to refresh: log in first")
        status, body = await self.transport(self.app.token_url, {"grant_type": "refresh_token", "refresh_token": old.refresh_token,
                                                                 "client_id": self.app.client_id})
        if status != 200:
            if 400 <= status < 500:            # refused, not unreachable: the grant is gone, and so is the stored copy
                self.storage.delete()
                self._tokens = None
            raise OAuthError(f"token refresh failed: {status}")
        return self._take(body, old.refresh_token)

    async def get_valid_access_token(self) -> str | None:
        """The access token, refreshed first when (nearly) expired; None when not logged in or the refresh failed.
        Concurrent callers share one refresh."""
        t = self.tokens
        if t is None:
            return None
        if t.is_expired(self.clock()):
            if self._refreshing is None:
                self._refreshing = asyncio.Lock()
            async with self._refreshing:
                t = self.tokens
                if t is not None and t.is_expired(self.clock()):
                    try:
                        t = await self.refresh_tokens()
                    except OAuthError:
                        return None
        return t.access_token if t else None

    def logout(self) -> None:
        self.storage.delete()
        self._tokens = None


async def login(client: OAuthClient, ask: Callable[[str], Awaitable[str]], out: Callable[[str], None] = print) -> OAuthTokens:
    """Interactive log-in: print the URL, wait for the pasted code, exchange it."""
    out(f"Open this URL, sign in, and paste the code shown afterwards:\n\n  {client.get_authorize_url()}\n")
    tokens = await client.exchange_code(await ask("code: "))
    out(f"logged in to {client.app.name}; the token is kept in {client.storage.path}")
    return tokens


def mask(secret: str | None, keep: int = 8) -> str:
    if not secret:
        return "(none)"
    return secret[:keep] + "…" if len(secret) > keep else "…"


def auth_report(provider: str, api_key_env: str, client: OAuthClient | None, env: dict[str, str] | None = None,
                now: float | None = None) -> tuple[str, list[str]]:
    """Which credential a request to ``provider`` will carry (rollouts/check_auth.py:19-126): ``("oauth" | "api_key" |
    "none", lines)``. A stored OAuth log-in wins over an API key in the environment, and the report says so, because the
    two are billed differently."""
    env = os.environ if env is None else env
    key = env.get(api_key_env, "") if api_key_env else ""
    lines = [f"{api_key_env or '(no key variable)'}: {mask(key)}"]
    tokens = client.tokens if client is not None else None
    if tokens is not None:
        left = tokens.expires_at - (time.time() if now is None else now)
        lines.append(f"OAuth log-in ({client.app.name}): {mask(tokens.access_token)} " +
                     (f"valid for {left / 60:.0f} more minutes" if left > 0 else "expired: refreshed on next use"))
    else:
        lines.append("OAuth log-in: none")
    using = "oauth" if tokens is not None else "api_key" if key else "none"
    lines.append({"oauth": f"requests to {provider} use the OAuth log-in (billed to the subscription)" +
                           ("; the API key in the environment is NOT used" if key else ""),
                  "api_key": f"requests to {provider} use the API key (billed to the API account)",
                  "none": f"no credential for {provider}: log in or set {api_key_env or 'an API key'}"}[using])
    return using, lines
