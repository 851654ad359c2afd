"""Argument checks for the remote-execution helpers (shared/shared/validation.py:14-190): each returns the
normalised value or raises ``ValueError`` naming what is wrong."""

from __future__ import annotations

import os
import re
import stat


def validate_port(port: int) -> int:
    if isinstance(port, bool) or not isinstance(port, int) or not 1 <= port <= 65535:
        raise ValueError(f"port must be an integer in 1..65535, got {port!r}")
    return port


def validate_timeout(timeout: int | float, min_value: float = 1, max_value: float = 3600) -> int | float:
    if isinstance(timeout, bool) or not isinstance(timeout, (int, float)) or not min_value <= timeout <= max_value:
        raise ValueError(f"timeout must be a number in {min_value}..{max_value} seconds, got {timeout!r}")
    return timeout


_HOST = re.compile(r"^(?=.{1,253}$)([A-Za-z0-9]([A-Za-z0-9-]{0,61}[A-Za-z0-9])?)(\.[A-Za-z0-9]([A-Za-z0-9-]{0,61}[A-Za-z0-9])?)*$")
_IPV6 = re.compile(r"^[0-9A-Fa-f:]+$")


def validate_hostname(hostname: str) -> str:
    h = (hostname or "").strip()
    if not h or not (_HOST.match(h) or (":" in h and _IPV6.match(h))):
        raise ValueError(f"not a host name or address: {hostname!r}")
    return h


def validate_username(username: str) -> str:
    u = (username or "").strip()
    if not re.match(r"^[A-Za-z_][A-Za-z0-9_.-]{0,31}\$?$", u):
        raise ValueError(f"not a login name: {username!r}")
    return u


def validate_ssh_key_path(path: str, check_permissions: bool = True) -> str:
    """Expanded path of a private key that exists, is a file and (optionally) is not readable by group / others."""
    p = os.path.abspath(os.path.expanduser(path or ""))
    if not os.path.isfile(p):
        raise ValueError(f"ssh key not found: {path!r}")
    if check_permissions and stat.S_IMODE(os.stat(p).st_mode) & 0o077:
        raise ValueError(f"ssh key {p} is accessible by group or others (chmod 600)")
    return p


def parse_ssh_target(target: str) -> tuple[str, str, int]:
    """``user@host[:port]`` -> (user, host, port)."""
    m = re.match(r"^(?P<u>[^@]+)@(?P<h>[^:]+|\[[^\]]+\])(:(?P<p>\d+))?$", (target or "").strip())
    if not m:
        raise ValueError(f"expected user@host[:port], got {target!r}")
    host = m["h"].strip("[]")
    return validate_username(m["u"]), validate_hostname(host), validate_port(int(m["p"] or 22))
