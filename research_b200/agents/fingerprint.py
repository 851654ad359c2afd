"""Fingerprints of evaluation and session configurations (rollouts/fingerprint.py:37-314).

A fingerprint answers two questions about a stored result: *was it produced with the same configuration?*
(``config_hash``: a stable hash of what determines the outcome: endpoint without credentials, the names of the scoring
and message-building functions, sample limit, a checksum of the dataset) and *with the same code?* (``git_sha`` and
whether the tree was dirty). Function bodies are not hashed: the commit is the authority on code, which is why an
evaluation refuses a dirty tree unless told otherwise and why lambdas (whose names say nothing) are refused for the
functions that matter.
"""

from __future__ import annotations

import hashlib
import json
import subprocess
import sys
from dataclasses import asdict, is_dataclass
from pathlib import Path
from typing import Any, Callable


# ------------------------------------------------------------------------------------------- pieces
def canonical_json(obj: Any) -> str:
    """Deterministic JSON: sorted keys, no whitespace, non-JSON values through ``repr``-free ``str``."""
    return json.dumps(obj, sort_keys=True, separators=(",", ":"), default=str)


def hash_str(s: str) -> str:
    return hashlib.sha256(s.encode()).hexdigest()[:16]


def git_info(cwd: str | Path | None = None) -> tuple[str, bool]:
    """``(short sha, dirty)`` of the repository that holds ``cwd`` (default: this package); ``("unknown", False)``
    outside a repository or without git."""
    where = str(cwd or Path(__file__).resolve().parent)
    try:
        sha = subprocess.run(["git", "rev-parse", "--short", "HEAD"], cwd=where, capture_output=True, text=True, timeout=5)
        if sha.returncode != 0:
            return "unknown", False
        status = subprocess.run(["git", "status", "--porcelain"], cwd=where, capture_output=True, text=True, timeout=10)
        return sha.stdout.strip(), bool(status.stdout.strip()) if status.returncode == 0 else False
    except (OSError, subprocess.SubprocessError):
        return "unknown", False


def require_clean_git(*, allow_dirty: bool = False, cwd: str | Path | None = None) -> tuple[str, bool]:
    """``git_info`` that raises on uncommitted changes unless ``allow_dirty``: a result labelled with a commit must
    come from that commit."""
    sha, dirty = git_info(cwd)
    if dirty and not allow_dirty:
        raise RuntimeError(f"uncommitted changes on top of {sha}: commit them, or pass allow_dirty=True and accept that the "
                           "fingerprint's commit does not describe the code that ran")
    return sha, dirty


def callable_name(fn: Callable[..., Any], *, allow_lambda: bool = False) -> str:
    """``module.qualname``. Lambdas are refused unless allowed: every lambda of a module has the same name."""
    module = getattr(fn, "__module__", "") or ""
    qual = getattr(fn, "__qualname__", None) or getattr(fn, "__name__", None) or type(fn).__qualname__
    if getattr(fn, "__name__", "") == "<lambda>" and not allow_lambda:
        raise ValueError(f"a lambda cannot be fingerprinted (its name says nothing): define a named function instead of {module}.{qual}")
    return f"{module}.{qual}" if module else qual


def file_checksum(path: str | Path, max_bytes: int = 1 << 20) -> str:
    """Hash of the first ``max_bytes`` of a file plus its size (``"missing"`` if it cannot be read)."""
    try:
        p = Path(path)
        with open(p, "rb") as f:
            head = f.read(max_bytes)
        return hashlib.sha256(head + str(p.stat().st_size).encode()).hexdigest()[:16]
    except OSError:
        return "missing"


def fingerprint_short(fp: dict[str, Any]) -> str:
    """``confighash@gitsha`` with a ``*`` for a dirty tree."""
    return f"{str(fp.get('config_hash', '????????'))[:8]}@{fp.get('git_sha', 'unknown')}{'*' if fp.get('git_dirty') else ''}"


def _plain(obj: Any) -> Any:
    if is_dataclass(obj) and not isinstance(obj, type):
        return asdict(obj)
    return obj


# ------------------------------------------------------------------------------------------- evaluations
def fingerprint_eval(config, tools: list[str] | None = None, dataset_path: str | Path | None = None, allow_dirty: bool = False,
                     cwd: str | Path | None = None) -> dict[str, Any]:
    """Fingerprint of an evaluation (``agents.dtypes.EvalConfig``): endpoint minus credentials, the names of
    ``score_fn`` / ``prepare_messages`` / ``environment_factory`` / the stop handler, ``max_samples`` and ``max_turns``,
    and the dataset's checksum. ``tools`` (what the environment actually offered) is recorded beside the hash."""
    sha, dirty = require_clean_git(allow_dirty=allow_dirty, cwd=cwd)
    ep = dict(_plain(config.endpoint))
    for k in [k for k in ep if "key" in k.lower() or "token" in k.lower() or "secret" in k.lower()]:
        ep.pop(k)
    cfg: dict[str, Any] = {"endpoint": ep, "score_fn": callable_name(config.score_fn), "max_samples": config.max_samples,
                           "max_turns": getattr(config, "max_turns", None)}
    if getattr(config, "prepare_messages", None) is not None:
        cfg["prepare_messages"] = callable_name(config.prepare_messages)
    if getattr(config, "environment_factory", None) is not None:
        cfg["environment_factory"] = callable_name(config.environment_factory, allow_lambda=True)
    stop = getattr(getattr(config, "run_config", None), "handle_stop", None)
    if stop is not None:
        cfg["handle_stop"] = callable_name(stop, allow_lambda=True)
    if dataset_path is not None:
        cfg["dataset_checksum"], cfg["dataset_path"] = file_checksum(dataset_path), str(dataset_path)
    return {"config_hash": hash_str(canonical_json(cfg)), "git_sha": sha, "git_dirty": dirty, "domain": "eval",
            "endpoint_summary": f"{config.endpoint.provider}/{config.endpoint.model}", "tools": sorted(tools or []),
            "dataset_path": str(dataset_path) if dataset_path is not None else None}


# ------------------------------------------------------------------------------------------- sessions
def fingerprint_session(model: str, env: str, tools: list[str], system_prompt: str | None = None,
                        cwd: str | Path | None = None) -> dict[str, Any]:
    """Fingerprint of an interactive session: model, environment name, tool names and a hash of the system prompt
    (the prompt itself is not stored). A dirty tree is normal while working and only recorded."""
    cfg: dict[str, Any] = {"model": model, "env": env, "tools": sorted(tools)}
    if system_prompt:
        cfg["system_prompt_hash"] = hash_str(system_prompt)
    sha, dirty = git_info(cwd)
    return {"config_hash": hash_str(canonical_json(cfg)), "git_sha": sha, "git_dirty": dirty, "domain": "session", "model": model,
            "env": env, "tools": sorted(tools)}


# ------------------------------------------------------------------------------------------- comparison
def compare_fingerprints(a: dict[str, Any], b: dict[str, Any]) -> dict[str, Any]:
    return {"same_config": a.get("config_hash") == b.get("config_hash"), "same_code": a.get("git_sha") == b.get("git_sha") and
            not (a.get("git_dirty") or b.get("git_dirty")), "a": fingerprint_short(a), "b": fingerprint_short(b)}


def warn_if_changed(saved: dict[str, Any] | None, current: dict[str, Any], context: str = "", file=None) -> bool:
    """On resume: say (on stderr) when the configuration or, with the same configuration, the code has changed since
    ``context`` was created. Returns True if anything was said; records without a fingerprint are left alone."""
    if not saved:
        return False
    out = file or sys.stderr
    said = False
    if saved.get("config_hash") and current.get("config_hash") and saved["config_hash"] != current["config_hash"]:
        print(f"warning: the configuration changed since {context or 'this record'} was created\n"
              f"  saved:   {fingerprint_short(saved)}\n  current: {fingerprint_short(current)}", file=out)
        said = True
    elif saved.get("git_sha") and current.get("git_sha") and saved["git_sha"] != current["git_sha"]:
        print(f"note: code version changed since {context or 'this record'}: {saved['git_sha']} -> {current['git_sha']}", file=out)
        said = True
    return said
