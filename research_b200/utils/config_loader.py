"""Experiment configs are Python files that define ``config`` (frozen dataclasses derived with
``dataclasses.replace``): ``load_config_from_file`` executes one and returns that object
(rollouts/config/loader.py:14-65); ``fingerprint`` hashes a config together with the git state
(rollouts/fingerprint.py:168-296)."""

from __future__ import annotations

import hashlib
import importlib.util
import json
import subprocess
from dataclasses import asdict, is_dataclass
from pathlib import Path
from typing import Any


def load_config_from_file(path: str | Path, attr: str = "config") -> Any:
    path = Path(path)
    assert path.exists(), f"config file {path} not found"
    spec = importlib.util.spec_from_file_location(f"_rb_config_{path.stem}", path)
    assert spec is not None and spec.loader is not None
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert hasattr(mod, attr), f"{path} does not define `{attr}`"
    return getattr(mod, attr)


def config_to_dict(cfg: Any) -> Any:
    if is_dataclass(cfg) and not isinstance(cfg, type):
        return {k: config_to_dict(v) for k, v in asdict(cfg).items()}
    if isinstance(cfg, dict):
        return {str(k): config_to_dict(v) for k, v in cfg.items()}
    if isinstance(cfg, (list, tuple)):
        return [config_to_dict(v) for v in cfg]
    if isinstance(cfg, (str, int, float, bool)) or cfg is None:
        return cfg
    return getattr(cfg, "__name__", repr(cfg))


def git_state(cwd: str | Path | None = None) -> dict[str, Any]:
    def run(*a: str) -> str:
        try:
            return subprocess.run(["git", *a], cwd=cwd, capture_output=True, text=True, timeout=5).stdout.strip()
        except (OSError, subprocess.TimeoutExpired):
            return ""

    return {"commit": run("rev-parse", "HEAD"), "dirty": bool(run("status", "--porcelain"))}


def fingerprint(cfg: Any, include_git: bool = True, cwd: str | Path | None = None) -> dict[str, Any]:
    d = config_to_dict(cfg)
    payload = json.dumps(d, sort_keys=True)
    out = {"config_hash": hashlib.sha256(payload.encode()).hexdigest()[:16], "config": d}
    if include_git:
        out["git"] = git_state(cwd)
    return out
