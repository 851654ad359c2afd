"""Load a config object from a Python file and check it against the protocols (rollouts/config/loader.py:14-103)."""

from __future__ import annotations

import importlib.util
import inspect
import sys
from pathlib import Path
from typing import Any


def load_config_from_file(config_path: str | Path, config_name: str = "config") -> Any:
    """Execute ``config_path`` as a module and return its ``config_name`` attribute. The file's directory is on
    ``sys.path`` while it runs, so a config may import helpers that sit beside it."""
    path = Path(config_path).resolve()
    if not path.exists():
        raise FileNotFoundError(f"config file not found: {path}")
    if path.suffix != ".py":
        raise ValueError(f"config must be a .py file: {path}")
    spec = importlib.util.spec_from_file_location(f"_rb_config_{path.stem}", path)
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot import {path}")
    module = importlib.util.module_from_spec(spec)
    sys.path.insert(0, str(path.parent))
    try:
        spec.loader.exec_module(module)
    finally:
        sys.path.remove(str(path.parent))
    if not hasattr(module, config_name):
        raise AttributeError(f"{path} defines no '{config_name}' (found: {[n for n in vars(module) if not n.startswith('_')][:12]})")
    return getattr(module, config_name)


def validate_config_protocol(config: Any, protocol_class: type) -> list[str]:
    """Names of the protocol's members that ``config`` lacks (empty list = it satisfies the protocol)."""
    wanted = [n for n, _ in inspect.getmembers(protocol_class) if not n.startswith("_")]
    wanted += [n for n in getattr(protocol_class, "__annotations__", {}) if n not in wanted]
    missing = []
    for name in wanted:
        if not hasattr(config, name):
            missing.append(name)
        elif callable(getattr(protocol_class, name, None)) and not callable(getattr(config, name)):
            missing.append(f"{name} (not callable)")
    return missing
