"""Generic evaluation entry point driven by a config file (rollouts/run_eval.py:32-395).

    python -m research_b200.run_eval --config my_eval_config.py [--output result.json] [--workspace-root DIR]

The config file defines ``config``, an object with

* a dataset: ``load_dataset(...) -> list[dict]`` plus ``dataset.dataset_path`` / ``dataset.annotation_files`` and
  optional ``filters`` (``platforms`` / ``applications`` / ``ui_types`` / ``limit``) — every annotation file is loaded
  with the filters, the global limit is applied afterwards — or simply ``rows`` (a list of dicts);
* a model: either ``model`` satisfying ``config.protocols.HasModelConfig`` or the flat fields ``provider``,
  ``model_name``, ``api_base``, ``temperature``, ``max_output_tokens`` (+ ``api_key_env_var``);
* ``environment``: a zero-argument factory of the environment every sample runs in (may be ``None``);
* ``to_trajectory(row) -> Trajectory``: the conversation a sample starts from (its ``metadata`` travels into the result);
* optionally ``score_fn(trajectory, row)``; without one, an environment with ``compute_reward(text, bbox, img_size)``
  scores samples whose trajectory metadata carries ``bbox`` and ``img_size`` (the screen-grounding case of the
  reference), anything else gets reward 0;
* ``experiment_name``, ``max_concurrent`` (default 10), ``max_turns``, ``save_jsonl``, ``save_dir``.

Every sample runs through the agent loop under a concurrency limit; a failing sample is recorded with its error and
does not stop the run; results stream to ``<result_dir>/<experiment>_results.jsonl`` as they finish. Returns / writes
``{"summary": {...}, "results": [...]}``. Remote model providers need their API key in the environment; the check
happens before any sample runs. asyncio replaces the reference's trio nursery.
"""

from __future__ import annotations

import argparse
import asyncio
import inspect
import json
import logging
import os
import sys
import time
from pathlib import Path
from typing import Any

from .agents.agents import run_agent
from .agents.dtypes import Actor, AgentState, Endpoint, RunConfig, Score, Trajectory
from .config.loader import load_config_from_file as _load_plain
from .config.protocols import HasModelConfig

logger = logging.getLogger(__name__)

PROVIDER_KEYS = {"openai": "OPENAI_API_KEY", "anthropic": "ANTHROPIC_API_KEY", "gemini": "GEMINI_API_KEY",
                 "google": "GOOGLE_API_KEY"}


def load_config_from_file(config_path: Path | str, workspace_root: Path | str | None = None) -> Any:
    """Load ``config`` from a Python file. With ``workspace_root`` (a checkout deployed elsewhere, e.g. by a remote
    push), relative dataset paths of the config are resolved against it and the root joins ``sys.path`` so that the
    config's own imports work."""
    if workspace_root is not None:
        root = str(Path(workspace_root).resolve())
        if root not in sys.path:
            sys.path.insert(0, root)
    cfg = _load_plain(config_path, "config")
    ds = getattr(cfg, "dataset", None)
    if workspace_root is not None and ds is not None and hasattr(ds, "dataset_path"):
        p = Path(ds.dataset_path)
        if not p.is_absolute():
            try:
                object.__setattr__(ds, "dataset_path", Path(workspace_root) / p)
            except Exception:  # noqa: BLE001 - a config that forbids the rewrite keeps its path
                logger.warning("could not rebase dataset path %s onto %s", p, workspace_root)
    return cfg


def _load_rows(config: Any) -> list[dict]:
    if getattr(config, "rows", None) is not None:
        rows = list(config.rows)
    else:
        assert getattr(config, "load_dataset", None) is not None, "config must define load_dataset (or rows)"
        ds = config.dataset
        assert Path(ds.dataset_path).exists(), f"dataset not found: {ds.dataset_path}"
        flt = getattr(config, "filters", None)
        rows = []
        accepted = set(inspect.signature(config.load_dataset).parameters)
        for ann in getattr(ds, "annotation_files", None) or [None]:
            kw = {"data_path": ds.dataset_path, "annotation_file": ann, "limit": None}
            for name in ("platforms", "applications", "ui_types"):
                kw[name] = (getattr(flt, name, None) or None) if flt is not None else None
            takes_kwargs = any(p.kind is inspect.Parameter.VAR_KEYWORD for p in inspect.signature(config.load_dataset).parameters.values())
            part = config.load_dataset(**(kw if takes_kwargs else {k: v for k, v in kw.items() if k in accepted}))
            logger.debug("loaded %d samples from %s", len(part), ann)
            rows.extend(part)
    limit = getattr(getattr(config, "filters", None), "limit", None)
    if limit is None:
        limit = getattr(config, "limit", None)
    return rows[:limit] if limit is not None else rows


def endpoint_from_config(config: Any) -> Endpoint:
    model = getattr(config, "model", None)
    if model is not None and isinstance(model, HasModelConfig):
        return model.to_endpoint()
    env_var = getattr(model, "api_key_env_var", None) or getattr(config, "api_key_env_var", None)
    key = os.getenv(env_var, "") if env_var else ""
    if env_var:
        logger.info("api key from %s: %s", env_var, ("***" + key[-4:]) if key else "NOT FOUND")
    return Endpoint(provider=config.provider, model=config.model_name, api_base=getattr(config, "api_base", ""), api_key=key,
                    temperature=getattr(config, "temperature", 1.0), max_tokens=getattr(config, "max_output_tokens", 1024),
                    engine=getattr(config, "engine", None))


def _reward(config: Any, environment: Any, trajectory: Trajectory, final_text: Any, row: dict) -> float:
    fn = getattr(config, "score_fn", None)
    if fn is not None:
        s = fn(trajectory, row)
        return float(s.reward) if isinstance(s, Score) else float(s)
    meta = getattr(trajectory, "metadata", None) or {}
    if environment is not None and hasattr(environment, "compute_reward") and "bbox" in meta and "img_size" in meta:
        return float(environment.compute_reward(final_text, meta["bbox"], meta["img_size"]))
    return 0.0


async def run_evaluation(config: Any, result_dir: Path | str) -> dict:
    """Run every sample of the config's dataset; see the module docstring for what the config provides."""
    result_dir = Path(result_dir)
    result_dir.mkdir(parents=True, exist_ok=True)
    rows = _load_rows(config)
    logger.info("total: %d samples", len(rows))
    endpoint = endpoint_from_config(config)
    logger.info("endpoint: %s @ %s, model %s", endpoint.provider, endpoint.api_base, endpoint.model)
    factory = getattr(config, "environment", None)
    to_trajectory = getattr(config, "to_trajectory", None)
    assert to_trajectory is not None, "config must define to_trajectory(row)"
    max_concurrent = int(getattr(config, "max_concurrent", 10))
    max_turns = int(getattr(config, "max_turns", 10))
    sem = asyncio.Semaphore(max_concurrent)
    results: list[dict | None] = [None] * len(rows)
    name = getattr(config, "experiment_name", "evaluation")
    jsonl = open(result_dir / f"{name}_results.jsonl", "w") if getattr(config, "save_jsonl", True) else None
    lock = asyncio.Lock()
    done = 0
    t_start = time.time()

    async def record(i: int, result: dict) -> None:
        nonlocal done
        results[i] = result
        done += 1
        if jsonl is not None:
            async with lock:
                jsonl.write(json.dumps(result, default=str) + "\n")
                jsonl.flush()
        if getattr(config, "show_progress", True):
            print(f"\r[{done}/{len(rows)}] last reward {result.get('reward', 0.0):.3f}", end="", file=sys.stderr, flush=True)

    async def run_sample(i: int, row: dict) -> None:
        async with sem:
            try:
                traj = to_trajectory(row)
                env = factory() if factory is not None else None
                if asyncio.iscoroutine(env):
                    env = await env
                state = AgentState(Actor(traj, endpoint), env, max_turns=max_turns)
                final = (await run_agent(state, getattr(config, "run_config", None) or RunConfig()))[-1]
                msgs = final.actor.trajectory.messages
                text = msgs[-1].content if msgs else ""
                reward = _reward(config, env, final.actor.trajectory, text, row)
                res = {"sample_id": i, "response": text if isinstance(text, str) else str(text), "turns": final.turn_idx,
                       "reward": reward, "stop_reason": final.stop.value if final.stop else None, "success": final.stop is not None}
                meta = getattr(traj, "metadata", None)
                if meta:
                    res["metadata"] = meta
            except Exception as e:  # noqa: BLE001 - one failing sample must not stop the evaluation
                logger.exception("sample %d/%d failed: %s", i + 1, len(rows), e)
                res = {"sample_id": i, "error": f"{type(e).__name__}: {e}", "success": False}
            await record(i, res)

    try:
        await asyncio.gather(*[run_sample(i, r) for i, r in enumerate(rows)])
    finally:
        if jsonl is not None:
            jsonl.close()
        if getattr(config, "show_progress", True):
            print(file=sys.stderr)
    completed = sum(1 for r in results if r and r.get("success"))
    total_reward = sum(r.get("reward", 0.0) for r in results if r and "reward" in r)
    summary = {"experiment_name": name, "total_samples": len(rows), "completed": completed, "errors": len(rows) - completed,
               "mean_reward": total_reward / completed if completed else 0.0, "total_reward": total_reward,
               "wall_s": round(time.time() - t_start, 2)}
    logger.info("summary: %s", summary)
    return {"summary": summary, "results": results}


def check_api_key(provider: str) -> str | None:
    """Name of the environment variable a remote provider needs but that is unset, else None."""
    var = PROVIDER_KEYS.get(provider.lower())
    return var if (var is not None and not os.getenv(var)) else None


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Run an evaluation described by a config file")
    ap.add_argument("--config", type=Path, required=True, help="Python file that defines `config`")
    ap.add_argument("--output", type=Path, help="output JSON file (default: <save_dir>/<experiment>_<timestamp>/results.json)")
    ap.add_argument("--workspace-root", type=Path, help="root against which the config's relative paths are resolved")
    args = ap.parse_args(argv)
    config = load_config_from_file(args.config, args.workspace_root)
    if getattr(config, "to_trajectory", None) is None:
        print("config lacks to_trajectory(row): nothing to run", file=sys.stderr)
        return 1
    endpoint = endpoint_from_config(config)
    missing = check_api_key(endpoint.provider) if not endpoint.api_key else None
    if missing:
        print(f"error: provider '{endpoint.provider}' needs {missing} in the environment", file=sys.stderr)
        return 1
    from .utils.logging_config import setup_logging

    name = getattr(config, "experiment_name", "evaluation")
    result_dir = Path(getattr(config, "save_dir", "results")) / f"{name}_{time.strftime('%Y%m%d-%H%M%S')}"
    result_dir.mkdir(parents=True, exist_ok=True)
    setup_logging(log_file=result_dir / "eval.log")
    out = asyncio.run(run_evaluation(config, result_dir))
    path = args.output or (result_dir / "results.json")
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(out, indent=2, default=str))
    print(json.dumps(out["summary"]))
    return 0 if out["summary"]["errors"] == 0 else 2


if __name__ == "__main__":
    raise SystemExit(main())
