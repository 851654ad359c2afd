"""The evaluation "dev loop" behind the web front end (rollouts/frontend/server.py:47-1886): look at the configs of a
project, preview their datasets, write a new config from a form, launch a config as a child process, follow its output
while it runs, stop it, and read the results afterwards.

Everything here is plain Python on a project folder laid out as ::

    <project>/configs/NN_name.py     evaluation configs (what ``python -m research_b200.run_eval --config`` takes)
    <project>/data|datasets/         .jsonl / .csv / .json datasets
    <project>/results/<run>/         what runs wrote (results.json, report.json, *_results.jsonl)

so it is testable without a browser; ``frontend/server.py`` mounts it under ``/api/dev``. A config file is never
executed to be *looked at* (``describe_config`` reads its syntax tree); it runs only when launched, in a child
process of its own process group, and stopping a run signals exactly that group.
"""

from __future__ import annotations

import ast
import csv
import json
import os
import re
import signal
import subprocess
import sys
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

DATASET_SUFFIXES = (".jsonl", ".csv", ".json")
MAX_OUTPUT_LINES = 20_000


# ------------------------------------------------------------------------------------------- datasets
def preview_dataset(path: str | Path, n: int = 5) -> dict[str, Any]:
    """First ``n`` rows of a .jsonl / .csv / .json (list) file, the union of their field names in first-seen order, and
    the row count (lines for .jsonl and .csv, so huge files are counted without being parsed)."""
    p = Path(path)
    if not p.is_file():
        raise FileNotFoundError(p)
    rows: list[dict[str, Any]] = []
    if p.suffix == ".jsonl":
        total = 0
        with open(p) as f:
            for line in f:
                if not line.strip():
                    continue
                total += 1
                if len(rows) < n:
                    rows.append(json.loads(line))
    elif p.suffix == ".csv":
        with open(p, newline="") as f:
            reader = csv.DictReader(f)
            total = 0
            for row in reader:
                total += 1
                if len(rows) < n:
                    rows.append(dict(row))
    elif p.suffix == ".json":
        data = json.loads(p.read_text())
        if isinstance(data, dict):                                    # {"data": [...]} and the like: first list value
            data = next((v for v in data.values() if isinstance(v, list)), [data])
        total, rows = len(data), [r if isinstance(r, dict) else {"value": r} for r in data[:n]]
    else:
        raise ValueError(f"unsupported dataset type {p.suffix!r}: expected one of {DATASET_SUFFIXES}")
    fields: list[str] = []
    for r in rows:
        fields += [k for k in r if k not in fields]
    return {"path": str(p), "total_rows": total, "fields": fields, "rows": rows}


# ------------------------------------------------------------------------------------------- configs
def _literal(node: ast.AST) -> Any:
    try:
        return ast.literal_eval(node)
    except (ValueError, SyntaxError):
        return ast.unparse(node)


def describe_config(source: str) -> dict[str, Any]:
    """What a config file says, read from its syntax tree: top-level ``NAME = literal`` assignments, keyword arguments of
    top-level constructor calls (``config = Config(model_name=..., ...)`` -> ``config.model_name``), the names of the
    functions and classes it defines, the tools it declares (dict literals with a ``"name"`` and a ``"description"``),
    and the docstring."""
    tree = ast.parse(source)
    out: dict[str, Any] = {"doc": ast.get_docstring(tree) or "", "fields": {}, "functions": [], "classes": [], "tools": []}
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)):
            out["functions"].append(node.name)
        elif isinstance(node, ast.ClassDef):
            out["classes"].append(node.name)
            for sub in node.body:                                      # dataclass-style defaults: Class.field
                if isinstance(sub, ast.AnnAssign) and isinstance(sub.target, ast.Name) and sub.value is not None:
                    out["fields"][f"{node.name}.{sub.target.id}"] = _literal(sub.value)
        elif isinstance(node, (ast.Assign, ast.AnnAssign)):
            targets = node.targets if isinstance(node, ast.Assign) else [node.target]
            value = node.value
            if value is None or not all(isinstance(t, ast.Name) for t in targets):
                continue
            name = targets[0].id
            if isinstance(value, ast.Call):
                for kw in value.keywords:
                    if kw.arg:
                        out["fields"][f"{name}.{kw.arg}"] = _literal(kw.value)
            else:
                out["fields"][name] = _literal(value)
    for node in ast.walk(tree):
        if isinstance(node, ast.Dict):
            keys = [k.value for k in node.keys if isinstance(k, ast.Constant)]
            if "name" in keys and "description" in keys:
                d = _literal(node)
                if isinstance(d, dict):
                    out["tools"].append({"name": d.get("name"), "description": d.get("description"),
                                         "parameters": d.get("parameters", d.get("input_schema", {}))})
    return out


CONFIG_TEMPLATE = '''"""{doc}"""

from research_b200.agents.dtypes import Message, Trajectory
from research_b200.agents.presets import get_preset
from research_b200.frontend.devloop import load_rows, match_score

experiment_name = {experiment_name!r}
provider = {provider!r}
model_name = {model_name!r}
api_base = {api_base!r}
api_key_env_var = {api_key_env_var!r}
temperature = {temperature!r}
max_output_tokens = {max_output_tokens!r}
max_turns = {max_turns!r}
max_concurrent = {max_concurrent!r}
save_dir = {save_dir!r}

DATASET_PATH = {dataset_path!r}
NUM_SAMPLES = {num_samples!r}
PROMPT_FIELD = {prompt_field!r}
ANSWER_FIELD = {answer_field!r}
SYSTEM_PROMPT = {system_prompt!r}
PRESET = {preset!r}

rows = load_rows(DATASET_PATH, NUM_SAMPLES)


def environment():
    return get_preset(PRESET).environment(".") if PRESET else None


def to_trajectory(row):
    messages = ([Message("system", SYSTEM_PROMPT)] if SYSTEM_PROMPT else []) + [Message("user", {user_template!r}.format(**row))]
    return Trajectory(tuple(messages), metadata={{"answer": row.get(ANSWER_FIELD)}} if ANSWER_FIELD else {{}})


def score_fn(trajectory, row):
    return match_score(trajectory, row.get(ANSWER_FIELD)) if ANSWER_FIELD else 0.0


from types import SimpleNamespace

config = SimpleNamespace(**{{k: v for k, v in globals().items() if not k.startswith("_")}})
'''


def load_rows(path: str | Path, limit: int | None = None) -> list[dict[str, Any]]:
    """Rows of a dataset file for a generated config (all of them, or the first ``limit``)."""
    p = Path(path)
    if p.suffix == ".jsonl":
        rows = [json.loads(line) for line in p.read_text().splitlines() if line.strip()]
    elif p.suffix == ".csv":
        with open(p, newline="") as f:
            rows = [dict(r) for r in csv.DictReader(f)]
    else:
        data = json.loads(p.read_text())
        rows = data if isinstance(data, list) else next((v for v in data.values() if isinstance(v, list)), [])
    return rows[:limit] if limit else rows


def match_score(trajectory: Any, answer: Any) -> float:
    """1.0 when the last assistant message contains the expected answer (compared as text, case-insensitively; numbers
    also by value of the last number in the reply), else 0.0."""
    if answer is None:
        return 0.0
    reply = next((m.text() for m in reversed(trajectory.messages) if m.role == "assistant"), "")
    want = str(answer).strip().lower()
    if want and want in reply.lower():
        return 1.0
    nums = re.findall(r"-?\d+(?:\.\d+)?", reply.replace(",", ""))
    try:
        return float(bool(nums) and abs(float(nums[-1]) - float(want)) < 1e-6)
    except ValueError:
        return 0.0


def generate_config(data: dict[str, Any]) -> str:
    """Source of a ``run_eval`` config from the form's fields. ``user_template`` is a ``str.format`` template over the
    row's fields (default: the prompt field alone); every value is embedded with ``repr``, so no field can inject code."""
    prompt_field = data.get("prompt_field") or "prompt"
    d = {"doc": str(data.get("description") or f"Evaluation {data.get('experiment_name', 'experiment')}").replace('"""', "'''"),
         "experiment_name": str(data.get("experiment_name") or "experiment"), "provider": str(data.get("provider") or "openai"),
         "model_name": str(data.get("model_name") or ""), "api_base": str(data.get("api_base") or ""),
         "api_key_env_var": str(data.get("api_key_env_var") or ""), "temperature": float(data.get("temperature", 0.0)),
         "max_output_tokens": int(data.get("max_output_tokens", 1024)), "max_turns": int(data.get("max_turns", 1)),
         "max_concurrent": int(data.get("max_concurrent", 8)), "save_dir": str(data.get("save_dir") or "results"),
         "dataset_path": str(data.get("dataset_path") or ""), "num_samples": int(data["num_samples"]) if data.get("num_samples") else None,
         "prompt_field": prompt_field, "answer_field": data.get("answer_field") or None, "system_prompt": str(data.get("system_prompt") or ""),
         "preset": data.get("preset") or None, "user_template": str(data.get("user_template") or "{" + prompt_field + "}")}
    src = CONFIG_TEMPLATE.format(**d)
    ast.parse(src)                                                     # what is written must at least be Python
    return src


# ------------------------------------------------------------------------------------------- runs
@dataclass
class Run:
    run_id: str
    config_name: str
    argv: list[str]
    process: subprocess.Popen | None
    started_at: float
    status: str = "running"                  # running | completed | failed | killed
    exit_code: int | None = None
    lines: list[str] = field(default_factory=list)
    dropped: int = 0                         # lines discarded from the front once MAX_OUTPUT_LINES was reached
    result_dir: str | None = None

    def info(self) -> dict[str, Any]:
        return {"run_id": self.run_id, "config_name": self.config_name, "status": self.status, "exit_code": self.exit_code,
                "started_at": self.started_at, "elapsed_s": round(time.time() - self.started_at, 1) if self.status == "running" else None,
                "output_lines": self.dropped + len(self.lines), "pid": self.process.pid if self.process else None}


class RunRegistry:
    """Child processes started from the front end. Output is read by one thread per run into a bounded list; readers
    poll ``output(run_id, since)`` with the line number they have reached (what a server-sent-event stream does)."""

    def __init__(self) -> None:
        self.runs: dict[str, Run] = {}
        self._lock = threading.Lock()
        self._counter = 0

    def launch(self, config_name: str, argv: list[str], cwd: str | Path | None = None, env: dict[str, str] | None = None) -> Run:
        with self._lock:
            self._counter += 1
            run_id = f"run_{self._counter}_{int(time.time())}"
        p = subprocess.Popen(argv, cwd=str(cwd) if cwd else None, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                             bufsize=1, start_new_session=True)      # its own process group: kill() signals the group
        run = Run(run_id, config_name, argv, p, time.time())
        with self._lock:
            self.runs[run_id] = run
        threading.Thread(target=self._pump, args=(run,), daemon=True, name=f"devloop-{run_id}").start()
        return run

    def _pump(self, run: Run) -> None:
        assert run.process is not None and run.process.stdout is not None
        for line in run.process.stdout:
            with self._lock:
                run.lines.append(line.rstrip("\n"))
                if len(run.lines) > MAX_OUTPUT_LINES:
                    cut = len(run.lines) - MAX_OUTPUT_LINES
                    del run.lines[:cut]
                    run.dropped += cut
        code = run.process.wait()
        with self._lock:
            run.exit_code = code
            if run.status != "killed":
                run.status = "completed" if code == 0 else "failed"

    def output(self, run_id: str, since: int = 0) -> dict[str, Any]:
        """Lines from absolute line number ``since`` on, the number to ask with next, and whether the run is over."""
        with self._lock:
            run = self.runs[run_id]
            start = max(since - run.dropped, 0)
            return {"lines": list(run.lines[start:]), "next": run.dropped + len(run.lines), "status": run.status,
                    "exit_code": run.exit_code, "done": run.status != "running"}

    def wait(self, run_id: str, timeout: float = 60.0) -> Run:
        run = self.runs[run_id]
        deadline = time.monotonic() + timeout
        while run.status == "running" and time.monotonic() < deadline:
            time.sleep(0.02)
        return run

    def kill(self, run_id: str, grace_s: float = 3.0) -> bool:
        """SIGTERM to the run's process group, SIGKILL after ``grace_s`` if it is still there. False if it was over."""
        run = self.runs[run_id]
        p = run.process
        if p is None or p.poll() is not None:
            return False
        with self._lock:
            run.status = "killed"
        for sig, wait_s in ((signal.SIGTERM, grace_s), (signal.SIGKILL, 2.0)):
            try:
                os.killpg(p.pid, sig)                                   # pid == pgid (start_new_session)
            except ProcessLookupError:
                break
            try:
                p.wait(wait_s)
                break
            except subprocess.TimeoutExpired:
                continue
        return True

    def delete(self, run_id: str) -> bool:
        """Forget a finished run (a running one must be killed first)."""
        with self._lock:
            run = self.runs.get(run_id)
            if run is None or run.status == "running":
                return False
            del self.runs[run_id]
            return True

    def list(self) -> list[dict[str, Any]]:
        with self._lock:
            return [r.info() for r in sorted(self.runs.values(), key=lambda r: r.started_at, reverse=True)]


# ------------------------------------------------------------------------------------------- the project
class DevLoop:
    def __init__(self, project: str | Path, python: str = sys.executable):
        self.project = Path(project).resolve()
        self.python = python
        self.runs = RunRegistry()

    # ---- paths: names from requests never leave their folder
    def _inside(self, folder: Path, name: str, suffixes: tuple[str, ...] = ()) -> Path:
        p = (folder / name).resolve()
        if folder.resolve() not in p.parents or (suffixes and p.suffix not in suffixes):
            raise ValueError(f"not a name inside {folder.name}/: {name!r}")
        return p

    @property
    def configs_dir(self) -> Path:
        return self.project / "configs"

    @property
    def results_dir(self) -> Path:
        return self.project / "results"

    # ---- configs
    def list_configs(self) -> list[dict[str, Any]]:
        if not self.configs_dir.is_dir():
            return []
        return [{"name": f.stem, "file": f.name, "modified": f.stat().st_mtime, "size": f.stat().st_size}
                for f in sorted(self.configs_dir.glob("*.py")) if not f.name.startswith("_")]

    def load_config(self, name: str) -> dict[str, Any]:
        f = self._inside(self.configs_dir, name if name.endswith(".py") else name + ".py", (".py",))
        source = f.read_text()
        try:
            described = describe_config(source)
        except SyntaxError as e:
            described = {"error": f"syntax error at line {e.lineno}: {e.msg}"}
        return {"name": f.stem, "source": source, **described}

    def next_config_name(self, stem: str) -> str:
        """``NN_stem`` with NN one above the highest number in use (configs sort in creation order)."""
        nums = [int(m.group(1)) for c in self.list_configs() if (m := re.match(r"(\d+)_", c["name"]))]
        clean = re.sub(r"[^a-zA-Z0-9_]+", "_", stem).strip("_") or "config"
        return f"{max(nums, default=0) + 1:02d}_{clean}"

    def save_config(self, data: dict[str, Any], name: str | None = None, overwrite: bool = False) -> dict[str, Any]:
        source = data["source"] if "source" in data else generate_config(data)
        ast.parse(source)
        name = name or self.next_config_name(str(data.get("experiment_name") or "config"))
        f = self._inside(self.configs_dir, name + ".py", (".py",))
        if f.exists() and not overwrite:
            raise FileExistsError(f"{f.name} exists")
        f.parent.mkdir(parents=True, exist_ok=True)
        f.write_text(source)
        return {"name": name, "file": str(f), "source": source}

    def dataset_preview_for_config(self, name: str, n: int = 5) -> dict[str, Any]:
        fields = self.load_config(name).get("fields", {})
        path = next((v for k, v in fields.items() if isinstance(v, str) and k.split(".")[-1].lower() in ("dataset_path", "data_path")), None)
        if not path:
            raise ValueError(f"config {name} names no dataset_path")
        p = Path(path)
        return preview_dataset(p if p.is_absolute() else self.project / p, n)

    # ---- datasets, models
    def list_datasets(self) -> list[dict[str, Any]]:
        out = []
        for folder in ("data", "datasets"):
            d = self.project / folder
            if d.is_dir():
                out += [{"path": str(f.relative_to(self.project)), "size": f.stat().st_size, "type": f.suffix[1:]}
                        for f in sorted(d.rglob("*")) if f.is_file() and f.suffix in DATASET_SUFFIXES]
        return out

    def preview(self, rel_path: str, n: int = 5) -> dict[str, Any]:
        p = (self.project / rel_path).resolve()
        if self.project not in p.parents:
            raise ValueError("dataset path leaves the project")
        return preview_dataset(p, n)

    @staticmethod
    def list_models() -> dict[str, list[dict[str, Any]]]:
        from ..agents.providers.models import get_models, get_providers

        return {prov: [{"name": m.name, "context_window": m.context_window, "supports_tools": m.supports_tools,
                        "input_per_mtok": m.input_per_mtok, "output_per_mtok": m.output_per_mtok} for m in get_models(prov)]
                for prov in get_providers()}

    # ---- results
    def list_traces(self) -> list[dict[str, Any]]:
        if not self.results_dir.is_dir():
            return []
        out = []
        for d in sorted((p for p in self.results_dir.iterdir() if p.is_dir()), key=lambda p: p.stat().st_mtime, reverse=True):
            summary = self._summary(d)
            if summary is not None:
                out.append({"id": d.name, "modified": d.stat().st_mtime, "summary": summary})
        return out

    @staticmethod
    def _summary(d: Path) -> dict[str, Any] | None:
        for name, key in (("results.json", "summary"), ("report.json", "summary")):
            f = d / name
            if f.is_file():
                try:
                    return json.loads(f.read_text()).get(key, {})
                except ValueError:
                    return {"error": f"{name} is not valid JSON"}
        return {} if any(d.glob("*_results.jsonl")) else None

    def get_trace(self, trace_id: str, limit: int = 200) -> dict[str, Any]:
        d = self._inside(self.results_dir, trace_id)
        if not d.is_dir():
            raise FileNotFoundError(trace_id)
        samples: list[Any] = []
        if (d / "results.json").is_file():
            samples = json.loads((d / "results.json").read_text()).get("results", [])
        elif (d / "samples.jsonl").is_file():
            samples = [json.loads(line) for line in (d / "samples.jsonl").read_text().splitlines() if line.strip()]
        else:
            for f in sorted(d.glob("*_results.jsonl")):
                samples += [json.loads(line) for line in f.read_text().splitlines() if line.strip()]
        return {"id": trace_id, "summary": self._summary(d) or {}, "total": len(samples), "samples": samples[:limit]}

    # ---- launching
    def launch(self, name: str, extra_args: list[str] | None = None) -> dict[str, Any]:
        f = self._inside(self.configs_dir, name if name.endswith(".py") else name + ".py", (".py",))
        if not f.is_file():
            raise FileNotFoundError(f.name)
        env = dict(os.environ, PYTHONUNBUFFERED="1")
        root = str(Path(__file__).resolve().parents[2])                # the checkout this package runs from
        env["PYTHONPATH"] = root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
        argv = [self.python, "-m", "research_b200.run_eval", "--config", str(f), *(extra_args or [])]
        return self.runs.launch(f.stem, argv, cwd=self.project, env=env).info()
