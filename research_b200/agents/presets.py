"""Named agent configurations: system prompt + environment factory + turn budget
(rollouts/agent_presets/)."""

from __future__ import annotations

import importlib
import importlib.util
import json
import re
import sys
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Callable

from .environments import (AskUserQuestionEnvironment, BasicEnvironment, BrowsingEnvironment, CalculatorEnvironment,
                           ComposedEnvironment, GitWorktreeEnvironment, LocalFilesystemEnvironment, REPLEnvironment)


@dataclass(frozen=True)
class AgentPreset:
    name: str
    description: str
    system_prompt: str
    environment: Callable[[str], Any]       # working directory -> environment
    max_turns: int = 30


_CODING = ("You are a careful software engineer working in the user's repository. Read before you edit, make the "
           "smallest change that solves the task, run the tests, and say plainly what you verified and what you did not.")

PRESETS: dict[str, AgentPreset] = {p.name: p for p in [
    AgentPreset("chat", "plain conversation, no tools", "You are a helpful assistant.", lambda cwd: BasicEnvironment(), 1),
    AgentPreset("calculator", "arithmetic with a calculator tool", "Use the calculator for every computation.",
                lambda cwd: CalculatorEnvironment(), 10),
    AgentPreset("coding", "read / write / edit / bash in the working directory", _CODING,
                lambda cwd: LocalFilesystemEnvironment(cwd), 50),
    AgentPreset("coding-git", "coding in a per-session git worktree with automatic commits", _CODING,
                lambda cwd: GitWorktreeEnvironment(cwd), 50),
    AgentPreset("coding-interactive", "coding plus questions to the user", _CODING + " Ask when requirements are ambiguous.",
                lambda cwd: ComposedEnvironment([LocalFilesystemEnvironment(cwd), AskUserQuestionEnvironment()]), 50),
    AgentPreset("research", "web search / fetch and a Python scratchpad",
                "Answer with sources. Search, read the pages you cite, compute with the REPL when numbers matter.",
                lambda cwd: ComposedEnvironment([BrowsingEnvironment(), REPLEnvironment()]), 30),
]}


# ------------------------------------------------------------------------------------------- presets as files
# environment names a preset file (and the command line) may use -> factory(working directory, tool preset)
ENVIRONMENTS: dict[str, Callable[[str, Any], Any]] = {
    "none": lambda cwd, tools: BasicEnvironment(),
    "calculator": lambda cwd, tools: CalculatorEnvironment(),
    "coding": lambda cwd, tools: LocalFilesystemEnvironment(cwd, tools=tools or "full"),
    "git": lambda cwd, tools: GitWorktreeEnvironment(cwd),
    "coding-interactive": lambda cwd, tools: ComposedEnvironment([LocalFilesystemEnvironment(cwd, tools=tools or "full"), AskUserQuestionEnvironment()]),
    "browsing": lambda cwd, tools: BrowsingEnvironment(),
    "repl": lambda cwd, tools: REPLEnvironment(),
    "research": lambda cwd, tools: ComposedEnvironment([BrowsingEnvironment(), REPLEnvironment()]),
    "ask_user": lambda cwd, tools: AskUserQuestionEnvironment(),
}


def environment_from_spec(spec: str, cwd: str = ".", tools: Any = None) -> Any:
    """``coding`` or ``coding+ask_user+browsing``: one environment, or the composition of several (``+`` as on the command
    line of the reference: rollouts/toolslash_spec.md). Unknown names are an error that lists the known ones."""
    from .environments import compose

    names = [n.strip() for n in spec.split("+") if n.strip()]
    if not names:
        raise KeyError("empty environment spec")
    unknown = [n for n in names if n not in ENVIRONMENTS]
    if unknown:
        raise KeyError(f"unknown environment(s) {unknown}; available: {sorted(ENVIRONMENTS)}")
    if len(set(names)) != len(names):
        raise KeyError(f"an environment appears twice in {spec!r}")
    built = [ENVIRONMENTS[n](cwd, tools) for n in names]
    return built[0] if len(built) == 1 else compose(*built)
PRESET_DIR = Path(__file__).resolve().parent / "preset_files"
USER_PRESET_DIR = Path.home() / ".research_b200" / "presets"


@dataclass(frozen=True)
class AgentPresetConfig:
    """A preset as data (rollouts/agent_presets/base_preset.py:17-82): model, environment name and system prompt, kept in
    a Python file ``<name>_<id>_<parent id>.py`` that exports ``config``. A variant imports its parent's ``config`` and
    changes fields with ``dataclasses.replace``, so the file name records the lineage and the file the difference."""

    name: str
    model: str                              # "provider/model"
    env: str                                # a key of ENVIRONMENTS
    system_prompt: str
    thinking: bool = True
    temperature: float | None = None
    working_dir: Path | None = None
    tools: str | None = None                # tool preset of the coding environment: full | readonly | no-write
    max_turns: int = 50
    description: str = ""

    def save(self, path: str | Path) -> None:
        Path(path).write_text(json.dumps(asdict(self), indent=2, default=str))

    @classmethod
    def load(cls, path: str | Path) -> "AgentPresetConfig":
        d = json.loads(Path(path).read_text())
        if d.get("working_dir") is not None:
            d["working_dir"] = Path(d["working_dir"])
        return cls(**d)

    def to_cli_args(self) -> dict[str, Any]:
        """The fields as the chat command's arguments (unset optional ones left out)."""
        out: dict[str, Any] = {"model": self.model, "env": self.env, "system_prompt": self.system_prompt, "thinking": self.thinking}
        for k in ("temperature", "working_dir", "tools"):
            if getattr(self, k) is not None:
                out[k] = getattr(self, k)
        return out

    def to_preset(self) -> AgentPreset:
        if self.env not in ENVIRONMENTS:
            raise KeyError(f"preset {self.name!r} names unknown environment {self.env!r}; available: {sorted(ENVIRONMENTS)}")
        factory, tools, fixed = ENVIRONMENTS[self.env], self.tools, self.working_dir
        return AgentPreset(self.name, self.description or f"{self.model} in {self.env}", self.system_prompt,
                           lambda cwd: factory(str(fixed) if fixed is not None else cwd, tools), self.max_turns)


USER_PRESET_YAML = Path.home() / ".research_b200" / "presets.yaml"


def load_yaml_presets(path: str | Path) -> dict[str, AgentPresetConfig]:
    """Presets written as YAML: either one preset (``model: ... env: ... system_prompt: ...``) or several under their names
    (``fast-coder: {model: ..., env: ..., system_prompt: ...}``). Unknown keys are an error (a typo must not be ignored)."""
    import yaml

    p = Path(path)
    data = yaml.safe_load(p.read_text()) or {}
    if not isinstance(data, dict):
        raise TypeError(f"{p} must hold a mapping")
    allowed = set(AgentPresetConfig.__dataclass_fields__)
    single = "model" in data and "env" in data
    out = {}
    for name, body in ({data.get("name", p.stem): data} if single else data).items():
        if not isinstance(body, dict):
            raise TypeError(f"{p}: preset {name!r} must be a mapping")
        unknown = set(body) - allowed
        if unknown:
            raise KeyError(f"{p}: preset {name!r} has unknown field(s) {sorted(unknown)}; allowed: {sorted(allowed)}")
        fields_ = {"name": name, **body}
        if fields_.get("working_dir") is not None:
            fields_["working_dir"] = Path(fields_["working_dir"]).expanduser()
        missing = [k for k in ("model", "env", "system_prompt") if k not in fields_]
        if missing:
            raise KeyError(f"{p}: preset {name!r} lacks {missing}")
        out[name] = AgentPresetConfig(**fields_)
    return out


def _load_preset_file(path: Path) -> AgentPresetConfig:
    if path.suffix == ".json":
        return AgentPresetConfig.load(path)
    if path.suffix in (".yaml", ".yml"):
        found = load_yaml_presets(path)
        if len(found) != 1:
            raise KeyError(f"{path} defines {len(found)} presets ({sorted(found)}): name one of them instead of the file")
        return next(iter(found.values()))
    if path.parent.resolve() == PRESET_DIR:      # shipped presets are package modules: relative imports of a parent work
        module = importlib.import_module(f"{__package__}.preset_files.{path.stem}")
    else:
        spec = importlib.util.spec_from_file_location(f"_rb_preset_{path.stem}", path)
        if spec is None or spec.loader is None:
            raise ImportError(f"cannot load a preset from {path}")
        module = importlib.util.module_from_spec(spec)
        sys.path.insert(0, str(path.parent))      # a variant may import its parent that sits beside it
        try:
            spec.loader.exec_module(module)
        finally:
            sys.path.remove(str(path.parent))
    config = getattr(module, "config", None)
    if not isinstance(config, AgentPresetConfig):
        raise TypeError(f"{path} must define `config`, an AgentPresetConfig (found {type(config).__name__})")
    return config


_NUMBERED = re.compile(r"^(?P<stem>.+)_(?P<id>\d+)_(?P<parent>\d+)$")


def list_presets(preset_dir: str | Path | None = None) -> list[str]:
    """Names of the preset files (without ``.py``) of ``preset_dir``; by default the shipped ones, then the user's."""
    dirs = [Path(preset_dir)] if preset_dir is not None else [PRESET_DIR, USER_PRESET_DIR]
    names = [f.stem for d in dirs if d.is_dir() for f in sorted(d.glob("*.py")) if not f.name.startswith("_")]
    for y in ([d / "presets.yaml" for d in dirs] if preset_dir is not None else [USER_PRESET_YAML]):
        if y.is_file():
            try:
                names += sorted(load_yaml_presets(y))
            except (KeyError, TypeError, ValueError):
                pass                                   # a broken file is reported when a preset of it is asked for
    return names


def load_preset(name: str, preset_dir: str | Path | None = None) -> AgentPresetConfig:
    """By file path (``~/presets/mine.py``, ``.json``), by full file name (``careful_coder_01_01``) or by the name
    without numbers (``careful_coder``: the highest-numbered file of that stem wins, i.e. the latest variant)."""
    p = Path(name).expanduser()
    if p.suffix in (".py", ".json", ".yaml", ".yml") or "/" in name:
        if not p.is_file():
            raise FileNotFoundError(f"preset file not found: {p}")
        return _load_preset_file(p)
    dirs = [Path(preset_dir)] if preset_dir is not None else [USER_PRESET_DIR, PRESET_DIR]
    for y in ([d / "presets.yaml" for d in dirs] if preset_dir is not None else [USER_PRESET_YAML]):
        if y.is_file():
            found = load_yaml_presets(y)
            if name in found:
                return found[name]
    for d in dirs:
        if (d / f"{name}.py").is_file():
            return _load_preset_file(d / f"{name}.py")
    best: tuple[int, Path] | None = None
    for d in dirs:
        for f in (d.glob("*.py") if d.is_dir() else ()):
            m = _NUMBERED.match(f.stem)
            if m and m.group("stem") == name and (best is None or int(m.group("id")) > best[0]):
                best = (int(m.group("id")), f)
    if best is None:
        raise KeyError(f"unknown preset {name!r}; built in: {sorted(PRESETS)}; files: {list_presets(preset_dir)}")
    return _load_preset_file(best[1])


def get_preset(name: str) -> AgentPreset:
    """A built-in preset by name, else a preset file (see ``load_preset``)."""
    if name in PRESETS:
        return PRESETS[name]
    try:
        return load_preset(name).to_preset()
    except (KeyError, FileNotFoundError) as e:
        raise KeyError(f"unknown preset {name!r}; available: {sorted(PRESETS) + list_presets()}") from e
