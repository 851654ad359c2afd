"""Ready-made frozen config pieces that satisfy ``config.protocols`` (rollouts/config/base.py:25-374).

Use them as they are, override fields inline, or compose them into a project config::

    @dataclass(frozen=True)
    class MyConfig:
        model: BaseModelConfig = field(default_factory=lambda: BaseModelConfig(model_name="claude-sonnet-4"))
        evaluation: BaseEvaluationConfig = ...
"""

from __future__ import annotations

import json
import logging
import os
from dataclasses import asdict, dataclass, fields, is_dataclass
from pathlib import Path
from typing import Any, Callable

from ..agents.dtypes import Endpoint, EvalConfig, Message, RunConfig

logger = logging.getLogger(__name__)

# provider -> (default API base, environment variable that holds the key)
PROVIDER_DEFAULTS: dict[str, tuple[str, str]] = {
    "openai": ("https://api.openai.com/v1", "OPENAI_API_KEY"),
    "anthropic": ("https://api.anthropic.com", "ANTHROPIC_API_KEY"),
    "google": ("https://generativelanguage.googleapis.com/v1beta", "GOOGLE_API_KEY"),
    "native": ("", ""), "sglang": ("http://127.0.0.1:30000", ""), "vllm": ("http://127.0.0.1:8000/v1", ""), "mock": ("", ""),
}


def infer_provider_from_model(model_name: str) -> str:
    """Provider implied by a model name: ``claude-*`` -> anthropic, ``gpt-* / o1-* / o3-* / o4-*`` -> openai,
    ``gemini-*`` -> google; otherwise the text before the first dash (``openai`` when there is none)."""
    m = model_name.lower()
    if "claude" in m or "anthropic" in m:
        return "anthropic"
    if any(p in m for p in ("gpt-", "o1-", "o3-", "o4-")):
        return "openai"
    if "gemini" in m:
        return "google"
    return model_name.split("-")[0] if "-" in model_name else "openai"


@dataclass(frozen=True)
class BaseModelConfig:
    model_name: str = "gpt-4o-mini"
    provider: str = "openai"
    api_base: str = "https://api.openai.com/v1"
    api_key_env_var: str = "OPENAI_API_KEY"
    temperature: float = 0.7
    max_tokens: int = 4096
    max_retries: int = 3
    timeout: float = 120.0

    def resolved(self) -> tuple[str, str, str]:
        """(provider, api_base, api_key_env_var) after checking the provider against the model name: a config that
        names a Claude model under provider ``openai`` is corrected, together with the base URL and key variable
        (local providers - native / sglang / vllm / mock - are never overridden)."""
        provider, base, env = self.provider, self.api_base, self.api_key_env_var
        implied = infer_provider_from_model(self.model_name)
        if provider in ("openai", "anthropic", "google") and implied in ("openai", "anthropic", "google") and implied != provider:
            logger.warning("provider %r does not match model %r; using %r", provider, self.model_name, implied)
            provider = implied
            base, env = PROVIDER_DEFAULTS[implied]
        return provider, base, env

    def to_endpoint(self) -> Endpoint:
        """An empty key (variable unset) is passed on as such: the caller decides whether that is an error."""
        provider, base, env = self.resolved()
        return Endpoint(provider=provider, model=self.model_name, api_base=base, api_key=os.getenv(env, "") if env else "",
                        temperature=self.temperature, max_tokens=self.max_tokens, max_retries=self.max_retries,
                        timeout=self.timeout)


@dataclass(frozen=True)
class BaseEnvironmentConfig:
    env_name: str
    max_steps: int = 100
    timeout_seconds: float = 300.0

    def prepare_messages(self, sample_data: dict[str, Any]) -> list[Message]:
        """Default: the row's ``prompt`` field (or the row itself, printed) as one user message."""
        return [Message("user", sample_data.get("prompt", str(sample_data)))]


@dataclass(frozen=True)
class BaseEvaluationConfig:
    environment: BaseEnvironmentConfig
    eval_name: str = "evaluation"
    num_samples: int = 100
    max_concurrent: int = 4
    max_turns: int = 10
    output_dir: Path = Path("results")
    verbose: bool = True
    show_progress: bool = True
    stream_tokens: bool = False
    run_config: RunConfig | None = None

    def to_eval_config(self, endpoint: Endpoint, prepare_messages: Callable[[dict[str, Any]], list[Message]] | None,
                       score_fn: Callable[..., Any], environment_factory: Callable[..., Any] | None = None) -> EvalConfig:
        rc = self.run_config or RunConfig(show_progress=self.show_progress)
        return EvalConfig(endpoint=endpoint, score_fn=score_fn, environment_factory=environment_factory,
                          prepare_messages=prepare_messages or self.environment.prepare_messages,
                          max_turns=min(self.max_turns, self.environment.max_steps), max_samples=self.num_samples,
                          max_concurrent=self.max_concurrent, output_dir=str(self.output_dir), eval_name=self.eval_name,
                          run_config=rc)


def _plain(obj: Any) -> Any:
    if is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: _plain(getattr(obj, f.name)) for f in fields(obj)}
    if isinstance(obj, (list, tuple)):
        return [_plain(v) for v in obj]
    if isinstance(obj, dict):
        return {str(k): _plain(v) for k, v in obj.items()}
    if isinstance(obj, Path):
        return str(obj)
    if callable(obj):
        return getattr(obj, "__qualname__", repr(obj))
    return obj


@dataclass(frozen=True)
class BaseOutputConfig:
    output_dir: Path = Path("results")
    experiment_name: str = "experiment"
    verbose: bool = True
    log_level: str = "INFO"

    def save_config(self, config: Any, path: Path | str) -> None:
        """Write ``config`` (any dataclass, nested ones included; callables by name) as JSON."""
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(_plain(config) if is_dataclass(config) else asdict(config), indent=2, default=str))

    @staticmethod
    def load_config(config_class: type, path: Path | str) -> Any:
        """Rebuild a flat dataclass from JSON written by ``save_config`` (``Path`` fields are restored)."""
        data = json.loads(Path(path).read_text())
        kw = {}
        for f in fields(config_class):
            if f.name in data:
                v = data[f.name]
                kw[f.name] = Path(v) if (f.type in (Path, "Path") and isinstance(v, str)) else v
        return config_class(**kw)
