"""Small model registry with context sizes and prices per million tokens
(rollouts/models.py:35-462, trimmed to families this framework serves or commonly proxies)."""

from __future__ import annotations

from dataclasses import dataclass

from ..dtypes import Cost, Usage


@dataclass(frozen=True)
class ModelInfo:
    name: str
    provider: str
    context_window: int
    input_per_mtok: float = 0.0
    output_per_mtok: float = 0.0
    supports_tools: bool = True


MODELS: dict[str, ModelInfo] = {m.name: m for m in [
    ModelInfo("Qwen/Qwen2.5-0.5B-Instruct", "native", 32768),
    ModelInfo("Qwen/Qwen3-0.6B", "native", 40960),
    ModelInfo("Qwen/Qwen3-30B-A3B", "native", 40960),
    ModelInfo("meta-llama/Meta-Llama-3-8B-Instruct", "native", 8192),
    ModelInfo("gpt-4o-mini", "openai", 128000, 0.15, 0.60),
    ModelInfo("gpt-4o", "openai", 128000, 2.50, 10.0),
    ModelInfo("claude-3-5-haiku-latest", "anthropic", 200000, 0.80, 4.0),
    ModelInfo("gemini-2.0-flash", "google", 1000000, 0.10, 0.40),
]}


def get_model(name: str) -> ModelInfo | None:
    return MODELS.get(name)


def estimate_cost(model: str, usage: Usage) -> Cost:
    info = MODELS.get(model)
    if info is None:
        return Cost()
    return Cost(input=usage.input_tokens * info.input_per_mtok / 1e6, output=usage.output_tokens * info.output_per_mtok / 1e6)
