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
    cache_read_per_mtok: float = 0.0
    cache_write_per_mtok: float = 0.0
    max_output_tokens: int = 8192
    supports_thinking: bool = False
    supports_images: bool = False


MODELS: dict[str, ModelInfo] = {m.name: m for m in [
    ModelInfo("Qwen/Qwen2.5-0.5B-Instruct", "native", 32768),
    ModelInfo("Qwen/Qwen3-0.6B", "native", 40960),
    ModelInfo("Qwen/Qwen3-30B-A3B", "native", 40960),
    ModelInfo("meta-llama/Meta-Llama-3-8B-Instruct", "native", 8192),
    ModelInfo("gpt-4o-mini", "openai", 128000, 0.15, 0.60, cache_read_per_mtok=0.075, max_output_tokens=16384, supports_images=True),
    ModelInfo("gpt-4o", "openai", 128000, 2.50, 10.0, cache_read_per_mtok=1.25, max_output_tokens=16384, supports_images=True),
    ModelInfo("o3-mini", "openai", 200000, 1.10, 4.40, cache_read_per_mtok=0.55, max_output_tokens=100000, supports_thinking=True),
    ModelInfo("claude-3-5-haiku-latest", "anthropic", 200000, 0.80, 4.0, cache_read_per_mtok=0.08, cache_write_per_mtok=1.0, supports_images=True),
    ModelInfo("claude-sonnet-4-5", "anthropic", 200000, 3.0, 15.0, cache_read_per_mtok=0.30, cache_write_per_mtok=3.75,
              max_output_tokens=64000, supports_thinking=True, supports_images=True),
    ModelInfo("gemini-2.0-flash", "google", 1000000, 0.10, 0.40, cache_read_per_mtok=0.025, supports_images=True),
    ModelInfo("gemini-2.5-pro", "google", 1000000, 1.25, 10.0, cache_read_per_mtok=0.31, max_output_tokens=65536, supports_thinking=True,
              supports_images=True),
]}


def get_model(name: str, provider: str | None = None) -> ModelInfo | None:
    """Exact name, else the longest registered name that the given name starts with (dated snapshots such as
    ``gpt-4o-2024-08-06``), optionally restricted to one provider."""
    info = MODELS.get(name)
    if info is None:
        hits = [m for m in MODELS.values() if name.startswith(m.name.removesuffix("-latest"))]
        info = max(hits, key=lambda m: len(m.name)) if hits else None
    if info is not None and provider and info.provider != provider:
        return None
    return info


def get_models(provider: str | None = None) -> list[ModelInfo]:
    return [m for m in MODELS.values() if provider is None or m.provider == provider]


def get_providers() -> list[str]:
    return sorted({m.provider for m in MODELS.values()})


def register_model(info: ModelInfo) -> None:
    MODELS[info.name] = info


def estimate_cost(model: str, usage: Usage) -> Cost:
    from .base import calculate_cost_from_usage

    return calculate_cost_from_usage(usage, get_model(model))
