"""Provider registry: maps ``Endpoint.provider`` to a rollout function
(rollouts/providers/__init__.py:48-71)."""

from __future__ import annotations

from typing import Awaitable, Callable

from ..dtypes import Actor, RunConfig
from .base import (ContextTooLongError, NonRetryableError, ProviderError, RateLimiter, add_cache_control_to_last_content,
                   async_retry, backoff_delay, calculate_cost_from_usage, classify_http_status, classify_server_error,
                   explain_server_error, parse_context_overflow, prepare_messages_for_llm, retry, sanitize_request_for_logging)
from .chat import ScriptedLLM, messages_to_openai, rollout_openai_compatible
from .models import MODELS, ModelInfo, estimate_cost, get_model, get_models, get_providers, register_model
from .streaming import (aggregate_anthropic_stream, aggregate_google_stream, aggregate_openai_responses_stream,
                        aggregate_openai_stream, messages_to_anthropic, messages_to_google, messages_to_openai_responses,
                        rollout_anthropic, rollout_google, rollout_openai_responses, rollout_openai_streaming, sse_events)
from .token_level import (build_input_ids_from_trajectory, generate_sglang, generate_vllm, rollout_native_token_level,
                          rollout_sglang_token_level, rollout_vllm_token_level)
from .tool_parsers import parse_hermes_tool_calls, parse_json_tool_calls, parse_tool_calls, render_tools_system_prompt

RolloutFn = Callable[[Actor, RunConfig], Awaitable[Actor]]

_TEXT: dict[str, RolloutFn] = {"openai": rollout_openai_compatible, "sglang": rollout_openai_compatible,
                               "vllm": rollout_openai_compatible, "native": rollout_native_token_level,
                               "openai-stream": rollout_openai_streaming, "openai-responses": rollout_openai_responses,
                               "anthropic": rollout_anthropic, "google": rollout_google}
_TOKEN: dict[str, RolloutFn] = {"native": rollout_native_token_level, "sglang": rollout_sglang_token_level,
                                "vllm": rollout_vllm_token_level}


def register_provider(name: str, fn: RolloutFn, token_level: bool = False) -> None:
    (_TOKEN if token_level else _TEXT)[name] = fn


def get_provider(name: str, token_level: bool = False) -> RolloutFn:
    table = _TOKEN if token_level else _TEXT
    if name not in table and token_level and name in _TEXT:
        table = _TEXT
    if name not in table:
        raise NonRetryableError(f"unknown provider {name!r}; registered: {sorted(set(_TEXT) | set(_TOKEN))}")
    return table[name]


__all__ = ["add_cache_control_to_last_content", "calculate_cost_from_usage", "classify_server_error", "explain_server_error",
           "parse_context_overflow", "prepare_messages_for_llm", "sanitize_request_for_logging", "get_models", "get_providers",
           "register_model", "ContextTooLongError", "NonRetryableError", "ProviderError", "RateLimiter", "async_retry", "backoff_delay",
           "classify_http_status", "retry", "ScriptedLLM", "messages_to_openai", "rollout_openai_compatible", "MODELS",
           "ModelInfo", "estimate_cost", "get_model", "build_input_ids_from_trajectory", "generate_sglang",
           "generate_vllm", "rollout_native_token_level", "rollout_sglang_token_level", "rollout_vllm_token_level",
           "parse_hermes_tool_calls", "parse_json_tool_calls", "parse_tool_calls", "render_tools_system_prompt",
           "register_provider", "get_provider", "aggregate_anthropic_stream", "aggregate_google_stream",
           "aggregate_openai_responses_stream", "aggregate_openai_stream", "messages_to_anthropic", "messages_to_google",
           "messages_to_openai_responses", "rollout_anthropic", "rollout_google", "rollout_openai_responses",
           "rollout_openai_streaming", "sse_events"]
