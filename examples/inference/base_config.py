"""Inference examples (rollouts/examples/inference/base_config.py:13-204): build an engine for a preset or a checkpoint
directory, generate several samples per prompt, and report tokens, log-probabilities and prefix-cache hits."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from examples.common import default_tokenizer
from research_b200.inference import EngineConfig, InferenceEngine, SamplingParams
from research_b200.training.backends import load_model_weights


@dataclass(frozen=True)
class BaseConfig:
    model_name: str = "tiny-qwen2"
    prompts: tuple[str, ...] = ("Hello, my name is",)
    temperature: float = 0.7
    max_tokens: int = 30
    num_samples_per_prompt: int = 1
    cache_type: str = "radix"
    max_batch_size: int = 32
    max_model_len: int = 512
    kv_blocks: int = 256
    seed: int = 0


def test_inference(config: BaseConfig, tokenizer: Any = None, device: str | None = None) -> list[dict[str, Any]]:
    tokenizer = tokenizer or default_tokenizer()
    dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
    weights, model_cfg = load_model_weights(config.model_name, config.seed)
    dtype = torch.bfloat16 if dev.startswith("cuda") else torch.float32
    engine = InferenceEngine(EngineConfig(cache_type=config.cache_type, max_batch_size=config.max_batch_size, max_model_len=config.max_model_len,
                                          num_kv_blocks=config.kv_blocks, seed=config.seed), model_cfg,
                             {k: v.to(dtype) for k, v in weights.items()}, tokenizer=tokenizer, device=dev)
    try:
        ids = [tokenizer.encode(p) for p in config.prompts]
        outs = engine.generate(ids, SamplingParams(temperature=config.temperature, max_tokens=config.max_tokens), config.num_samples_per_prompt)
        results = []
        for o in outs:
            results.append({"prompt": tokenizer.decode(list(o.prompt_tokens)), "text": tokenizer.decode(list(o.completion_tokens), skip_special_tokens=True),
                            "num_tokens": len(o.completion_tokens), "sum_logprob": float(sum(o.logprobs)), "finish_reason": o.finish_reason,
                            "cached_tokens": o.cached_tokens, "weight_version": o.weight_version})
            print(f"[{results[-1]['finish_reason']:>6}] {results[-1]['num_tokens']:3d} tokens  logp {results[-1]['sum_logprob']:8.2f}  "
                  f"cached {o.cached_tokens:3d}  {results[-1]['prompt']!r} -> {results[-1]['text'][:40]!r}")
        return results
    finally:
        engine.shutdown()
