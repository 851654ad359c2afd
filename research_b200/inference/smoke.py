"""Tiny engine run used by the smoke entry point: prefill + CUDA-graph decode on one GPU."""

from __future__ import annotations

import torch

from ..models import get_preset, init_random_weights
from .engine import InferenceEngine
from .types import EngineConfig, SamplingParams


def engine_smoke(device: torch.device) -> None:
    cfg = get_preset("tiny-qwen2", num_layers=2)
    w = init_random_weights(cfg, seed=0, dtype=torch.bfloat16, device=device)
    eng = InferenceEngine(EngineConfig(max_batch_size=4, max_model_len=256, num_kv_blocks=64, ignore_eos=True,
                                       graph_batch_sizes=(2, 4)), cfg, w, device=device)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (20, 37, 5)]
    outs = eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=6, seed=1))
    assert all(len(o.completion_tokens) == 6 for o in outs)
    assert eng.check_invariants() == 0
    eng.shutdown()
