"""What the RL examples share: a small default ``GRPOConfig`` that runs anywhere, and the command line every example
script gets (``--steps``, ``--model``, ``--device``, ``--remote ssh-string``)."""

from __future__ import annotations

import argparse
from dataclasses import replace
from typing import Any, Callable

from examples.common import run_remote
from research_b200.training.grpo import GRPOConfig


def small_config(experiment_name: str, **kw: Any) -> GRPOConfig:
    base = GRPOConfig(experiment_name=experiment_name, model_name="tiny-qwen2", lr=1e-4, batch_size=4, n_samples_per_prompt=4,
                      num_minibatches=2, max_seq_len=256, max_tokens=24, temperature=1.0, num_steps=3, checkpoint_every=0,
                      max_batch_size=32, kv_blocks=256, output_dir="results/rl", loss="grpo_clipped")
    return replace(base, **kw)


def main(train: Callable[..., Any], script: str, default: GRPOConfig) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=default.num_steps)
    ap.add_argument("--model", default=default.model_name, help="preset name or checkpoint directory")
    ap.add_argument("--device", default=None)
    ap.add_argument("--remote", default="", help="user@host[:port]: run there instead of here")
    a = ap.parse_args()
    if a.remote:
        raise SystemExit(run_remote(script, ssh=a.remote))
    hist = train(replace(default, num_steps=a.steps, model_name=a.model), device=a.device)
    for i, m in enumerate(hist):
        print(f"step {i + 1}: reward {m.get('mean_reward', float('nan')):.3f}  loss {m.get('pg_loss', m.get('loss', float('nan'))):.4f}")
