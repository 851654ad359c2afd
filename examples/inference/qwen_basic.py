"""Basic generation check: model loading, log-probabilities, several samples per prompt
(python examples/inference/qwen_basic.py [--model DIR] [--remote user@host])."""

import argparse
import sys
from dataclasses import replace
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from examples.common import run_remote  # noqa: E402
from examples.inference.base_config import BaseConfig, test_inference  # noqa: E402

config = replace(BaseConfig(), prompts=("Hello, my name is", "The capital of France is", "To solve this math problem, I will"),
                 temperature=0.7, max_tokens=30, num_samples_per_prompt=2)

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=config.model_name)
    ap.add_argument("--remote", default="")
    a = ap.parse_args()
    if a.remote:
        raise SystemExit(run_remote(__file__, ssh=a.remote))
    results = test_inference(replace(config, model_name=a.model))
    assert len(results) == 6 and all(r["num_tokens"] > 0 for r in results), "a sample came back empty"
    print("PASSED: every sample has tokens and log-probabilities")
