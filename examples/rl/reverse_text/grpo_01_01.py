"""Reverse-text GRPO, experiment 01: the defaults of ``base_config`` (python examples/rl/reverse_text/grpo_01_01.py)."""

import sys
from dataclasses import replace
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from examples.rl.base_config import main  # noqa: E402
from examples.rl.reverse_text.base_config import DEFAULT, train  # noqa: E402

config = replace(DEFAULT, experiment_name="reverse_text_grpo_01_01", n_samples_per_prompt=8, lr=5e-5)

if __name__ == "__main__":
    main(train, __file__, config)
