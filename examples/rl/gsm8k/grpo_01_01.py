"""GSM8K-style GRPO, experiment 01 (python examples/rl/gsm8k/grpo_01_01.py)."""

import sys
from dataclasses import replace
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from examples.rl.base_config import main  # noqa: E402
from examples.rl.gsm8k.base_config import DEFAULT, train  # noqa: E402

config = replace(DEFAULT, experiment_name="gsm8k_grpo_01_01")

if __name__ == "__main__":
    main(train, __file__, config)
