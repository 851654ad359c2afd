"""Alphabet-sort GRPO, experiment 01 (python examples/rl/alphabet_sort/grpo_01_01.py)."""

import sys
from dataclasses import replace
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from examples.rl.alphabet_sort.base_config import DEFAULT, train  # noqa: E402
from examples.rl.base_config import main  # noqa: E402

config = replace(DEFAULT, experiment_name="alphabet_sort_grpo_01_01")

if __name__ == "__main__":
    main(train, __file__, config)
