"""SFT on the reverse-text task: teaches the tag format the RL stage rewards (python examples/sft/qwen_reverse_01_01.py)."""

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from examples.rl.reverse_text.base_config import SYSTEM_PROMPT, make_texts  # noqa: E402
from examples.sft.base_config import SFTExampleConfig, train  # noqa: E402

config = SFTExampleConfig(experiment_name="qwen_reverse_01_01", num_steps=30, batch_size=8, lr=2e-3)


def make_rows(n: int, seed: int = 0) -> list[dict]:
    return [{"messages": [{"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": t},
                          {"role": "assistant", "content": f"<reversed_text>{t[::-1]}</reversed_text>"}]} for t in make_texts(n, seed)]


if __name__ == "__main__":
    history, _ = train(config, make_rows(256))
    print(f"loss {history[0]['loss']:.3f} -> {history[-1]['loss']:.3f}")
