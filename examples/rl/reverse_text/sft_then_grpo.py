"""Two stages in one script (rollouts/examples/rl/reverse_text/sft_then_grpo.py:1-328): SFT the tag format, save an
HF-format checkpoint, then GRPO from that checkpoint with the LCS reward."""

import sys
from dataclasses import replace
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from examples.rl.reverse_text.base_config import DEFAULT, train as grpo  # noqa: E402
from examples.sft.base_config import SFTExampleConfig, train as sft  # noqa: E402
from examples.sft.qwen_reverse_01_01 import make_rows  # noqa: E402


def run(sft_steps: int = 40, rl_steps: int = 5, device: str | None = None, out: str = "results/reverse_text_two_stage", model: str = "tiny-qwen2"):
    hist, backend = sft(SFTExampleConfig(experiment_name="stage1_sft", model_name=model, num_steps=sft_steps, output_dir=out), make_rows(256), device=device)
    ckpt = backend.save_hf_checkpoint(Path(out) / "stage1_sft" / "hf")
    rl = grpo(replace(DEFAULT, experiment_name="stage2_grpo", model_name=str(ckpt), num_steps=rl_steps, output_dir=out, lr=2e-5), num_samples=64, device=device)
    return hist, rl


if __name__ == "__main__":
    s, r = run()
    print(f"sft loss {s[0]['loss']:.3f} -> {s[-1]['loss']:.3f}; rl reward {r[0]['mean_reward']:.3f} -> {r[-1]['mean_reward']:.3f}")
