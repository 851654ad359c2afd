"""One device: SFT on the reverse-text format, then GRPO from that checkpoint."""

from dataclasses import replace

from examples.integration_training.base_config import Config, OutputSection

config = replace(Config(), output=OutputSection(mode="sft_then_rl", experiment_name="01_debug_sft_rl"))
