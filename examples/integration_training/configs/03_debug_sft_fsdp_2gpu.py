"""Two ranks, sharded optimizer: the smallest multi-GPU run (also works as two CPU ranks with ``device="cpu"``)."""

from dataclasses import replace

from examples.integration_training.base_config import Config, OutputSection, SFTSection, TargetConfig

config = replace(Config(), target=TargetConfig(gpu_ranks=(0, 1), train_backend="fsdp"), sft=SFTSection(num_steps=100, batch_size=8),
                 output=OutputSection(mode="sft", experiment_name="03_debug_sft_fsdp_2gpu"))
