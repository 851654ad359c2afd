"""Four ranks, sharded optimizer (train.py relaunches itself under torch.distributed.run)."""

from dataclasses import replace

from examples.integration_training.base_config import Config, OutputSection, SFTSection, TargetConfig

config = replace(Config(), target=TargetConfig(gpu_ranks=(0, 1, 2, 3), train_backend="fsdp"), sft=SFTSection(num_steps=100, batch_size=16),
                 output=OutputSection(mode="sft", experiment_name="02_debug_sft_fsdp"))
