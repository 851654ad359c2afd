"""Config tree of the post-training driver (dev/integration_training/base_config.py): which devices and backend
(``target``), which model, the SFT and RL stages, where results go and which stage ``train.py`` runs (``output.mode``)."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class TargetConfig:
    gpu_ranks: tuple[int, ...] = (0,)
    train_backend: str = "pytorch"           # pytorch (one device) | fsdp (one rank per entry of gpu_ranks)
    device: str = "auto"                     # auto | cuda | cpu (cpu ranks talk over gloo)
    master_addr: str = "127.0.0.1"
    master_port: int = 29511


@dataclass(frozen=True)
class ModelSection:
    name: str = "tiny-qwen2"                 # preset or HF-format checkpoint directory
    max_length: int = 256


@dataclass(frozen=True)
class SFTSection:
    num_steps: int = 20
    batch_size: int = 8                      # global; split over the ranks
    lr: float = 1e-3
    warmup_steps: int = 2
    num_rows: int = 128
    checkpoint_every: int = 0


@dataclass(frozen=True)
class RLSection:
    num_steps: int = 3
    batch_size: int = 4
    n_samples_per_prompt: int = 4
    lr: float = 2e-5
    max_tokens: int = 24
    temperature: float = 0.7
    num_prompts: int = 64


@dataclass(frozen=True)
class OutputSection:
    mode: str = "sft"                        # sft | rl | sft_then_rl
    save_dir: str = "results/integration_training"
    experiment_name: str = "debug"


@dataclass(frozen=True)
class Config:
    target: TargetConfig = field(default_factory=TargetConfig)
    model: ModelSection = field(default_factory=ModelSection)
    sft: SFTSection = field(default_factory=SFTSection)
    rl: RLSection = field(default_factory=RLSection)
    output: OutputSection = field(default_factory=OutputSection)
    seed: int = 0
