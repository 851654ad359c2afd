"""research_b200: a Blackwell (sm_100a) native RL / LLM framework.

Layers (bottom to top):
  csrc/       hand-written CUDA kernels (tcgen05/TMEM/TMA) and the C++ engine core
  ops/        Python entry points of the kernels, each with a PyTorch reference twin
  models/     functional model math (oracles) and the kernel-backed model runner
  inference/  continuous-batching engine: scheduler, paged KV, radix cache, CUDA graphs
  parallel/   symmetric peer memory, fused TP / FSDP / EP collectives, weight sync
  training/   backends, losses, GRPO / SFT loops, rollout generation, data buffer
  miniray/    process launch, GPU affinity, NCCL env
  agents/     agent runtime, environments, providers, evaluation, session store
  utils/      logging, config loading, timing, fingerprints
"""

__version__ = "0.1.0"
