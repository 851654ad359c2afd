"""GRPO training driver: rollouts on the native engine -> group advantages -> training step ->
in-place weight sync, repeated (``GRPOConfig`` / ``grpo_train`` of rollouts/training/grpo.py:41-869).

What changed underneath, deliberately:
* the reference launches an external SGLang/vLLM server in tmux and talks HTTP; here the engine
  is the in-process ``InferenceEngine`` on the same GPU (or one replica per rank);
* the reference trains on one GPU only; with an initialised process group every rank runs a
  rollout replica on its share of the prompts and the step is sharded data parallel;
* weights reach the engine through one reshard-copy kernel from the trainer's flat bucket
  (``parallel.weight_sync``), not through ``torch.save`` to /dev/shm + ``/update_weights_from_disk``.
Artefacts match: ``config.json``, ``metrics.jsonl``, ``rollouts.jsonl`` under the run directory.
"""

from __future__ import annotations

import asyncio
import json
import os
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Callable

import torch
import torch.distributed as dist

from ..inference import EngineConfig, InferenceEngine, SamplingParams
from ..parallel.weight_sync import sync_engine_from_buckets
from .backends import FSDPTrainingBackend, PyTorchTrainingBackend, load_model_weights
from .datasets.data_buffer import DataBuffer
from .loops.rl_loop import prepare_grpo_batch
from .losses import compute_group_advantages
from .metrics import JSONLLogger, MetricsLogger
from .rollout_gen.async_rollout_manager import AsyncRolloutManager
from .types import RolloutConfig, Sample, Status, TrainerConfig


@dataclass(frozen=True)
class GRPOConfig:
    model_name: str = "tiny-qwen2"             # preset name or HF-format checkpoint directory
    dtype: str = "bfloat16"
    inference_backend: str = "native"          # "native" (in-process engine); "sglang"/"vllm" use weight_sync engines
    inference_port: int = 30000
    inference_cuda_device_ids: tuple[int, ...] = (0,)
    mem_fraction: float = 0.7
    trainer_cuda_device_ids: tuple[int, ...] = (0,)
    lr: float = 1e-6
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    num_minibatches: int = 8
    batch_size: int = 8
    n_samples_per_prompt: int = 8
    max_seq_len: int = 1024
    max_tokens: int = 512
    temperature: float = 0.8
    max_turns: int = 1
    use_tito: bool = True
    trajectory_strategy: str = "interleaved"
    checkpoint_path: str | None = None
    num_steps: int = 100
    log_every: int = 1
    checkpoint_every: int = 20
    sync_weights_every: int = 1
    output_dir: str = "results/rl"
    experiment_name: str = "grpo"
    loss: str = "grpo"                          # grpo | grpo_clipped | grpo_masked
    cache_type: str = "radix"
    max_batch_size: int = 256
    kv_blocks: int = 0
    seed: int = 0
    normalize_advantage_std: bool = False

    def save(self, path: Path | str) -> None:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(asdict(self), indent=2))


def _setup_output_dir(config: GRPOConfig) -> Path:
    name = os.environ.get("ROLLOUTS_RUN_NAME") or f"{config.experiment_name}_{time.strftime('%Y%m%d-%H%M%S')}"
    out = Path(config.output_dir) / name
    out.mkdir(parents=True, exist_ok=True)
    return out


def _create_tito_generate_fn(engine: InferenceEngine, config: GRPOConfig, tokenizer=None) -> Callable:
    """Token-in/token-out generation: prompts are token-id lists (or text when a tokenizer exists)."""

    def generate(prompts: list[Any], **kw) -> list[Sample]:
        toks = []
        for p in prompts:
            if isinstance(p, (list, tuple)) and p and isinstance(p[0], int):
                toks.append(list(p))
            else:
                assert tokenizer is not None, "text prompts need a tokenizer"
                text = p if isinstance(p, str) else tokenizer.apply_chat_template(p, tokenize=False, add_generation_prompt=True)
                toks.append(tokenizer.encode(text))
        outs = engine.generate(toks, SamplingParams(temperature=config.temperature, max_tokens=config.max_tokens))
        samples = []
        for p, o in zip(prompts, outs):
            n_p, n_c = len(o.prompt_tokens), len(o.completion_tokens)
            meta = {"finish_reason": o.finish_reason, "cached_tokens": o.cached_tokens}
            if tokenizer is not None:
                meta["response_text"] = tokenizer.decode(list(o.completion_tokens))
            samples.append(Sample(prompt=p if not isinstance(p, tuple) else list(p), tokens=list(o.prompt_tokens + o.completion_tokens),
                                  response_length=n_c, loss_mask=[0.0] * n_p + [1.0] * n_c,
                                  rollout_log_probs=list(o.logprobs), status=Status.COMPLETED if o.finish_reason == "stop" else Status.TRUNCATED,
                                  metadata=meta, weight_version=o.weight_version))
        return samples

    generate.batched = True     # the rollout manager may pass the prompts of all groups in one call
    return generate


def _prepare_training_batch(batch, advantages: torch.Tensor, max_seq_len: int) -> dict[str, Any]:
    return prepare_grpo_batch(batch, advantages, max_seq_len)


def grpo_train(config: GRPOConfig, prompts: list[Any], score_fn: Callable[[Sample], Any],
               environment_cls: type | None = None, metrics_logger: MetricsLogger | None = None,
               device: str | torch.device | None = None, tokenizer=None, ground_truths: list[Any] | None = None,
               filter_fn: Callable | None = None) -> list[dict[str, float]]:
    """Run ``config.num_steps`` GRPO steps; returns the per-step metrics (also written to metrics.jsonl)."""
    return asyncio.run(_grpo_train_async(config, prompts, score_fn, environment_cls, metrics_logger, device, tokenizer,
                                         ground_truths, filter_fn))


async def _grpo_train_async(config, prompts, score_fn, environment_cls, metrics_logger, device, tokenizer,
                            ground_truths, filter_fn) -> list[dict[str, float]]:
    distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    rank = dist.get_rank() if distributed else 0
    world = dist.get_world_size() if distributed else 1
    dev = torch.device(device) if device is not None else torch.device(
        f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cpu")
    out_dir = _setup_output_dir(config)
    if rank == 0:
        config.save(out_dir / "config.json")
    logger = metrics_logger or (JSONLLogger(out_dir) if rank == 0 else None)

    weights, model_cfg = load_model_weights(config.checkpoint_path or config.model_name, config.seed)
    tcfg = TrainerConfig(num_minibatches=config.num_minibatches, max_grad_norm=config.max_grad_norm)
    kw = dict(device=dev, loss_fn=config.loss, lr=config.lr, weight_decay=config.weight_decay, trainer_config=tcfg,
              checkpoint_dir=out_dir / "checkpoints")
    backend = FSDPTrainingBackend(model_cfg, weights, **kw) if distributed else PyTorchTrainingBackend(model_cfg, weights, **kw)
    ecfg = EngineConfig(cache_type=config.cache_type, max_batch_size=config.max_batch_size,
                        max_model_len=max(config.max_seq_len + config.max_tokens, 64), num_kv_blocks=config.kv_blocks,
                        seed=config.seed * 1009 + rank, ignore_eos=tokenizer is None)
    engine = InferenceEngine(ecfg, model_cfg, backend.model.state_dict(), tokenizer=tokenizer, device=dev)
    del weights

    my_prompts = prompts[rank::world] if distributed else prompts
    my_truths = ground_truths[rank::world] if (ground_truths and distributed) else ground_truths
    buffer = DataBuffer(my_prompts, seed=config.seed, ground_truths=my_truths)
    gen_fn = _create_tito_generate_fn(engine, config, tokenizer)
    if environment_cls is not None and not config.use_tito:
        from .agent_integration import make_agent_generate_fn

        gen_fn = make_agent_generate_fn(engine, environment_cls, config, tokenizer)
    rollout_cfg = RolloutConfig(batch_size=max(config.batch_size // world, 1), n_samples_per_prompt=config.n_samples_per_prompt,
                                generate_fn=gen_fn, score_fn=score_fn, filter_fn=filter_fn)
    manager = AsyncRolloutManager(buffer, rollout_cfg)
    plan = None
    history: list[dict[str, float]] = []
    from ..utils.timing import PhaseTimer

    timer = PhaseTimer(device)     # wall + device time + NVTX range per phase
    rollouts_file = open(out_dir / f"rollouts{'' if world == 1 else f'.rank{rank}'}.jsonl", "a")
    try:
        for step in range(config.num_steps):
            t0 = time.perf_counter()
            timer.reset()
            with timer.phase("rollout"):
                batch = await manager.generate_batch()
            for s in batch.samples:
                rec = {"step": step, "reward": s.reward, "tokens": len(s.tokens), "response_length": s.response_length,
                       "group": s.group_index, "weight_version": s.weight_version}
                text = (s.metadata or {}).get("response_text")
                if text is not None:                       # with a tokenizer the record is readable (trace viewer)
                    p = s.prompt
                    rec["prompt"] = (p[-1].get("content", "") if isinstance(p, list) and p and isinstance(p[-1], dict) else str(p))[:2000]
                    rec["response"] = str(text)[:4000]
                    if s.ground_truth is not None:
                        rec["ground_truth"] = str(s.ground_truth)[:500]
                rollouts_file.write(json.dumps(rec) + "\n")
            adv = compute_group_advantages(batch.rewards, batch.group_indices, config.normalize_advantage_std)
            tb = _prepare_training_batch(batch, adv, config.max_seq_len)
            n = tb["input_ids"].shape[0]
            if n % config.num_minibatches != 0:  # keep whole micro-batches
                keep = max(config.num_minibatches, n - n % config.num_minibatches)
                tb = {k: (v[:keep] if isinstance(v, torch.Tensor) and v.shape[0] == n else v) for k, v in tb.items()}
            with timer.phase("train"):
                fb = await backend.forward_backward(tb).result()
                opt = await backend.optim_step().result()
            with timer.phase("sync"):
                if (step + 1) % config.sync_weights_every == 0:
                    plan = sync_engine_from_buckets(engine, backend.buckets, plan)
                    engine.weight_version = backend.weight_version
            m = {**fb, **opt, "mean_reward": sum(batch.rewards) / max(len(batch.rewards), 1),
                 **timer.summary(), "step_s": time.perf_counter() - t0,
                 "num_samples": float(len(batch)), "weight_version": float(backend.weight_version),
                 "cache_hit_tokens": float(engine.cache_stats()["hit_tokens"])}
            history.append(m)
            if logger is not None and step % config.log_every == 0:
                logger.log(m, step)
            if config.checkpoint_every and (step + 1) % config.checkpoint_every == 0:
                backend.save_checkpoint(step + 1, {k: v for k, v in m.items() if isinstance(v, float)})
                (out_dir / "rollout_state.json").write_text(json.dumps(manager.state_dict()))
    finally:
        rollouts_file.close()
        if logger is not None:
            logger.finish()
        engine.shutdown()
    return history
