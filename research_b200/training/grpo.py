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
    # several inference devices disjoint from the trainers': "replicas" = one engine per device on its own prompts;
    # "tensor" = ONE tensor-parallel engine over all of them (what the reference's external server does with the same
    # device tuple, rollouts/training/grpo.py:172-199), fed by the kernel weight sync into its sharded layout
    inference_parallelism: str = "replicas"
    # mixture-of-experts models on several ranks: the experts are split over the ranks for BOTH the update (every rank
    # keeps parameters, gradients and optimizer state of its own experts only) and the rollouts (data-parallel engines in
    # lock step, tokens dispatched to the experts' owners); the kernel weight sync then only moves a rank's own experts
    expert_parallel: bool = False
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


def device_roles(config: GRPOConfig, world: int) -> tuple[list[int], list[int]] | None:
    """Ranks that train and ranks that serve when ``trainer_cuda_device_ids`` and ``inference_cuda_device_ids`` name
    DISJOINT device sets that together make up the job (rollouts/training/grpo.py:55,59,172-199 places the SGLang
    engine and the trainer on different device tuples): the first ``len(trainer ids)`` ranks train, the rest serve,
    and rank ``r`` runs on device ``(trainer ids + inference ids)[r]``. None = every rank does both (same devices)."""
    t, e = tuple(config.trainer_cuda_device_ids), tuple(config.inference_cuda_device_ids)
    if set(t) & set(e) or len(t) + len(e) != world or not t or not e:
        return None
    return list(range(len(t))), list(range(len(t), len(t) + len(e)))


async def _grpo_train_async(config, prompts, score_fn, environment_cls, metrics_logger, device, tokenizer,
                            ground_truths, filter_fn) -> list[dict[str, float]]:
    distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    rank = dist.get_rank() if distributed else 0
    world = dist.get_world_size() if distributed else 1
    roles = device_roles(config, world) if distributed else None
    if roles is not None:
        return await _grpo_train_disjoint(config, roles, prompts, score_fn, environment_cls, metrics_logger, device, tokenizer,
                                          ground_truths, filter_fn)
    dev = torch.device(device) if device is not None else torch.device(
        f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cpu")
    out_dir = _setup_output_dir(config)
    if rank == 0:
        config.save(out_dir / "config.json")
    logger = metrics_logger or (JSONLLogger(out_dir) if rank == 0 else None)

    weights, model_cfg = load_model_weights(config.checkpoint_path or config.model_name, config.seed, device=dev)
    tcfg = TrainerConfig(num_minibatches=config.num_minibatches, max_grad_norm=config.max_grad_norm)
    kw = dict(device=dev, loss_fn=config.loss, lr=config.lr, weight_decay=config.weight_decay, trainer_config=tcfg,
              checkpoint_dir=out_dir / "checkpoints")
    ep_mode = bool(config.expert_parallel) and distributed and model_cfg.is_moe
    if ep_mode:
        from .backends.fsdp import FSDPConfig

        kw["config"] = FSDPConfig(expert_parallel=True)
    backend = FSDPTrainingBackend(model_cfg, weights, **kw) if distributed else PyTorchTrainingBackend(model_cfg, weights, **kw)
    ecfg = EngineConfig(cache_type=config.cache_type, max_batch_size=config.max_batch_size,
                        max_model_len=max(config.max_seq_len + config.max_tokens, 64), num_kv_blocks=config.kv_blocks,
                        seed=config.seed * 1009 + rank, ignore_eos=tokenizer is None)
    ep = None
    if ep_mode:
        from ..parallel.ep import ExpertParallel

        ep = ExpertParallel(backend.comm)
    if ep_mode and dev.type == "cuda":
        from .native_model import LazyStateDict

        engine_weights = LazyStateDict(backend.model)      # the engine copies its own experts only, tensor by tensor
    else:
        engine_weights = backend.model.state_dict()
    engine = InferenceEngine(ecfg, model_cfg, engine_weights, tokenizer=tokenizer, device=dev, ep=ep)
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


class _SizeProbe:
    """Stands in for a communicator to learn how much parameter storage a bucket layout asks for."""

    def __init__(self, world: int):
        self.world, self.shape = world, None

    def alloc(self, shape, dtype=torch.bfloat16, zero: bool = False):
        from ..parallel.symm import SymmBuffer

        self.shape = tuple(shape)
        return SymmBuffer(torch.empty(0, dtype=dtype), [0] * self.world)


class _Prealloc:
    """Hands a buffer that was allocated earlier to the one ``alloc`` call of a bucket layout."""

    def __init__(self, buf):
        self.buf = buf

    def alloc(self, shape, dtype=torch.bfloat16, zero: bool = False):
        assert tuple(shape) == tuple(self.buf.local.shape) and dtype == self.buf.local.dtype and self.buf is not None
        buf, self.buf = self.buf, None
        return buf


async def _grpo_train_disjoint(config, roles, prompts, score_fn, environment_cls, metrics_logger, device, tokenizer,
                               ground_truths, filter_fn) -> list[dict[str, float]]:
    """GRPO with the trainers and the engines on different GPUs of one node.

    Per step: the engine ranks generate and score their share of the prompt groups; the samples travel to the
    trainer ranks (one object all-gather); the trainers split the GROUPS among themselves, run the sharded
    forward/backward + optimizer step; then every engine pulls the new parameters out of a trainer's flat bucket
    over NVLink with one ``reshard_copy`` launch that writes its own packed layout (the bucket lives in symmetric
    memory allocated over ALL ranks, so the engines hold a mapping of it; host barriers fence the copy on both
    sides). On CPU groups the parameters travel with a broadcast instead."""
    from ..parallel.symm import LayoutComm, PeerComm
    from .backends.native import build_buckets
    from .rollout_gen.rollout_generation import convert_to_batch

    trainer_ranks, engine_ranks = roles
    rank, world = dist.get_rank(), dist.get_world_size()
    T, E = len(trainer_ranks), len(engine_ranks)
    is_trainer = rank in trainer_ranks
    engine_tp = config.inference_parallelism == "tensor" and E > 1
    ids = tuple(config.trainer_cuda_device_ids) + tuple(config.inference_cuda_device_ids)
    if device is not None:
        dev = torch.device(device)
    elif torch.cuda.is_available():
        dev = torch.device("cuda", ids[rank])
        torch.cuda.set_device(dev)
    else:
        dev = torch.device("cpu")
    out_dir = _setup_output_dir(config)
    if rank == 0:
        config.save(out_dir / "config.json")
    logger = metrics_logger or (JSONLLogger(out_dir) if rank == 0 else None)
    tgroup = dist.new_group(trainer_ranks)         # every rank creates both groups, in the same order
    egroup = dist.new_group(engine_ranks)
    _ = egroup
    world_comm = PeerComm(dist.group.WORLD, dev)
    weights, model_cfg = load_model_weights(config.checkpoint_path or config.model_name, config.seed)
    on_gpu = dev.type == "cuda"
    dtype = torch.bfloat16 if on_gpu else torch.float32
    # The parameter storage is allocated in the world-wide symmetric memory BEFORE any rank allocates in a sub-group:
    # with torch 2.11 a world-wide symmetric-memory rendezvous that follows a sub-group one on only some of the ranks
    # never completes (its exchanges appear to be numbered per process, not per group), so once the trainers have
    # rendezvoused among themselves (flags, gradients) they and the engines can no longer meet.
    probe = _SizeProbe(T)
    build_buckets(model_cfg, LayoutComm(T, torch.device("cpu")), dtype, False, param_comm=probe, with_grads=False)
    shared_params = _Prealloc(world_comm.alloc(probe.shape, dtype, zero=True))
    backend = engine = manager = None
    if is_trainer:
        tcfg = TrainerConfig(num_minibatches=config.num_minibatches, max_grad_norm=config.max_grad_norm)
        backend = FSDPTrainingBackend(model_cfg, weights, comm=PeerComm(tgroup, dev), device=dev, param_comm=shared_params,
                                      loss_fn=config.loss, lr=config.lr, weight_decay=config.weight_decay, trainer_config=tcfg,
                                      checkpoint_dir=out_dir / "checkpoints")
        buckets = backend.buckets
    else:
        buckets = build_buckets(model_cfg, LayoutComm(T, dev), dtype, False, param_comm=shared_params, with_grads=False)
        ei = engine_ranks.index(rank)
        tp = None
        if engine_tp:
            # one engine over all engine ranks: every one of them runs the same schedule on the same prompts with the
            # same seeds (the fused GEMM + all-reduce launches keep them in step); only the first reports samples
            from ..parallel.tp import TensorParallel

            tp = TensorParallel(PeerComm(egroup, dev), max_rows=max(config.max_batch_size * 64 + 64, 2048), max_cols=max(model_cfg.hidden_size, 1024))
            ei, n_engines = 0, 1
        else:
            n_engines = E
        ecfg = EngineConfig(cache_type=config.cache_type, max_batch_size=config.max_batch_size,
                            max_model_len=max(config.max_seq_len + config.max_tokens, 64), num_kv_blocks=config.kv_blocks,
                            seed=config.seed * 1009 + ei, ignore_eos=tokenizer is None, tensor_parallel_size=E if engine_tp else 1)
        engine = InferenceEngine(ecfg, model_cfg, weights, tokenizer=tokenizer, device=dev, tp=tp)
        mine = prompts[ei::n_engines]
        truths = ground_truths[ei::n_engines] if ground_truths else None
        gen_fn = _create_tito_generate_fn(engine, config, tokenizer)
        if environment_cls is not None and not config.use_tito:
            from .agent_integration import make_agent_generate_fn

            gen_fn = make_agent_generate_fn(engine, environment_cls, config, tokenizer)
        manager = AsyncRolloutManager(DataBuffer(mine, seed=config.seed, ground_truths=truths),
                                      RolloutConfig(batch_size=max(config.batch_size // n_engines, 1), n_samples_per_prompt=config.n_samples_per_prompt,
                                                    generate_fn=gen_fn, score_fn=score_fn, filter_fn=filter_fn))
    del weights
    dist.barrier()
    plan = None
    history: list[dict[str, float]] = []
    rollouts_file = open(out_dir / f"rollouts.rank{rank}.jsonl", "a") if not is_trainer else None
    try:
        for step in range(config.num_steps):
            t0 = time.perf_counter()
            mine_out: list[dict] = []
            if not is_trainer:
                batch = await manager.generate_batch()
                ei = engine_ranks.index(rank)
                for s in batch.samples:
                    if not engine_tp:
                        s.group_index = (s.group_index or 0) * E + ei      # group ids stay distinct across engines
                    rollouts_file.write(json.dumps({"step": step, "reward": s.reward, "tokens": len(s.tokens),
                                                    "response_length": s.response_length, "group": s.group_index,
                                                    "weight_version": s.weight_version}) + "\n")
                    if not engine_tp or ei == 0:                           # the ranks of one engine all hold the same samples
                        mine_out.append(s.to_dict())
            t_roll = time.perf_counter() - t0
            gathered: list = [None] * world
            dist.all_gather_object(gathered, mine_out)
            samples = [Sample.from_dict(d) for part in gathered for d in (part or [])]
            m: dict[str, float] = {"rollout_s": t_roll, "num_samples": float(len(samples)),
                                   "mean_reward": sum(s.reward for s in samples) / max(len(samples), 1)}
            t1 = time.perf_counter()
            if is_trainer:
                ti = trainer_ranks.index(rank)
                groups = sorted({s.group_index for s in samples})
                my_groups = set(groups[ti::T])                                # whole groups per trainer
                part = [s for s in samples if s.group_index in my_groups]
                tb_batch = convert_to_batch(part)
                adv = compute_group_advantages(tb_batch.rewards, tb_batch.group_indices, config.normalize_advantage_std)
                tb = _prepare_training_batch(tb_batch, adv, config.max_seq_len)
                n = tb["input_ids"].shape[0]
                if n % config.num_minibatches != 0:
                    keep = max(config.num_minibatches, n - n % config.num_minibatches)
                    tb = {k: (v[:keep] if isinstance(v, torch.Tensor) and v.shape[0] == n else v) for k, v in tb.items()}
                fb = await backend.forward_backward(tb).result()
                opt = await backend.optim_step().result()
                m.update(fb)
                m.update(opt)
                backend.buckets.finish_pending()
                if on_gpu:
                    torch.cuda.synchronize(dev)
            m["train_s"] = time.perf_counter() - t1
            t2 = time.perf_counter()
            if (step + 1) % config.sync_weights_every == 0:
                dist.barrier()                                                  # the trainers' parameters are final
                t2 = time.perf_counter()                                        # (an engine waited for the trainers here)
                if on_gpu:
                    if not is_trainer:
                        src = trainer_ranks[engine_ranks.index(rank) % T]
                        plan = sync_engine_from_buckets(engine, buckets, plan, src_rank=src)       # each rank pulls its shard of the layout
                        torch.cuda.synchronize(dev)
                else:
                    flat = buckets.params
                    dist.broadcast(flat, src=trainer_ranks[0])
                    if not is_trainer:
                        sync_engine_from_buckets(engine, buckets)
                dist.barrier()                                                  # the engines have read them
                if not is_trainer:
                    engine.weight_version = step + 1
            m["sync_s"] = time.perf_counter() - t2
            m["step_s"] = time.perf_counter() - t0
            m["weight_version"] = float(step + 1)
            history.append(m)
            if logger is not None and step % config.log_every == 0:
                logger.log({k: v for k, v in m.items() if isinstance(v, (int, float))}, step)
            if is_trainer and config.checkpoint_every and (step + 1) % config.checkpoint_every == 0:
                backend.save_checkpoint(step + 1, {k: v for k, v in m.items() if isinstance(v, float)})
    finally:
        if rollouts_file is not None:
            rollouts_file.close()
        if logger is not None:
            logger.finish()
        if engine is not None:
            engine.shutdown()
    return history
