"""End-to-end GRPO step benchmark: rollouts on the in-process engine, policy-gradient step on the kernel
backend, trainer -> engine weight sync, all on the GPUs of one process group (one rank per GPU under
``torch.distributed.run``; a single process otherwise). This is the loop of the reference's headline
example (rollouts/examples/rl/gsm8k/base_config.py:132, rollouts/training/grpo.py:113) with synthetic
prompts and a synthetic reward, since neither datasets nor checkpoints can be fetched.

    python -m research_b200.utils.grpo_bench --model qwen2.5-0.5b --prompts 32 --samples 8 --max-tokens 256

Prints one JSON line: seconds per phase (rollout / train / sync, device time), generated and trained
tokens per second and samples per second over the measured steps (the first step is warm-up).
"""

from __future__ import annotations

import argparse
import json
import os
import tempfile

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-0.5b")
    ap.add_argument("--prompts", type=int, default=32, help="prompts per step (per job)")
    ap.add_argument("--samples", type=int, default=8, help="samples per prompt")
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--minibatches", type=int, default=8)
    ap.add_argument("--loss", default="grpo_clipped")
    ap.add_argument("--device", default=None)
    ap.add_argument("--expert-parallel", action="store_true", help="MoE models on several ranks: experts split over the ranks for rollouts and update")
    ap.add_argument("--engine-tp", action="store_true", help="with --trainers: the serving ranks form ONE tensor-parallel engine")
    ap.add_argument("--trainers", type=int, default=0,
                    help="several ranks: the first N ranks only train, the others only serve (disjoint device sets); 0 = every rank does both")
    args = ap.parse_args()

    import torch.distributed as dist

    from ..models import get_preset
    from ..training.grpo import GRPOConfig, grpo_train

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
    rank = dist.get_rank() if world > 1 else 0
    cfg = get_preset(args.model)
    g = torch.Generator().manual_seed(0)
    n_prompts = args.prompts * (args.steps + 2)
    prompts = [torch.randint(3, cfg.vocab_size, (int(n),), generator=g).tolist()
               for n in torch.randint(args.prompt_len // 2, args.prompt_len + 1, (n_prompts,), generator=g)]
    out = tempfile.mkdtemp(prefix="grpo_bench_")
    gcfg = GRPOConfig(model_name=args.model, lr=1e-6, batch_size=args.prompts, n_samples_per_prompt=args.samples,
                      num_minibatches=args.minibatches, max_tokens=args.max_tokens, max_seq_len=args.prompt_len + args.max_tokens,
                      temperature=1.0, num_steps=args.steps + 1, output_dir=out, checkpoint_every=0, loss=args.loss,
                      max_batch_size=min(256, args.prompts * args.samples // max(world - args.trainers, 1)))
    if args.expert_parallel:
        import dataclasses

        gcfg = dataclasses.replace(gcfg, expert_parallel=True)
    disjoint = world > 1 and 0 < args.trainers < world
    if disjoint:
        import dataclasses

        gcfg = dataclasses.replace(gcfg, trainer_cuda_device_ids=tuple(range(args.trainers)),
                                   inference_cuda_device_ids=tuple(range(args.trainers, world)),
                                   inference_parallelism="tensor" if args.engine_tp else "replicas",
                                   max_batch_size=min(256, args.prompts * args.samples) if args.engine_tp else gcfg.max_batch_size)
    hist = grpo_train(gcfg, prompts, lambda s: float(sum(s.tokens[-s.response_length:]) % 2), device=args.device)
    steps = hist[1:]                      # the first step pays one-time set-up (graph capture, allocator growth)
    n = len(steps)
    phase = {k: sum(h.get(k, 0.0) for h in steps) / n for k in ("step_s", "rollout_s", "train_s", "sync_s", "num_samples", "sync_dev_ms")}
    if disjoint:
        # every rank reports its own phases (an engine does not train, a trainer does not generate): the slowest rank counts
        t = torch.tensor([phase[k] for k in sorted(phase)], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        phase = dict(zip(sorted(phase), t.tolist()))
    mean = phase.__getitem__
    samples = mean("num_samples") * (1 if disjoint else world)      # disjoint ranks all see the gathered samples
    gen_tokens = samples * args.max_tokens
    trained_tokens = samples * (args.prompt_len * 0.75 + args.max_tokens)     # prompts are U[len/2, len]
    row = {"bench": "grpo_step", "model": args.model, "world": world,
           "placement": (f"{args.trainers} trainer ranks + " + (f"one tensor-parallel engine over {world - args.trainers} ranks" if args.engine_tp
                                                                 else f"{world - args.trainers} engine ranks")) if disjoint else ("every rank trains and serves" + (", experts split over the ranks" if args.expert_parallel else "")),
           "samples_per_step": samples,
           "max_tokens": args.max_tokens, "prompt_len": f"U[{args.prompt_len // 2},{args.prompt_len}]", "loss": args.loss,
           "step_s": round(mean("step_s"), 4),
           "rollout_s": round(mean("rollout_s"), 4), "train_s": round(mean("train_s"), 4), "sync_s": round(mean("sync_s"), 5),
           "sync_device_ms": round(mean("sync_dev_ms"), 3),     # same-GPU placement: the copy kernel's device time (sync_s is its launch)
           "rollout_tokens_per_s": round(gen_tokens / max(mean("rollout_s"), 1e-9), 1),
           "train_tokens_per_s": round(trained_tokens / max(mean("train_s"), 1e-9), 1),
           "samples_per_s": round(samples / max(mean("step_s"), 1e-9), 2),
           "phase_keys": sorted(k for k in steps[0] if k.endswith("_s"))}
    if rank == 0:
        print(json.dumps(row), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
