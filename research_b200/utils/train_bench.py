"""Training throughput of the native backend: tokens/s and model FLOP utilisation for one model shape.

    python -m research_b200.utils.train_bench --model llama-3-8b --seq 4096 --batch 1 --steps 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m research_b200.utils.train_bench --model llama-3-8b --seq 4096 --batch 1

A step is ``forward_backward`` (host batch -> pinned -> device, forward, backward) plus ``optim_step``
(reduce-scatter, clip, AdamW, parameter all-gather). Timed with CUDA events between barriers, maximum
over ranks; weak scaling (``--batch`` is per rank). Random-init weights, uniform random tokens.
"""

from __future__ import annotations

import argparse
import json
import os

import torch


def model_flops_per_token(cfg, seq: int) -> float:
    """6 * matmul parameters + causal attention (12 * L * d_head * Hq * seq / 2 per token)."""
    d, L, F = cfg.hidden_size, cfg.num_layers, cfg.intermediate_size
    qkv = d * (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim
    attn = qkv + cfg.num_heads * cfg.head_dim * d
    dense_layers = L
    matmul_params = 0.0
    if getattr(cfg, "is_moe", False):
        # a token multiplies with the router, its top-k experts and the shared experts (the ACTIVE parameters)
        dense_layers = min(cfg.first_k_dense_replace, L)
        Fm = cfg.moe_intermediate_size
        matmul_params += (L - dense_layers) * (attn + d * cfg.num_experts + 3 * d * Fm * (cfg.num_experts_per_tok + cfg.n_shared_experts))
    matmul_params += dense_layers * (attn + 3 * d * F) + cfg.vocab_size * d
    return 6.0 * matmul_params + 12.0 * L * cfg.num_heads * cfg.head_dim * seq / 2


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-0.5b")
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=2, help="sequences per rank per step")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--loss", default="sft")
    ap.add_argument("--no-checkpointing", action="store_true")
    ap.add_argument("--micro-batch", type=int, default=1, help="sequences per forward/backward pass")
    ap.add_argument("--kernel-table", default="", help="write a table of device time per kernel (one extra step under the "
                                                       "PyTorch profiler, after the timed steps) to this file")
    ap.add_argument("--peak-tflops", type=float, default=1426.3, help="sustained cuBLAS bf16 TFLOP/s per GPU for the MFU line")
    ap.add_argument("--expert-parallel", action="store_true", help="several ranks, MoE models: every rank keeps (and updates) its own "
                                                                   "experts only; tokens travel to the experts' owners and back")
    ap.add_argument("--layers", type=int, default=0, help="keep only the first N layers of the preset (a model that does not "
                                                          "fit otherwise; the output says so)")
    args = ap.parse_args()

    import torch.distributed as dist

    from ..models import get_preset
    from ..training.backends.fsdp import FSDPTrainingBackend
    from ..training.backends.native import NativeTrainingBackend
    from ..training.types import TrainerConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = get_preset(args.model, num_layers=args.layers) if args.layers else get_preset(args.model)
    kw = dict(loss_fn=args.loss, lr=1e-5, trainer_config=TrainerConfig(micro_batch_size=args.micro_batch), activation_checkpointing=not args.no_checkpointing,
              need_entropy=False)
    if world > 1:
        from ..training.backends.fsdp import FSDPConfig

        backend = FSDPTrainingBackend(cfg, None, config=FSDPConfig(expert_parallel=args.expert_parallel,
                                                                   gradient_checkpointing=not args.no_checkpointing), **kw)
    else:
        backend = NativeTrainingBackend(cfg, None, device=dev, **kw)
    g = torch.Generator().manual_seed(1234 + local)

    def batch():
        ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq), generator=g)
        return {"input_ids": ids, "labels": ids.clone(), "loss_mask": torch.ones(args.batch, args.seq)}

    def step():
        m = backend.forward_backward(batch()).wait()
        backend.optim_step().wait()
        return m

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        m = step()
    t1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([t0.elapsed_time(t1) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    tokens = args.batch * args.seq * world
    tok_s = tokens / (ms.item() * 1e-3)
    mfu = tok_s / world * model_flops_per_token(cfg, args.seq) / (args.peak_tflops * 1e12)
    if local == 0 and int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"metric": "train_tokens_per_s", "model": args.model + (f" (first {args.layers} of its layers)" if args.layers else ""),
                          "n_gpus": world, "seq_len": args.seq,
                          "batch_per_gpu": args.batch, "ms_per_step": round(ms.item(), 2), "value": round(tok_s, 1),
                          "mfu_of_sustained_cublas": round(mfu, 3), "loss": round(float(m.get("loss", 0.0)), 4),
                          "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1),
                          "activation_checkpointing": not args.no_checkpointing, "expert_parallel": bool(args.expert_parallel and world > 1),
                          "dtype": "bf16", "data": "synthetic"}))
    if args.kernel_table and local == 0:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
        total = sum(e.device_time_total for e in rows) or 1.0
        with open(args.kernel_table, "w") as f:
            f.write(f"# device time per kernel, one training step ({args.model}, batch {args.batch} x seq {args.seq}, "
                    f"micro-batch {args.micro_batch}); total {total / 1e3:.1f} ms under the profiler\n")
            for e in rows[:40]:
                f.write(f"{e.device_time_total / total * 100:5.1f}%  n={e.count:5d}  avg={e.device_time_total / max(e.count, 1):9.1f}us  {e.key[:110]}\n")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
