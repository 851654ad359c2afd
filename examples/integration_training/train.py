"""Post-training driver (dev/integration_training/train.py:391-450, run_fsdp.sh:30-36):

    python examples/integration_training/train.py examples/integration_training/configs/01_debug_sft_rl.py
    python examples/integration_training/train.py examples/integration_training/configs/03_debug_sft_fsdp_2gpu.py

The stage (``sft`` / ``rl`` / ``sft_then_rl``) comes from ``config.output.mode``. With ``train_backend = "fsdp"`` and
more than one rank the script relaunches itself under ``torch.distributed.run`` (one process per rank, rendezvous on
127.0.0.1) unless it already runs inside such a launch; every rank then builds the sharded-optimizer backend, takes its
slice of each global batch, and rank 0 writes metrics and checkpoints."""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import subprocess
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from examples.common import default_tokenizer  # noqa: E402
from examples.integration_training.base_config import Config  # noqa: E402
from research_b200.utils.config_loader import config_to_dict, load_config_from_file  # noqa: E402


def _device(cfg: Config, local_rank: int) -> str:
    want = cfg.target.device
    if want == "cpu" or (want == "auto" and not torch.cuda.is_available()):
        return "cpu"
    return f"cuda:{local_rank}"


def run_sft(cfg: Config, tokenizer, out: Path) -> tuple[list[dict], object]:
    import torch.distributed as dist

    from examples.sft.qwen_reverse_01_01 import make_rows
    from research_b200.training.backends import (FSDPTrainingBackend, PyTorchTrainingBackend, create_warmup_cosine_scheduler,
                                                 load_model_weights)
    from research_b200.training.datasets.sft import load_sft_dataset
    from research_b200.training.loops.sft_loop import run_sft_training
    from research_b200.training.metrics import JSONLLogger
    from research_b200.training.types import SFTTrainingConfig

    distributed = dist.is_initialized() and dist.get_world_size() > 1
    rank, world = (dist.get_rank(), dist.get_world_size()) if distributed else (0, 1)
    dev = _device(cfg, int(os.environ.get("LOCAL_RANK", "0")))
    weights, mc = load_model_weights(cfg.model.name, cfg.seed)
    kw = dict(device=dev, loss_fn="sft", lr=cfg.sft.lr, lr_schedule=create_warmup_cosine_scheduler(cfg.sft.warmup_steps, cfg.sft.num_steps),
              checkpoint_dir=out / "checkpoints")
    backend = FSDPTrainingBackend(mc, weights, **kw) if distributed else PyTorchTrainingBackend(mc, weights, **kw)
    samples = load_sft_dataset(make_rows(cfg.sft.num_rows, cfg.seed), tokenizer, max_length=cfg.model.max_length)[rank::world]
    loop = SFTTrainingConfig(num_steps=cfg.sft.num_steps, batch_size=max(cfg.sft.batch_size // world, 1), log_every=1,
                             checkpoint_every=cfg.sft.checkpoint_every)
    hist = asyncio.run(run_sft_training(backend, samples, loop, JSONLLogger(out) if rank == 0 else None, pad_token_id=tokenizer.pad_token_id))
    return hist, backend


def run_rl(cfg: Config, tokenizer, out: Path, model_name: str) -> list[dict]:
    from examples.rl.reverse_text.base_config import make_prompts, make_texts, reverse_text_score_fn
    from research_b200.training.grpo import GRPOConfig, grpo_train

    g = GRPOConfig(experiment_name="rl", model_name=model_name, lr=cfg.rl.lr, batch_size=cfg.rl.batch_size, n_samples_per_prompt=cfg.rl.n_samples_per_prompt,
                   num_minibatches=1, max_seq_len=cfg.model.max_length, max_tokens=cfg.rl.max_tokens, temperature=cfg.rl.temperature,
                   num_steps=cfg.rl.num_steps, checkpoint_every=0, max_batch_size=32, kv_blocks=256, output_dir=str(out), loss="grpo_clipped", seed=cfg.seed)
    prompts, truths = make_prompts(make_texts(cfg.rl.num_prompts, cfg.seed))
    return grpo_train(g, prompts, lambda s: reverse_text_score_fn(s, tokenizer), tokenizer=tokenizer, ground_truths=truths,
                      device=_device(cfg, int(os.environ.get("LOCAL_RANK", "0"))))


def launch_command(cfg: Config, script: str, config_path: str) -> list[str]:
    return [sys.executable, "-m", "torch.distributed.run", f"--nproc-per-node={len(cfg.target.gpu_ranks)}", "--nnodes=1",
            f"--master-addr={cfg.target.master_addr}", f"--master-port={cfg.target.master_port}", script, config_path]


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Post-training (SFT / RL) from a config file")
    ap.add_argument("config")
    a = ap.parse_args(argv)
    cfg: Config = load_config_from_file(a.config)
    use_fsdp = cfg.target.train_backend == "fsdp" and len(cfg.target.gpu_ranks) > 1
    if use_fsdp and os.environ.get("RANK") is None:
        env = os.environ.copy()
        if _device(cfg, 0) != "cpu":
            env["CUDA_VISIBLE_DEVICES"] = ",".join(str(r) for r in cfg.target.gpu_ranks)
        print(f"sharded backend on ranks {cfg.target.gpu_ranks}: relaunching under torch.distributed.run", flush=True)
        return subprocess.run(launch_command(cfg, str(Path(__file__).resolve()), str(Path(a.config).resolve())), env=env).returncode
    if use_fsdp:
        from research_b200.training.distributed_utils import init_process_group

        if _device(cfg, 0) != "cpu":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        init_process_group("gloo" if _device(cfg, 0) == "cpu" else "nccl")
    rank = int(os.environ.get("RANK", "0"))
    out = Path(cfg.output.save_dir) / cfg.output.experiment_name
    tokenizer = default_tokenizer()
    if rank == 0:
        out.mkdir(parents=True, exist_ok=True)
        (out / "config.json").write_text(json.dumps(config_to_dict(cfg), indent=2))
    model_name, summary = cfg.model.name, {}
    if cfg.output.mode in ("sft", "sft_then_rl"):
        hist, backend = run_sft(cfg, tokenizer, out)
        summary["sft"] = {"first_loss": hist[0]["loss"], "last_loss": hist[-1]["loss"], "steps": len(hist)}
        if cfg.output.mode == "sft_then_rl":
            model_name = str(backend.save_hf_checkpoint(out / "sft_hf"))
    if cfg.output.mode in ("rl", "sft_then_rl"):
        rl = run_rl(cfg, tokenizer, out, model_name)
        summary["rl"] = {"first_reward": rl[0]["mean_reward"], "last_reward": rl[-1]["mean_reward"], "steps": len(rl)}
    if rank == 0:
        (out / "summary.json").write_text(json.dumps(summary, indent=2))
        print(json.dumps(summary), flush=True)
    if use_fsdp:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
