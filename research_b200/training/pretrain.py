"""Language-model pretraining from a TOML experiment file (the reference ships the package as a placeholder with one
config, pretrain/configs/dsv3_tiny.toml:1-16: ``[model]`` hidden_size / num_layers / num_attention_heads / num_experts /
num_active_experts, ``[training]`` batch_size / seq_len / lr, ``[data]`` path). Here the file drives a real loop:

* the model section becomes a sparse mixture-of-experts ``ModelConfig`` (a DeepSeek-V3-style layout: sigmoid router,
  one shared expert, the first layer dense), or a dense one when ``num_experts`` is 0;
* data are packed token shards (``training/datasets/packed_shards.py``) found under ``[data].path``; when that
  directory has none, ``synthetic = true`` in ``[data]`` (or ``synthetic=True`` to ``pretrain``) substitutes a
  repeating-pattern token stream so the loop can be exercised anywhere;
* every step is ``forward_backward`` + ``optim_step`` of a ``TrainingBackend`` (next-token cross-entropy, warm-up +
  cosine learning rate, gradient clipping), with tokens/s and the loss logged per step and an optional checkpoint.

    python -m research_b200.training.pretrain configs/dsv3_tiny.toml --steps 100 [--synthetic]
"""

from __future__ import annotations

import argparse
import json
import time
import tomllib
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Any, Callable, Iterator, Sequence

import torch

from ..models.config import ModelConfig


@dataclass(frozen=True)
class PretrainModel:
    hidden_size: int = 1024
    num_layers: int = 4
    num_attention_heads: int = 8
    num_kv_heads: int = 0              # 0: same as the attention heads
    num_experts: int = 8
    num_active_experts: int = 2
    vocab_size: int = 32768
    intermediate_size: int = 0         # 0: 8/3 of the hidden size rounded up to 128 (dense layers / shared expert)
    moe_intermediate_size: int = 0     # 0: intermediate_size / num_active_experts rounded up to 128
    num_shared_experts: int = 1
    first_dense_layers: int = 1


@dataclass(frozen=True)
class PretrainTraining:
    batch_size: int = 4
    seq_len: int = 2048
    lr: float = 1e-4
    steps: int = 100
    warmup_steps: int = 10
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    seed: int = 0
    checkpoint_every: int = 0
    checkpoint_dir: str = ""


@dataclass(frozen=True)
class PretrainData:
    path: str = ""
    bos_id: int = 1
    synthetic: bool = False


@dataclass(frozen=True)
class PretrainConfig:
    model: PretrainModel = field(default_factory=PretrainModel)
    training: PretrainTraining = field(default_factory=PretrainTraining)
    data: PretrainData = field(default_factory=PretrainData)

    @staticmethod
    def from_toml(path: str | Path) -> "PretrainConfig":
        raw = tomllib.loads(Path(path).read_text())
        unknown = set(raw) - {"model", "training", "data"}
        if unknown:
            raise ValueError(f"{path}: unknown sections {sorted(unknown)}")

        def section(cls, d: dict[str, Any]):
            bad = set(d) - set(cls.__dataclass_fields__)
            if bad:
                raise ValueError(f"{path}: [{cls.__name__[8:].lower()}] has unknown keys {sorted(bad)}")
            return cls(**d)

        return PretrainConfig(section(PretrainModel, raw.get("model", {})), section(PretrainTraining, raw.get("training", {})),
                              section(PretrainData, raw.get("data", {})))

    def model_config(self) -> ModelConfig:
        m = self.model
        if m.hidden_size % m.num_attention_heads:
            raise ValueError("hidden_size must be a multiple of num_attention_heads")
        up128 = lambda x: -(-int(x) // 128) * 128                                        # noqa: E731
        inter = m.intermediate_size or up128(m.hidden_size * 8 / 3)
        common = dict(vocab_size=m.vocab_size, hidden_size=m.hidden_size, num_layers=m.num_layers, num_heads=m.num_attention_heads,
                      num_kv_heads=m.num_kv_heads or m.num_attention_heads, head_dim=m.hidden_size // m.num_attention_heads,
                      intermediate_size=inter, max_position_embeddings=max(self.training.seq_len, 2048), tie_word_embeddings=False,
                      attention_bias=False)
        if m.num_experts == 0:
            return ModelConfig(family="llama", **common)
        if not 0 < m.num_active_experts <= m.num_experts:
            raise ValueError("num_active_experts must lie in 1..num_experts")
        return ModelConfig(family="glm4_moe", num_experts=m.num_experts, num_experts_per_tok=m.num_active_experts,
                           moe_intermediate_size=m.moe_intermediate_size or up128(inter / m.num_active_experts),
                           router_type="sigmoid", norm_topk_prob=True, n_shared_experts=m.num_shared_experts,
                           first_k_dense_replace=min(m.first_dense_layers, m.num_layers), **common)


def synthetic_batches(vocab: int, batch: int, seq_len: int, seed: int = 0) -> Iterator[dict[str, torch.Tensor]]:
    """Sequences ``t[i+1] = (a * t[i] + c) mod vocab`` with a few (a, c) pairs: learnable, so the loss must fall."""
    g = torch.Generator().manual_seed(seed)
    rules = [(3, 1), (5, 7), (7, 3), (11, 5)]
    while True:
        start = torch.randint(0, vocab, (batch,), generator=g)
        which = torch.randint(0, len(rules), (batch,), generator=g)
        rows = []
        for s, w in zip(start.tolist(), which.tolist()):
            a, c = rules[w]
            row = [s]
            for _ in range(seq_len - 1):
                row.append((a * row[-1] + c) % vocab)
            rows.append(row)
        ids = torch.tensor(rows, dtype=torch.long)
        yield {"input_ids": ids, "labels": ids.clone()}


def shard_batches(files: Sequence[Path], batch: int, seq_len: int, bos_id: int, rank: int = 0, world: int = 1) -> Iterator[dict[str, torch.Tensor]]:
    """Rows of ``seq_len`` packed tokens with their next-token labels (the last position of a row has none). Loops over
    the shards for ever."""
    from .datasets.packed_shards import packed_batches

    packs = packed_batches(files, batch * seq_len, seq_len, bos_id, rank, world, loop=True)
    for inputs, targets, _cu in packs:
        ids = inputs.view(batch, seq_len).long()
        nxt = targets.view(batch, seq_len).long()
        labels = torch.cat([ids[:, :1], nxt[:, :-1]], 1)             # the backend shifts labels left by one itself
        yield {"input_ids": ids, "labels": labels}


def find_shards(path: str) -> list[Path]:
    p = Path(path) if path else None
    return sorted(p.glob("*.bin")) if p and p.is_dir() else []


def pretrain(cfg: PretrainConfig, steps: int | None = None, device: str | None = None, synthetic: bool | None = None,
             backend_factory: Callable[..., Any] | None = None, log: Callable[[str], None] | None = print,
             kernel_table: str | Path | None = None) -> list[dict[str, float]]:
    """Run the loop; returns one metrics dict per step (``loss``, ``lr``, ``grad_norm``, ``tokens_per_s``, ``step_s``).
    ``kernel_table`` (CUDA only): after the loop, one more step runs under the PyTorch profiler and the device time
    per kernel is written to that file."""
    from .backends.native import NativeTrainingBackend, warmup_cosine
    from .types import TrainerConfig

    t = cfg.training
    steps = steps if steps is not None else t.steps
    mc = cfg.model_config()
    make = backend_factory or NativeTrainingBackend
    backend = make(mc, device=device, loss_fn="pretrain", lr=t.lr, weight_decay=t.weight_decay, seed=t.seed,
                   trainer_config=TrainerConfig(max_grad_norm=t.max_grad_norm), lr_schedule=warmup_cosine(t.warmup_steps, max(steps, 1)),
                   checkpoint_dir=t.checkpoint_dir or None)
    files = find_shards(cfg.data.path)
    use_synth = synthetic if synthetic is not None else (cfg.data.synthetic or not files)
    if not use_synth and not files:
        raise FileNotFoundError(f"no *.bin token shards under {cfg.data.path!r}")
    if use_synth and not (cfg.data.synthetic or synthetic) and log:
        log(f"no token shards under {cfg.data.path!r}: using the synthetic stream")
    rank, world = getattr(backend, "rank", 0), getattr(backend, "world", 1)
    data = (synthetic_batches(mc.vocab_size, t.batch_size, t.seq_len, t.seed + rank) if use_synth
            else shard_batches(files, t.batch_size, t.seq_len, cfg.data.bos_id, rank, world))
    if log:
        log(f"model: {mc.family} {mc.num_params() / 1e6:.1f}M params, {mc.num_layers} layers, d={mc.hidden_size}"
            + (f", {mc.num_experts} experts top-{mc.num_experts_per_tok}" if mc.is_moe else "")
            + f" | batch {t.batch_size} x {t.seq_len} tokens, {steps} steps")
    history = []
    for step in range(steps):
        t0 = time.perf_counter()
        m = backend.forward_backward(next(data)).wait()
        o = backend.optim_step().wait()
        if str(backend.device).startswith("cuda"):
            torch.cuda.synchronize(backend.device)
        dt = time.perf_counter() - t0
        rec = {"step": step + 1, "loss": m["loss"], "lr": o["lr"], "grad_norm": o["grad_norm"], "step_s": dt,
               "tokens_per_s": world * t.batch_size * t.seq_len / dt}
        history.append(rec)
        if log:
            log(f"step {rec['step']:5d}  loss {rec['loss']:.4f}  lr {rec['lr']:.2e}  |g| {rec['grad_norm']:.3f}  {rec['tokens_per_s']:,.0f} tok/s")
        if t.checkpoint_every and t.checkpoint_dir and (step + 1) % t.checkpoint_every == 0:
            backend.save_checkpoint(step + 1, {"loss": rec["loss"]})
    if kernel_table and str(backend.device).startswith("cuda"):
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            backend.forward_backward(next(data)).wait()
            backend.optim_step().wait()
            torch.cuda.synchronize(backend.device)
        rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
        total = sum(e.device_time_total for e in rows) or 1.0
        with open(kernel_table, "w") as f:
            f.write(f"# device time per kernel, one pretraining step ({mc.family}, {mc.num_params() / 1e6:.0f}M params, batch "
                    f"{t.batch_size} x {t.seq_len}); total {total / 1e3:.1f} ms under the profiler\n")
            for e in rows[:40]:
                f.write(f"{e.device_time_total / total * 100:5.1f}%  n={e.count:5d}  avg={e.device_time_total / max(e.count, 1):9.1f}us  {e.key[:110]}\n")
    return history


def main(argv: Sequence[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Pretrain from a TOML config")
    ap.add_argument("config")
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--device", default=None)
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--seq-len", type=int, default=None, help="override [training].seq_len")
    ap.add_argument("--json", default="", help="write the per-step metrics here")
    ap.add_argument("--kernel-table", default="", help="write device time per kernel of one extra, profiled step here (CUDA)")
    a = ap.parse_args(argv)
    cfg = PretrainConfig.from_toml(a.config)
    if a.seq_len:
        cfg = replace(cfg, training=replace(cfg.training, seq_len=a.seq_len))
    hist = pretrain(cfg, a.steps, a.device, True if a.synthetic else None, kernel_table=a.kernel_table or None)
    if a.json:
        Path(a.json).write_text(json.dumps(hist))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
