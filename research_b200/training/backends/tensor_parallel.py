"""Tensor-parallel training of dense decoders, optionally times data parallelism (world = dp x tp).

The layout is the usual one for transformers. Inside each layer the projections that PRODUCE heads or hidden units
(q / k / v, gate / up) are split by output rows, so every rank computes its own heads and its own slice of the MLP with no
communication; the projections that CONSUME them (o, down) are split by input columns and yield partial sums that one
all-reduce per block completes. The output head is split over the vocabulary and the log-softmax runs on the shards
(max, sum of exponentials and the target's logit are reduced; the ``[tokens, vocabulary]`` logits never exist in one
place). Norms and the embedding are replicated.

Two autograd functions carry the communication: ``copy_to_group`` (identity forward, all-reduce of the gradient backward)
where replicated activations enter a split block, ``reduce_from_group`` (all-reduce forward, identity backward) where the
partial sums leave it. Everything else is the functional model of ``models/functional.py`` called with this rank's
weight shards and a config that says how many heads it holds, so the arithmetic of a rank is the oracle's own code.

The collectives are ``torch.distributed`` calls (gloo on CPU, NCCL on GPUs) and the matrix products are library
GEMMs: this backend is the plain, portable statement of tensor-parallel training with the same four-method surface and
loss registry as the other backends. The kernels that fuse these collectives into the GEMMs (``parallel/tp.py``) serve
the inference engine; they are not wired into this backend.
"""

from __future__ import annotations

from dataclasses import replace
from pathlib import Path
from typing import Any, Callable

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ...models.config import ModelConfig
from ...models.functional import attention, dense_mlp, rms_norm
from ...models.weights import init_random_weights
from ..losses import LOGPROB_LOSSES, shift_labels
from ..types import ImmediateTrainFuture, TrainerConfig, TrainFuture
from .torch_func import AdamWState, adamw_init, adamw_update

Params = dict[str, torch.Tensor]

# how a parameter is split over the tensor-parallel ranks: name suffix -> dimension (None: replicated)
ROW_SPLIT = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "q_proj.bias", "k_proj.bias", "v_proj.bias", "gate_proj.weight", "up_proj.weight")
COL_SPLIT = ("o_proj.weight", "down_proj.weight")
PARTIAL_GRAD = ("q_norm.weight", "k_norm.weight")      # replicated, but each rank sees only its own heads: gradients are summed


def split_dim(name: str) -> int | None:
    if name == "lm_head.weight" or name.endswith(ROW_SPLIT):
        return 0
    if name.endswith(COL_SPLIT):
        return 1
    return None


def shard_weights(full: Params, tp_rank: int, tp_size: int) -> Params:
    """This rank's share of a full state dict (Hugging Face names): equal contiguous slices along ``split_dim``."""
    out = {}
    for name, w in full.items():
        d = split_dim(name)
        if d is None or tp_size == 1:
            out[name] = w
        else:
            assert w.shape[d] % tp_size == 0, f"{name}: dimension {d} of size {w.shape[d]} does not divide over {tp_size} ranks"
            out[name] = w.chunk(tp_size, dim=d)[tp_rank].contiguous()
    return out


def unshard_weights(shards: list[Params]) -> Params:
    """The inverse of ``shard_weights`` from the shards of all ranks, in rank order."""
    return {name: (torch.cat([s[name] for s in shards], dim=split_dim(name)) if split_dim(name) is not None and len(shards) > 1 else shards[0][name])
            for name in shards[0]}


class _CopyToGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_group(x: torch.Tensor, group) -> torch.Tensor:
    return _CopyToGroup.apply(x, group) if group is not None else x


def reduce_from_group(x: torch.Tensor, group) -> torch.Tensor:
    return _ReduceFromGroup.apply(x, group) if group is not None else x


class _VocabParallelLogprob(torch.autograd.Function):
    """log p(target) and (optionally) the entropy of the softmax over a vocabulary that is split across ranks.
    ``logits`` is this rank's ``[..., V / tp]`` slice holding vocabulary entries ``[v0, v0 + V / tp)``."""

    @staticmethod
    def forward(ctx, logits, targets, v0, group, need_entropy):
        lf = logits.float()
        m = lf.max(-1).values
        if group is not None:
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = (lf - m[..., None]).exp()
        s = e.sum(-1)
        local = targets - v0
        mine = (local >= 0) & (local < lf.shape[-1]) & (targets >= 0)
        tl = torch.where(mine, lf.gather(-1, local.clamp(0, lf.shape[-1] - 1)[..., None])[..., 0], torch.zeros_like(m))
        stats = torch.stack([s, tl])
        if group is not None:
            dist.all_reduce(stats, group=group)
        s, tl = stats[0], stats[1]
        lse = m + s.log()
        p = e / s[..., None]
        lp = torch.where(targets >= 0, tl - lse, torch.zeros_like(lse))
        mean_logit = None
        ent = torch.zeros_like(lse)
        if need_entropy:
            mean_logit = (p * lf).sum(-1)
            if group is not None:
                dist.all_reduce(mean_logit, group=group)
            ent = lse - mean_logit
        ctx.save_for_backward(p, local, mine, targets, lf if need_entropy else None, mean_logit)
        ctx.in_dtype = logits.dtype
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        p, local, mine, targets, lf, mean_logit = ctx.saved_tensors
        g_lp = torch.where(targets >= 0, g_lp, torch.zeros_like(g_lp))
        d = -p * g_lp[..., None]
        d.scatter_add_(-1, local.clamp(0, p.shape[-1] - 1)[..., None], (g_lp * mine)[..., None])
        if lf is not None and g_ent is not None:
            d = d - g_ent[..., None] * p * (lf - mean_logit[..., None])
        return d.to(ctx.in_dtype), None, None, None, None


def vocab_parallel_logprob(logits: torch.Tensor, targets: torch.Tensor, v0: int, group, need_entropy: bool):
    return _VocabParallelLogprob.apply(logits, targets, v0, group, need_entropy)


def tp_forward_logprobs(params: Params, head: torch.Tensor, cfg_local: ModelConfig, ids: torch.Tensor, targets: torch.Tensor, v0: int, group,
                        need_entropy: bool):
    """The forward pass of one rank: replicated residual stream, split attention and MLP blocks, vocabulary-split head."""
    B, T = ids.shape
    positions = torch.arange(T, device=ids.device)[None].expand(B, T)
    x = F.embedding(ids, params["model.embed_tokens.weight"])
    for layer in range(cfg_local.num_layers):
        p = f"model.layers.{layer}."
        h = rms_norm(x, params[p + "input_layernorm.weight"], cfg_local.rms_norm_eps)
        x = x + reduce_from_group(attention(copy_to_group(h, group), params, p + "self_attn.", cfg_local, positions), group)
        h = rms_norm(x, params[p + "post_attention_layernorm.weight"], cfg_local.rms_norm_eps)
        x = x + reduce_from_group(dense_mlp(copy_to_group(h, group), params, p + "mlp."), group)
    x = rms_norm(x, params["model.norm.weight"], cfg_local.rms_norm_eps)
    logits = F.linear(copy_to_group(x, group), head)
    return vocab_parallel_logprob(logits, targets, v0, group, need_entropy)


class TensorParallelTrainingBackend:
    """``tp_size`` ranks share every sample (they must be fed the SAME batch); with ``world > tp_size`` the remaining factor is
    data parallelism: ranks ``[k * tp_size, (k + 1) * tp_size)`` form tensor-parallel group ``k`` and gradients are averaged
    over the ranks that hold the same shard. ``weights`` is the FULL state dict (every rank shards it itself)."""

    def __init__(self, model_config: ModelConfig, weights: Params | None = None, *, tp_size: int | None = None, device: torch.device | str | None = None,
                 loss_fn: str | Callable = "ce", loss_kwargs: dict | None = None, lr: float = 1e-5, betas: tuple[float, float] = (0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.0, trainer_config: TrainerConfig | None = None,
                 lr_schedule: Callable[[int], float] | None = None, checkpoint_dir: str | Path | None = None, need_entropy: bool | None = None,
                 seed: int = 0, dtype: torch.dtype = torch.float32, **_):
        assert not model_config.is_moe, "mixture-of-experts models train with expert parallelism (FSDPConfig(expert_parallel=True)), not with this backend"
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.tp_size = tp_size or self.world
        assert self.world % self.tp_size == 0, f"world size {self.world} is not a multiple of tp_size {self.tp_size}"
        self.dp_size = self.world // self.tp_size
        self.tp_rank, self.dp_rank = self.rank % self.tp_size, self.rank // self.tp_size
        self.tp_group = self.dp_group = None
        if self.world > 1:
            # every rank creates every group, in the same order (a requirement of new_group)
            for k in range(self.dp_size):
                g = dist.new_group(list(range(k * self.tp_size, (k + 1) * self.tp_size)))
                if k == self.dp_rank and self.tp_size > 1:
                    self.tp_group = g
            for j in range(self.tp_size):
                g = dist.new_group(list(range(j, self.world, self.tp_size)))
                if j == self.tp_rank and self.dp_size > 1:
                    self.dp_group = g
        cfg = model_config
        for what, n in (("attention heads", cfg.num_heads), ("key / value heads", cfg.num_kv_heads), ("MLP width", cfg.intermediate_size), ("vocabulary", cfg.vocab_size)):
            assert n % self.tp_size == 0, f"{what} ({n}) do not divide over {self.tp_size} tensor-parallel ranks"
        self.model_config = cfg
        self.cfg_local = replace(cfg, num_heads=cfg.num_heads // self.tp_size, num_kv_heads=cfg.num_kv_heads // self.tp_size,
                                 intermediate_size=cfg.intermediate_size // self.tp_size)
        self.device = torch.device(device or "cpu")
        self.dtype = dtype
        self.config = trainer_config or TrainerConfig()
        full = weights if weights is not None else init_random_weights(cfg, seed=seed)
        self.v_local = cfg.vocab_size // self.tp_size
        self.v0 = self.tp_rank * self.v_local
        self._install(full)
        self.loss_name = loss_fn if isinstance(loss_fn, str) else getattr(loss_fn, "__name__", "custom")
        self.loss_fn = LOGPROB_LOSSES[loss_fn] if isinstance(loss_fn, str) else loss_fn
        self.loss_kwargs = loss_kwargs or {}
        self.need_entropy = need_entropy if need_entropy is not None else self.loss_name.startswith("grpo")
        self.base_lr, self.lr, self.betas, self.eps, self.weight_decay = lr, lr, betas, eps, weight_decay
        self.lr_schedule = lr_schedule
        self.checkpoint_dir = Path(checkpoint_dir) if checkpoint_dir else None
        self.weight_version = 0
        self.current_step = 0
        self._accum = 0

    # ------------------------------------------------------------------ parameters
    def _install(self, full: Params) -> None:
        """fp32 master copies of this rank's shards (what the optimizer updates) and working copies in ``dtype``."""
        local = shard_weights({k: v.detach() for k, v in full.items()}, self.tp_rank, self.tp_size)
        self.master: Params = {k: v.to(self.device, torch.float32).clone() for k, v in local.items()}
        self.opt_state = adamw_init(self.master)
        self._refresh_working()

    def _refresh_working(self) -> None:
        self.params: Params = {k: v.detach().to(self.dtype).clone().requires_grad_(True) for k, v in self.master.items()}
        if self.model_config.tie_word_embeddings:
            # the head is this rank's rows of the embedding table, as a leaf of its own: its gradient is gathered into the
            # table's gradient after the backward pass (the look-up's gradient is replicated, the head's is split)
            table = self.master["model.embed_tokens.weight"]
            self.head = table[self.v0:self.v0 + self.v_local].detach().to(self.dtype).clone().requires_grad_(True)
        else:
            self.head = self.params["lm_head.weight"]

    def _sharded(self, name: str) -> bool:
        return split_dim(name) is not None and self.tp_size > 1

    # ------------------------------------------------------------------ batch preparation (as in the other backends)
    def _prepare(self, batch: dict[str, Any]) -> dict[str, torch.Tensor]:
        b = {k: (torch.as_tensor(v) if not isinstance(v, torch.Tensor) else v).to(self.device) for k, v in batch.items()
             if isinstance(v, (torch.Tensor, list, tuple))}
        labels = b.get("labels", b["input_ids"])
        mask = b.get("loss_mask")
        if mask is None:
            mask = (labels != -100).float()
            if "attention_mask" in b:
                mask = mask * b["attention_mask"].float()
        targets, shift_mask = shift_labels(labels, mask.float())
        b["targets"] = torch.where(shift_mask > 0, targets, torch.full_like(targets, -1))
        b["shift_mask"] = shift_mask
        return b

    def _check_same_batch(self, ids: torch.Tensor) -> None:
        """Ranks of one tensor-parallel group must see the same tokens: a cheap checksum catches a loader that feeds them
        different shards (the result would be silently wrong, not an error)."""
        if self.tp_group is None:
            return
        mine = torch.tensor([float(ids.double().sum()), float(ids.numel())], dtype=torch.float64, device=ids.device)
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.tp_group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.tp_group)
        assert torch.equal(lo, hi), "the ranks of a tensor-parallel group were given different batches"

    # ------------------------------------------------------------------ protocol
    def forward_backward(self, batch: dict[str, Any]) -> TrainFuture[dict[str, float]]:
        b = self._prepare(batch)
        self._check_same_batch(b["input_ids"])
        B = b["input_ids"].shape[0]
        n_micro = self.config.get_num_minibatches(B)
        mb = B // n_micro
        agg: dict[str, float] = {}
        for i in range(n_micro):
            sub = {k: (v[i * mb:(i + 1) * mb] if v.dim() > 0 and v.shape[0] == B else v) for k, v in b.items()}
            lp, ent = tp_forward_logprobs(self.params, self.head, self.cfg_local, sub["input_ids"], sub["targets"], self.v0, self.tp_group, self.need_entropy)
            out = self.loss_fn(lp, ent if self.need_entropy else None, sub, **self.loss_kwargs)
            loss, metrics = out
            assert torch.isfinite(loss), f"non-finite loss: {loss}"
            (loss / n_micro).backward()
            if "loss" not in metrics:
                agg["loss"] = agg.get("loss", 0.0) + float(loss.detach()) / n_micro
            for k, v in metrics.items():
                agg[k] = agg.get(k, 0.0) + float(v) / n_micro
        self._accum += 1
        agg["num_tokens"] = float(b["shift_mask"].sum())
        return ImmediateTrainFuture(agg, "forward_backward")

    def _collect_grads(self) -> Params:
        """Gradients of the master parameters for this step: averaged over accumulation and data parallelism, with the
        pieces that tensor parallelism leaves incomplete put together."""
        # copies: the reductions below work in place and must not touch ``.grad`` (this may be called more than once)
        grads = {k: (p.grad.detach().float().clone() if p.grad is not None else torch.zeros_like(p, dtype=torch.float32)) for k, p in self.params.items()}
        if self.model_config.tie_word_embeddings:
            hg = self.head.grad.detach().float().clone() if self.head.grad is not None else torch.zeros_like(self.head, dtype=torch.float32)
            if self.tp_group is not None:
                parts = [torch.empty_like(hg) for _ in range(self.tp_size)]
                dist.all_gather(parts, hg.contiguous(), group=self.tp_group)
                hg = torch.cat(parts, 0)
            grads["model.embed_tokens.weight"] = grads["model.embed_tokens.weight"] + hg
        if self.tp_group is not None:
            for k in grads:
                if k.endswith(PARTIAL_GRAD):
                    dist.all_reduce(grads[k], group=self.tp_group)
        scale = 1.0 / max(self._accum, 1)
        for k in grads:
            if self.dp_group is not None:
                dist.all_reduce(grads[k], group=self.dp_group)
                grads[k] = grads[k] * (scale / self.dp_size)
            elif scale != 1.0:
                grads[k] = grads[k] * scale
        return grads

    def _global_grad_norm(self, grads: Params) -> torch.Tensor:
        split = sum((g.double() ** 2).sum() for k, g in grads.items() if self._sharded(k))
        whole = sum((g.double() ** 2).sum() for k, g in grads.items() if not self._sharded(k))
        split = torch.as_tensor(split, dtype=torch.float64, device=self.device)
        if self.tp_group is not None:
            dist.all_reduce(split, group=self.tp_group)          # every rank holds a different slice of these
        return torch.sqrt(split + whole).float()

    def optim_step(self) -> TrainFuture[dict[str, float]]:
        assert self._accum > 0, "optim_step before any forward_backward"
        if self.lr_schedule is not None:
            self.lr = self.base_lr * self.lr_schedule(self.current_step)
        grads = self._collect_grads()
        norm = self._global_grad_norm(grads)
        max_norm = self.config.max_grad_norm or 0.0
        if max_norm > 0:
            coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
            grads = {k: g * coef for k, g in grads.items()}
        with torch.no_grad():
            self.master, self.opt_state = adamw_update(self.master, grads, self.opt_state, self.lr, self.betas, self.eps, self.weight_decay)
        self._refresh_working()
        self._accum = 0
        self.current_step += 1
        self.weight_version += 1
        return ImmediateTrainFuture({"lr": self.lr, "step": self.current_step, "grad_norm": float(norm)}, "optim_step")

    def _gather(self, local: Params) -> Params:
        """Full tensors from every rank's shards (replicated ones as they are)."""
        out = {}
        for k, v in local.items():
            if self._sharded(k) and self.tp_group is not None:
                parts = [torch.empty_like(v) for _ in range(self.tp_size)]
                dist.all_gather(parts, v.contiguous(), group=self.tp_group)
                out[k] = torch.cat(parts, dim=split_dim(k))
            else:
                out[k] = v.clone()
        return out

    def get_weights(self) -> TrainFuture[dict[str, Any]]:
        """The FULL state dict in the working dtype (a collective over the tensor-parallel group: every rank calls it)."""
        return ImmediateTrainFuture({k: v.to(self.dtype) for k, v in self._gather(self.master).items()}, "get_weights")

    def gathered_grads(self) -> Params:
        """The full gradient of the last backward passes, as ``optim_step`` would use it (for checks against an oracle)."""
        return self._gather(self._collect_grads())

    def load_weights(self, weights: dict[str, Any]) -> TrainFuture[None]:
        missing = {k for k in self.master if k not in weights}
        assert not missing, f"missing weights: {sorted(missing)[:5]}"
        state = self.opt_state
        self._install({k: weights[k] for k in self.master})
        self.opt_state = state                                  # new weights, same optimizer history
        self.weight_version += 1
        return ImmediateTrainFuture(None, "load_weights")

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, step: int | None = None, metrics: dict[str, float] | None = None) -> Path | None:
        """``<checkpoint_dir>/step_NNNNNN/``: the full model as a safetensors directory (written once, by global rank 0) and
        one optimizer-state file per tensor-parallel rank of the first data-parallel group."""
        from ...models.weights import save_safetensors_dir

        assert self.checkpoint_dir is not None, "no checkpoint_dir"
        step = self.current_step if step is None else step
        d = self.checkpoint_dir / f"step_{step:06d}"
        full = self._gather(self.master)
        if self.rank == 0:
            save_safetensors_dir({k: v.to(self.dtype) for k, v in full.items()}, self.model_config, d / "hf")
        if self.dp_rank == 0:
            d.mkdir(parents=True, exist_ok=True)
            torch.save({"m": self.opt_state.m, "v": self.opt_state.v, "opt_step": self.opt_state.step, "master": self.master, "step": self.current_step,
                        "weight_version": self.weight_version, "tp_size": self.tp_size, "metrics": metrics or {}}, d / f"optimizer_tp{self.tp_rank}.pt")
        if self.world > 1:
            dist.barrier()
        return d

    def load_checkpoint(self, path: Path | str) -> dict[str, Any]:
        d = torch.load(Path(path) / f"optimizer_tp{self.tp_rank}.pt", map_location=self.device, weights_only=False)
        assert d["tp_size"] == self.tp_size, f"checkpoint was written with tp_size {d['tp_size']}, this run has {self.tp_size}: load hf/ instead"
        self.master = d["master"]
        self.opt_state = AdamWState(d["opt_step"], d["m"], d["v"])
        self.current_step, self.weight_version = d["step"], d["weight_version"]
        self._refresh_working()
        return d.get("metrics", {})
