"""Functional training backend on ``torch.func`` (the reference plans this backend and ships it as a stub:
rollouts/training/backends/torch_func.py:27-176, "JAX-style functional training, immutable parameter updates").

Here it is a working backend over the functional model oracle (``models/functional.py``): parameters, gradient
accumulator and optimizer state are plain dicts of tensors that are *replaced*, never mutated, by pure functions
(``adamw_update``); gradients come from ``torch.func.grad`` of a closed-over loss, so per-sample gradients or other
transforms (``vmap``) compose with it. It is the slow, transparent counterpart of ``NativeTrainingBackend`` (same
four-method surface, same loss registry), meant for experiments and as a numerical cross-check of the kernel path,
not for throughput.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Callable, NamedTuple

import torch
from torch.func import grad

from ...models.config import ModelConfig
from ...models.functional import causal_lm_forward
from ...models.weights import init_random_weights
from ..losses import LOGPROB_LOSSES, shift_labels
from ..types import ImmediateTrainFuture, TrainerConfig, TrainFuture

Params = dict[str, torch.Tensor]


class AdamWState(NamedTuple):
    step: int
    m: Params
    v: Params


def adamw_init(params: Params) -> AdamWState:
    return AdamWState(0, {k: torch.zeros_like(p) for k, p in params.items()}, {k: torch.zeros_like(p) for k, p in params.items()})


def adamw_update(params: Params, grads: Params, state: AdamWState, lr: float, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.0) -> tuple[Params, AdamWState]:
    """One decoupled-weight-decay Adam step as a pure function: returns new parameters and a new state."""
    b1, b2 = betas
    t = state.step + 1
    m = {k: b1 * state.m[k] + (1 - b1) * g for k, g in grads.items()}
    v = {k: b2 * state.v[k] + (1 - b2) * g * g for k, g in grads.items()}
    c1, c2 = 1 - b1 ** t, 1 - b2 ** t
    new = {k: p * (1 - lr * weight_decay) - lr * (m[k] / c1) / ((v[k] / c2).sqrt() + eps) for k, p in params.items()}
    return new, AdamWState(t, m, v)


def global_norm(tree: Params) -> torch.Tensor:
    return torch.sqrt(sum((g.double() ** 2).sum() for g in tree.values())).float()


def clip_by_global_norm(grads: Params, max_norm: float) -> tuple[Params, torch.Tensor]:
    n = global_norm(grads)
    if max_norm and max_norm > 0:
        scale = torch.clamp(max_norm / (n + 1e-6), max=1.0)
        grads = {k: g * scale for k, g in grads.items()}
    return grads, n


def token_logprobs(params: Params, cfg: ModelConfig, ids: torch.Tensor, targets: torch.Tensor, need_entropy: bool):
    logits = causal_lm_forward(ids, params, cfg).float()
    lsm = torch.log_softmax(logits, -1)
    lp = lsm.gather(-1, targets.clamp(min=0)[..., None])[..., 0]
    lp = torch.where(targets >= 0, lp, torch.zeros_like(lp))
    ent = -(lsm.exp() * lsm).sum(-1) if need_entropy else None
    return lp, ent


class TorchFuncTrainingBackend:
    def __init__(self, model_config: ModelConfig, weights: Params | None = None, *, device: torch.device | str | None = None,
                 loss_fn: str | Callable = "grpo", loss_kwargs: dict | None = None, lr: float = 1e-5,
                 betas: tuple[float, float] = (0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0,
                 trainer_config: TrainerConfig | None = None, lr_schedule: Callable[[int], float] | None = None,
                 checkpoint_dir: str | Path | None = None, need_entropy: bool | None = None, seed: int = 0, dtype=torch.float32, **_):
        self.device = torch.device(device or "cpu")
        self.model_config = model_config
        self.config = trainer_config or TrainerConfig()
        weights = weights if weights is not None else init_random_weights(model_config, seed=seed)
        self.params: Params = {k: v.detach().to(self.device, dtype).clone() for k, v in weights.items()}
        self.opt_state = adamw_init(self.params)
        self.grads: Params | None = None
        self._accum = 0
        self.loss_name = loss_fn if isinstance(loss_fn, str) else getattr(loss_fn, "__name__", "custom")
        self.loss_fn = LOGPROB_LOSSES[loss_fn] if isinstance(loss_fn, str) else loss_fn
        self.loss_kwargs = loss_kwargs or {}
        self.need_entropy = need_entropy if need_entropy is not None else self.loss_name.startswith("grpo")
        self.base_lr, self.lr, self.betas, self.eps, self.weight_decay = lr, lr, betas, eps, weight_decay
        self.lr_schedule = lr_schedule
        self.checkpoint_dir = Path(checkpoint_dir) if checkpoint_dir else None
        self.rank, self.world = 0, 1
        self.weight_version = 0
        self.current_step = 0

    # ------------------------------------------------------------------ the pure loss
    def loss_of(self, params: Params, batch: dict[str, torch.Tensor]) -> tuple[torch.Tensor, dict[str, float]]:
        lp, ent = token_logprobs(params, self.model_config, batch["input_ids"], batch["targets"], self.need_entropy)
        return self.loss_fn(lp, ent, batch, **self.loss_kwargs)

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

    # ------------------------------------------------------------------ protocol
    def forward_backward(self, batch: dict[str, Any]) -> TrainFuture[dict[str, float]]:
        b = self._prepare(batch)
        B = b["input_ids"].shape[0]
        n_micro = self.config.get_num_minibatches(B)
        mb = B // n_micro
        agg: dict[str, float] = {}
        for i in range(n_micro):
            sub = {k: (v[i * mb:(i + 1) * mb] if v.dim() > 0 and v.shape[0] == B else v) for k, v in b.items()}
            seen: dict[str, float] = {}

            def scalar(p: Params):
                loss, metrics = self.loss_of(p, sub)
                seen.update(metrics)
                return loss / n_micro, loss.detach()

            g, loss = grad(scalar, has_aux=True)(self.params)
            metrics = seen
            assert torch.isfinite(loss), f"non-finite loss: {loss}"
            self.grads = g if self.grads is None else {k: self.grads[k] + g[k] for k in g}
            if "loss" not in metrics:
                agg["loss"] = agg.get("loss", 0.0) + float(loss) / n_micro
            for k, v in metrics.items():
                agg[k] = agg.get(k, 0.0) + float(v) / n_micro
        self._accum += 1
        agg["grad_norm_local"] = float(global_norm(self.grads))
        agg["num_tokens"] = float(b["shift_mask"].sum())
        return ImmediateTrainFuture(agg, "forward_backward")

    def optim_step(self) -> TrainFuture[dict[str, float]]:
        assert self.grads is not None, "optim_step before any forward_backward"
        if self.lr_schedule is not None:
            self.lr = self.base_lr * self.lr_schedule(self.current_step)
        grads = {k: g / max(self._accum, 1) for k, g in self.grads.items()}
        grads, norm = clip_by_global_norm(grads, self.config.max_grad_norm or 0.0)
        self.params, self.opt_state = adamw_update(self.params, grads, self.opt_state, self.lr, self.betas, self.eps, self.weight_decay)
        self.grads, self._accum = None, 0
        self.current_step += 1
        self.weight_version += 1
        return ImmediateTrainFuture({"lr": self.lr, "step": self.current_step, "grad_norm": float(norm)}, "optim_step")

    def get_weights(self) -> TrainFuture[dict[str, Any]]:
        return ImmediateTrainFuture({k: v.detach().clone() for k, v in self.params.items()}, "get_weights")

    def load_weights(self, weights: dict[str, Any]) -> TrainFuture[None]:
        missing = set(self.params) - set(weights)
        assert not missing, f"missing weights: {sorted(missing)[:5]}"
        self.params = {k: weights[k].detach().to(self.device, self.params[k].dtype).clone() for k in self.params}
        self.weight_version += 1
        return ImmediateTrainFuture(None, "load_weights")

    # ------------------------------------------------------------------ extras the functional form makes cheap
    def per_sample_grad_norms(self, batch: dict[str, Any]) -> torch.Tensor:
        """Gradient norm of every sample of the batch on its own (one ``grad`` call per row; the loss functions
        call ``.item()`` for their metrics, which ``vmap`` cannot trace)."""
        b = self._prepare(batch)
        B = b["input_ids"].shape[0]
        out = []
        for i in range(B):
            sub = {k: (v[i:i + 1] if v.dim() > 0 and v.shape[0] == B else v) for k, v in b.items()}
            out.append(global_norm(grad(lambda p: self.loss_of(p, sub)[0])(self.params)))
        return torch.stack(out)

    def save_checkpoint(self, step: int | None = None, metrics: dict[str, float] | None = None) -> Path:
        assert self.checkpoint_dir is not None, "no checkpoint_dir"
        path = self.checkpoint_dir / f"step_{step if step is not None else self.current_step:06d}.pt"
        path.parent.mkdir(parents=True, exist_ok=True)
        torch.save({"params": self.params, "m": self.opt_state.m, "v": self.opt_state.v, "opt_step": self.opt_state.step,
                    "step": self.current_step, "weight_version": self.weight_version, "metrics": metrics or {}}, path)
        return path

    def load_checkpoint(self, path: Path | str) -> dict[str, Any]:
        d = torch.load(path, map_location=self.device)
        self.params = d["params"]
        self.opt_state = AdamWState(d["opt_step"], d["m"], d["v"])
        self.current_step, self.weight_version = d["step"], d["weight_version"]
        return d.get("metrics", {})
