"""Training backend on the native model, the flat buckets and the sharded AdamW.

One implementation serves both public backends: ``PyTorchTrainingBackend`` (one GPU; the
reference's single-device backend, rollouts/training/backends/pytorch.py:42-730) and
``FSDPTrainingBackend`` (one rank per GPU; rollouts/training/backends/fsdp.py:61-766). The
Tinker-style surface is the reference's: ``forward_backward`` -> ``optim_step`` returning
futures, ``get_weights`` / ``load_weights``, checkpoints with ``weight_version`` and step.

Per step, end to end: the batch arrives as host tensors, is staged through pinned memory and
copied to the device, split into micro-batches, run forward+backward through the kernels
(gradients accumulate in the flat bucket), and ``optim_step`` runs reduce-scatter + clip +
AdamW + all-gather as three fused kernel families. Loss metrics come back with one
device->host read per ``forward_backward``.
"""

from __future__ import annotations

import json
import math
import re
import time
from pathlib import Path
from typing import Any, Callable

import torch

from ...models.config import ModelConfig
from ...models.weights import param_shapes, save_safetensors, save_safetensors_dir
from ...ops import train as T
from ...parallel.fsdp import FlatBuckets, ShardedAdamW
from ...parallel.symm import LocalComm, PeerComm
from ..losses import LOGPROB_LOSSES, shift_labels
from ..native_model import NativeCausalLM
from ..types import ImmediateTrainFuture, TrainerConfig, TrainFuture


def _chunk_of(name: str) -> int:
    if name.startswith("model.layers."):
        return 1 + int(name.split(".")[2])
    return 0 if name.startswith("model.embed") else 10_000


# Order of a layer's parameters inside its chunk: projections that share their input lie back to back (q|k|v,
# gate|up, and their biases), so each group runs as one stacked GEMM in forward, dgrad and wgrad.
_GROUPED = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
            "self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias",
            "mlp.gate_proj.weight", "mlp.up_proj.weight")


_EXPERT = re.compile(r"(.*\.mlp\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


def _order_key(name: str, chunk_of=_chunk_of) -> tuple:
    m = _EXPERT.match(name)
    if m:
        # a layer's experts: every expert's gate then up rows back to back ([E * 2F, d] as one stacked matrix), then
        # all down projections ([E * d, F]): the grouped expert GEMMs of training address them as two matrices
        proj = m.group(3)
        return (chunk_of(name), m.group(1), 1 if proj == "down_proj" else 0, int(m.group(2)), 0 if proj == "gate_proj" else 1, name)
    for i, suffix in enumerate(_GROUPED):
        if name.endswith(suffix):
            return (chunk_of(name), name[:-len(suffix)], i, name)
    return (chunk_of(name), name, len(_GROUPED), name)


def _shardable(name: str, shape: tuple, world: int) -> bool:
    """Sharded-parameter mode splits the rows of every weight matrix of the decoder layers (87 % of an 8B model);
    embeddings, the lm_head and all vectors stay whole on every rank (sharded gradients and optimizer state only)."""
    if not name.startswith("model.layers.") or len(shape) != 2 or ".experts." in name or name.endswith("gate.weight"):
        return False
    return shape[0] % world == 0 and (shape[0] // world * shape[1]) % 8 == 0 and shape[0] // world >= 64


_VECTOR_CHUNK = 9_000     # sharded mode: the layers' vectors (norm weights, biases) live in one chunk of their own


_EXPERT_CHUNK = 20_000    # expert-parallel training: a layer's own experts live in chunk _EXPERT_CHUNK + layer


def build_buckets(model_config: ModelConfig, comm, dtype: torch.dtype, shard_params: bool = False, param_comm=None,
                  with_grads: bool = True, expert_parallel: bool = False) -> FlatBuckets:
    """The flat parameter / gradient layout of a model for ``comm.world`` training ranks. A rank outside the training
    group (an inference engine on its own GPU) builds the SAME layout with a stand-in ``comm`` of the trainers' size and
    ``with_grads=False``: it then knows where every parameter lies in the trainers' storage (``param_comm``: the
    symmetric memory both sides share)."""
    all_shapes = param_shapes(model_config)
    chunk_of, rule = _chunk_of, None
    owned_rule, ep = None, None
    if expert_parallel and comm.world > 1 and model_config.is_moe:
        # Expert-parallel training: rank r keeps experts [r * E / W, (r + 1) * E / W) of every layer and nobody else
        # does: their parameters, gradients and optimizer state exist once in the job. Everything else is laid out as
        # before. Every rank lists the same NUMBER of experts, so offsets agree between the ranks although names differ.
        W, E = comm.world, model_config.num_experts
        assert E % W == 0, f"{E} experts do not split over {W} ranks"
        EL = E // W
        lo = comm.rank * EL

        def owned_rule(name):
            return _EXPERT.match(name) is not None

        all_shapes = {n: s for n, s in all_shapes.items()
                      if (m := _EXPERT.match(n)) is None or lo <= int(m.group(2)) < lo + EL}
        base_chunk_of = chunk_of

        def chunk_of(name, base=base_chunk_of):
            return _EXPERT_CHUNK + int(name.split(".")[2]) if _EXPERT.match(name) else base(name)

        ep = (comm.rank, W, EL)
    if shard_params and comm.world > 1:
        W = comm.world

        def rule(name, shape):
            return _shardable(name, shape, W)

        def chunk_of(name):      # a layer's chunk keeps its sharded matrices only
            return _chunk_of(name) if (not name.startswith("model.layers.") or rule(name, tuple(all_shapes[name]))) else _VECTOR_CHUNK

    shapes = sorted(all_shapes.items(), key=lambda kv: _order_key(kv[0], chunk_of))
    fb = FlatBuckets(comm, shapes, chunk_of, dtype=dtype, shard_rule=rule, param_comm=param_comm, with_grads=with_grads,
                     owned_rule=owned_rule)
    fb.expert_parallel = ep          # (rank, ranks, experts per rank) or None
    return fb


class NativeTrainingBackend:
    def __init__(self, model_config: ModelConfig, weights: dict[str, torch.Tensor] | None = None, *,
                 comm: PeerComm | None = None, device: torch.device | str | None = None,
                 loss_fn: str | Callable = "grpo", loss_kwargs: dict | None = None, lr: float = 1e-5,
                 betas: tuple[float, float] = (0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0,
                 trainer_config: TrainerConfig | None = None, lr_schedule: Callable[[int], float] | None = None,
                 checkpoint_dir: str | Path | None = None, activation_checkpointing: bool = False,
                 need_entropy: bool | None = None, seed: int = 0, overlap_comm: bool = True, shard_params: bool = False,
                 param_comm: PeerComm | None = None, expert_parallel: bool = False):
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda" if torch.cuda.is_available() else "cpu")
        self.comm = comm if comm is not None else LocalComm(self.device)
        self.rank, self.world = self.comm.rank, self.comm.world
        self.model_config = model_config
        self.config = trainer_config or TrainerConfig()
        on_gpu = self.device.type == "cuda"
        dtype = torch.bfloat16 if on_gpu else torch.float32
        self.shard_params = bool(shard_params) and self.world > 1
        self.expert_parallel = bool(expert_parallel) and self.world > 1 and model_config.is_moe
        assert not (self.expert_parallel and self.shard_params), "expert-parallel training keeps the other parameters replicated"
        self.buckets = build_buckets(model_config, self.comm, dtype, self.shard_params, param_comm, expert_parallel=self.expert_parallel)
        if weights is None and on_gpu:
            # random init written straight into the bucket (an 8B model never exists twice in memory)
            # whole tensors: the same seed on every rank gives every rank the same values; row slabs: seeded per rank
            g = torch.Generator(device=self.device).manual_seed(seed)
            g_slab = torch.Generator(device=self.device).manual_seed(seed * 1009 + 1 + self.rank)
            for n, sp in self.buckets.specs.items():
                v = self.buckets.param_view(n)       # the whole tensor, or this rank's row slab
                if n.endswith("norm.weight") or n.endswith("layernorm.weight"):
                    v.fill_(1.0)
                elif n.endswith(".bias"):
                    v.zero_()
                else:
                    v.normal_(0.0, model_config.init_std, generator=g_slab if (sp.sharded or sp.owned) else g)
        else:
            if weights is None:
                from ...models.weights import init_random_weights

                weights = init_random_weights(model_config, seed=seed)
            for n in self.buckets.specs:
                self.buckets.set_param(n, weights[n])
        self.comm.barrier_host()
        max_norm = self.config.max_grad_norm if self.config.max_grad_norm is not None else 0.0
        self.optimizer = ShardedAdamW(self.buckets, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      max_grad_norm=max_norm)
        self.base_lr = lr
        self.lr_schedule = lr_schedule
        # On the GPU the kernels write each gradient view in place of the old one on its first write of a window, so
        # the 2 bytes per parameter of the bucket are neither zeroed nor re-read per step.
        self.buckets.track_writes = on_gpu
        self.optimizer.zero_grads_after_step = not on_gpu
        # Reduce-scatter of a layer's gradients as soon as backward has left the layer, on a second stream
        # (what FSDP2's backward hooks do in the reference, rollouts/training/backends/fsdp.py:289-322).
        self.overlap_comm = bool(overlap_comm) and on_gpu and self.world > 1
        self._side = torch.cuda.Stream(self.device) if (bool(overlap_comm) and on_gpu) else None
        self._pass_reduced: set[int] = set()
        if self.overlap_comm:
            self.optimizer.overlap_grid = 64
        if self._side is not None:
            # AdamW (+ the parameter all-gather) of a step runs on the second stream, chunk by chunk in the order the
            # next forward pass needs the chunks (embedding, the layers' vectors, the layers, the head); the forward
            # waits chunk by chunk. On one GPU this hides the memory-bound update (30 bytes per parameter) under the
            # compute-bound first layers of the next step; on several it also hides the NVLink-bound pushes.
            self.optimizer.update_stream = self._side
            ids = {n: sp.chunk for n, sp in self.buckets.specs.items()}
            first = [ids[n] for n in ("model.embed_tokens.weight", "model.layers.0.input_layernorm.weight") if n in ids]
            def first_use(c):      # the layer whose forward needs chunk c first (a layer's own experts: that layer)
                layers = [int(sp.name.split(".")[2]) for sp in self.buckets._chunk_specs[c] if sp.name.startswith("model.layers.")]
                return min(layers) if layers else (-1 if any(sp.name.startswith("model.embed") for sp in self.buckets._chunk_specs[c]) else 1 << 30)

            rest = sorted((c for c in range(len(self.buckets.chunks)) if c not in first), key=first_use)
            self.optimizer.update_order = list(dict.fromkeys(first)) + rest
        self.model = NativeCausalLM(model_config, self.buckets, self.device, activation_checkpointing)
        self.loss_name = loss_fn if isinstance(loss_fn, str) else getattr(loss_fn, "__name__", "custom")
        self.loss_fn = LOGPROB_LOSSES[loss_fn] if isinstance(loss_fn, str) else loss_fn
        self.loss_kwargs = loss_kwargs or {}
        self.need_entropy = need_entropy if need_entropy is not None else self.loss_name.startswith("grpo")
        self.checkpoint_dir = Path(checkpoint_dir) if checkpoint_dir else None
        self.weight_version = 0
        self.current_step = 0
        self._poisoned = False
        self._accum = 0
        self._pinned: dict[str, torch.Tensor] = {}
        self.last_h2d_bytes = 0

    # ---------------------------------------------------------------- batch staging
    def _to_device(self, batch: dict[str, Any]) -> dict[str, torch.Tensor]:
        out = {}
        nbytes = 0
        for k, v in batch.items():
            if isinstance(v, (list, tuple)):
                v = torch.tensor(v)
            if not isinstance(v, torch.Tensor):
                continue
            if self.device.type == "cuda" and not v.is_cuda:
                pin = self._pinned.get(k)
                if pin is None or pin.shape != v.shape or pin.dtype != v.dtype:
                    pin = torch.empty(v.shape, dtype=v.dtype).pin_memory()
                    self._pinned[k] = pin
                pin.copy_(v)
                nbytes += pin.numel() * pin.element_size()
                v = pin.to(self.device, non_blocking=True)
            out[k] = v
        self.last_h2d_bytes = nbytes
        return out

    # ---------------------------------------------------------------- protocol
    def forward_backward(self, batch: dict[str, Any]) -> TrainFuture[dict[str, float]]:
        assert not self._poisoned, "backend is poisoned by an earlier failure; rebuild it"
        try:
            return ImmediateTrainFuture(self._forward_backward(batch), "forward_backward")
        except Exception:
            self._poisoned = True
            raise

    def _chunk_grads_final(self, chunk: int) -> None:
        """Autograd hook of the last micro-batch: backward has finished ``chunk``; reduce it beside the rest of backward."""
        if chunk in self._pass_reduced:
            return
        self._pass_reduced.add(chunk)
        ev = torch.cuda.Event()
        ev.record()
        self._side.wait_event(ev)
        with torch.cuda.stream(self._side):
            self.optimizer.reduce_chunk(chunk, 1.0, accumulate=self._accum > 0, overlapped=True)

    def _forward_backward(self, batch: dict[str, Any]) -> dict[str, float]:
        b = self._to_device(batch)
        ids = b["input_ids"]
        labels = b.get("labels", ids)
        mask = b.get("loss_mask")
        if mask is None:
            mask = (labels != -100).float()
            if "attention_mask" in b:
                mask = mask * b["attention_mask"].float()
        targets, shift_mask = shift_labels(labels, mask.float())
        targets = torch.where(shift_mask > 0, targets, torch.full_like(targets, -1))
        B = ids.shape[0]
        n_micro = self.config.get_num_minibatches(B)
        mb = B // n_micro
        agg: dict[str, float] = {}
        t0 = time.perf_counter()
        if self.overlap_comm:
            # every pass reduces its own gradients (summed into the fp32 slices), so each pass is a window of its own
            self.buckets.begin_window()
            self._pass_reduced.clear()
        for i in range(n_micro):
            sl = slice(i * mb, (i + 1) * mb)
            self.model.on_chunk_grads_final = self._chunk_grads_final if (self.overlap_comm and i == n_micro - 1) else None
            lp, ent = self.model.logprobs(ids[sl], targets[sl], self.need_entropy)
            sub = {k: (v[sl] if v.dim() > 0 and v.shape[0] == B else v) for k, v in b.items()}
            sub["shift_mask"] = shift_mask[sl]
            sub["targets"] = targets[sl]
            loss, metrics = self.loss_fn(lp, ent, sub, **self.loss_kwargs)
            assert torch.isfinite(loss).all(), f"non-finite loss: {loss}"
            (loss / n_micro).backward()
            if self.device.type != "cuda":
                self.model.collect_cpu_grads()
            for k, v in metrics.items():
                agg[k] = agg.get(k, 0.0) + float(v) / n_micro
            agg["loss"] = agg.get("loss", 0.0) + (float(loss.detach()) / n_micro if "loss" not in metrics else 0.0)
        self.model.on_chunk_grads_final = None
        if self.overlap_comm:
            # what no hook covered (the embedding, reached last), then the main stream joins the reductions
            ev = torch.cuda.Event()
            ev.record()
            self._side.wait_event(ev)
            with torch.cuda.stream(self._side):
                for c in range(len(self.buckets.chunks)):
                    if c not in self._pass_reduced:
                        self._pass_reduced.add(c)
                        self.optimizer.reduce_chunk(c, 1.0, accumulate=self._accum > 0, overlapped=True)
                done = torch.cuda.Event()
                done.record()
            torch.cuda.current_stream(self.device).wait_event(done)
        self._accum += 1
        agg["fwd_bwd_s"] = time.perf_counter() - t0
        agg["num_tokens"] = float(shift_mask.sum())
        return agg

    def optim_step(self, read_back: bool = True) -> TrainFuture[dict[str, float]]:
        """Clip, AdamW and parameter all-gather. ``read_back=False`` leaves the gradient norm on the device (no
        device-to-host read, so the host runs on into the next step's launches)."""
        assert not self._poisoned, "backend is poisoned by an earlier failure; rebuild it"
        try:
            if self.lr_schedule is not None:
                self.optimizer.lr = self.base_lr * self.lr_schedule(self.current_step)
            norm = self.optimizer.step(grad_scale=1.0 / max(self._accum, 1))
            self._accum = 0
            self.current_step += 1
            self.weight_version += 1
            out = {"lr": self.optimizer.lr, "step": self.current_step}
            if read_back:
                out["grad_norm"] = float(norm)
            return ImmediateTrainFuture(out, "optim_step")
        except Exception:
            self._poisoned = True
            raise

    def get_weights(self) -> TrainFuture[dict[str, Any]]:
        if self.expert_parallel:      # the whole model, the other ranks' experts included
            return ImmediateTrainFuture({n: v.detach().clone() for n, v in self.model.state_dict().items()}, "get_weights")
        return ImmediateTrainFuture({n: self.buckets.full_param(n).detach().clone() for n in self.buckets.specs},
                                    "get_weights")

    def load_weights(self, weights: dict[str, Any]) -> TrainFuture[None]:
        for n in self.buckets.specs:
            self.buckets.set_param(n, weights[n])
        self.optimizer.resync_master()
        self.comm.barrier_host()
        return ImmediateTrainFuture(None, "load_weights")

    # ---------------------------------------------------------------- checkpoints
    def save_checkpoint(self, step: int | None = None, metrics: dict[str, float] | None = None) -> Path:
        """``step_NNNN/``: HF ``model.safetensors`` + ``config.json`` (rank 0), one optimizer shard
        per rank, ``metadata.json`` with step / weight_version / metrics."""
        assert self.checkpoint_dir is not None, "checkpoint_dir not set"
        step = self.current_step if step is None else step
        path = self.checkpoint_dir / f"step_{step:04d}"
        return self.save_checkpoint_to_path(path, step, metrics)

    def save_checkpoint_to_path(self, path: Path | str, step: int | None = None, metrics: dict | None = None) -> Path:
        path = Path(path)
        path.mkdir(parents=True, exist_ok=True)
        if self.expert_parallel:
            gathered = {n: v.detach().cpu() for n, v in self.model.state_dict().items()}           # every rank's experts
        elif self.buckets.any_sharded and self.device.type != "cuda":
            gathered = {n: self.buckets.full_param(n).detach().cpu() for n in self.buckets.specs}   # a collective on CPU groups
        else:
            gathered = None
        if self.rank == 0:
            self.save_hf_checkpoint(path, gathered)
            meta = {"step": self.current_step if step is None else step, "weight_version": self.weight_version,
                    "timestamp": time.time(), "metrics": metrics or {}, "world_size": self.world,
                    "loss": self.loss_name}
            (path / "metadata.json").write_text(json.dumps(meta, indent=2))
        sd = self.optimizer.state_dict()
        flat = {}
        for key in ("master", "exp_avg", "exp_avg_sq"):
            for c, t in enumerate(sd[key]):
                flat[f"{key}.{c}"] = t
        save_safetensors(flat, path / f"optimizer-rank{self.rank:05d}-of-{self.world:05d}.safetensors",
                         {"step": sd["step"], "rank": self.rank, "world": self.world})
        self.comm.barrier_host()
        return path

    def save_hf_checkpoint(self, path: Path | str, weights: dict | None = None) -> Path:
        if weights is None:
            weights = {n: self.buckets.full_param(n).detach().cpu() for n in self.buckets.specs}
        save_safetensors_dir(weights, self.model_config, path, metadata={"weight_version": self.weight_version})
        return Path(path)

    def load_checkpoint(self, path: Path | str) -> dict[str, Any]:
        from ...models.weights import load_safetensors, load_safetensors_dir

        path = Path(path)
        weights, _ = load_safetensors_dir(path)
        weights = {k: v for k, v in weights.items() if k in self.buckets.specs}
        self.load_weights(weights)
        meta = json.loads((path / "metadata.json").read_text()) if (path / "metadata.json").exists() else {}
        shard = path / f"optimizer-rank{self.rank:05d}-of-{self.world:05d}.safetensors"
        if shard.exists():
            flat = load_safetensors(shard, self.device)
            n = len(self.buckets.chunks)
            self.optimizer.load_state_dict({"step": int(meta.get("step", 0)), "rank": self.rank, "world": self.world,
                                            "master": [flat[f"master.{c}"] for c in range(n)],
                                            "exp_avg": [flat[f"exp_avg.{c}"] for c in range(n)],
                                            "exp_avg_sq": [flat[f"exp_avg_sq.{c}"] for c in range(n)]})
        self.current_step = int(meta.get("step", 0))
        self.weight_version = int(meta.get("weight_version", 0))
        return meta

    def get_state_snapshot(self) -> dict[str, Any]:
        return {"step": self.current_step, "weight_version": self.weight_version, "lr": self.optimizer.lr,
                "poisoned": self._poisoned, "world_size": self.world, "rank": self.rank,
                "num_params": self.model_config.num_params(), "loss": self.loss_name,
                "device": str(self.device)}


def warmup_cosine(warmup_steps: int, total_steps: int, min_ratio: float = 0.1) -> Callable[[int], float]:
    """LR multiplier: linear warm-up then cosine decay to ``min_ratio``."""
    def f(step: int) -> float:
        if step < warmup_steps:
            return (step + 1) / max(warmup_steps, 1)
        t = min(1.0, (step - warmup_steps) / max(total_steps - warmup_steps, 1))
        return min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * t))

    return f
