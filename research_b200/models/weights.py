"""Random initialisation and HF-safetensors (de)serialisation of model weights.

File format: the Hugging Face checkpoint layout (``config.json`` + ``model.safetensors`` or
sharded ``model-0000i-of-0000n.safetensors`` with ``model.safetensors.index.json``), which is
the interchange format the reference writes with ``save_pretrained``
(rollouts/training/backends/pytorch.py:561-619). The safetensors container is written and
parsed here directly (8-byte header length, JSON header, raw little-endian tensor bytes) so
no extra dependency is needed.
"""

from __future__ import annotations

import json
import struct
import zlib
from collections.abc import Mapping
from pathlib import Path

import numpy as np
import torch

from .config import ModelConfig

_DT = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I64": torch.int64, "I32": torch.int32,
       "U8": torch.uint8, "F64": torch.float64, "BOOL": torch.bool}
_DT_INV = {v: k for k, v in _DT.items()}


def param_shapes(cfg: ModelConfig) -> dict[str, tuple[int, ...]]:
    """HF parameter names and shapes for ``cfg``."""
    d = cfg.hidden_size
    shapes: dict[str, tuple[int, ...]] = {"model.embed_tokens.weight": (cfg.vocab_size, d)}
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        shapes[p + "input_layernorm.weight"] = (d,)
        shapes[p + "post_attention_layernorm.weight"] = (d,)
        a = p + "self_attn."
        shapes[a + "q_proj.weight"] = (cfg.q_size, d)
        shapes[a + "k_proj.weight"] = (cfg.kv_size, d)
        shapes[a + "v_proj.weight"] = (cfg.kv_size, d)
        shapes[a + "o_proj.weight"] = (d, cfg.q_size)
        if cfg.attention_bias:
            shapes[a + "q_proj.bias"] = (cfg.q_size,)
            shapes[a + "k_proj.bias"] = (cfg.kv_size,)
            shapes[a + "v_proj.bias"] = (cfg.kv_size,)
        if cfg.qk_norm:
            shapes[a + "q_norm.weight"] = (cfg.head_dim,)
            shapes[a + "k_norm.weight"] = (cfg.head_dim,)
        m = p + "mlp."
        if cfg.is_moe and i >= cfg.first_k_dense_replace:
            F = cfg.moe_intermediate_size
            shapes[m + "gate.weight"] = (cfg.num_experts, d)
            if cfg.router_type == "sigmoid":
                shapes[m + "gate.e_score_correction_bias"] = (cfg.num_experts,)
            for e in range(cfg.num_experts):
                shapes[f"{m}experts.{e}.gate_proj.weight"] = (F, d)
                shapes[f"{m}experts.{e}.up_proj.weight"] = (F, d)
                shapes[f"{m}experts.{e}.down_proj.weight"] = (d, F)
            if cfg.n_shared_experts > 0:
                Fs = F * cfg.n_shared_experts
                shapes[m + "shared_experts.gate_proj.weight"] = (Fs, d)
                shapes[m + "shared_experts.up_proj.weight"] = (Fs, d)
                shapes[m + "shared_experts.down_proj.weight"] = (d, Fs)
        else:
            F = cfg.intermediate_size
            shapes[m + "gate_proj.weight"] = (F, d)
            shapes[m + "up_proj.weight"] = (F, d)
            shapes[m + "down_proj.weight"] = (d, F)
    shapes["model.norm.weight"] = (d,)
    if not cfg.tie_word_embeddings:
        shapes["lm_head.weight"] = (cfg.vocab_size, d)
    return shapes


def init_random_weights(cfg: ModelConfig, seed: int = 0, dtype=torch.float32, device="cpu") -> dict[str, torch.Tensor]:
    """N(0, init_std) matrices, unit norm weights, zero biases; deterministic in ``seed``."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for name, shape in param_shapes(cfg).items():
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            t = torch.ones(shape, dtype=dtype, device=dev)
        elif name.endswith(".bias"):
            t = torch.zeros(shape, dtype=dtype, device=dev)
        else:
            t = torch.empty(shape, dtype=torch.float32, device=dev).normal_(0.0, cfg.init_std, generator=g).to(dtype)
        out[name] = t
    return out


class LazyRandomWeights(Mapping):
    """Random-init weights materialised one tensor at a time: ``weights[name]`` builds the tensor (deterministic in
    ``(seed, name)``) and keeps no reference, so loading a 30B-parameter model into an engine needs the engine's own
    buffers plus one tensor, not a second full copy. Values differ from ``init_random_weights`` (per-name streams)."""

    def __init__(self, cfg: ModelConfig, seed: int = 0, dtype=torch.float32, device="cpu"):
        self.cfg, self.seed, self.dtype, self.device = cfg, seed, dtype, torch.device(device)
        self.shapes = param_shapes(cfg)

    def __getitem__(self, name: str) -> torch.Tensor:
        shape = self.shapes[name]
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            return torch.ones(shape, dtype=self.dtype, device=self.device)
        if name.endswith(".bias"):
            return torch.zeros(shape, dtype=self.dtype, device=self.device)
        g = torch.Generator(device=self.device).manual_seed((self.seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
        return torch.empty(shape, dtype=torch.float32, device=self.device).normal_(0.0, self.cfg.init_std, generator=g).to(self.dtype)

    def __iter__(self):
        return iter(self.shapes)

    def __len__(self) -> int:
        return len(self.shapes)


# ---------------------------------------------------------------------------- safetensors
def save_safetensors(tensors: dict[str, torch.Tensor], path: str | Path, metadata: dict | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _DT_INV[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = Path(str(path) + ".tmp")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    tmp.replace(path)


def load_safetensors(path: str | Path, device="cpu") -> dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        base = 8 + n
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        s, e = info["data_offsets"]
        dt = _DT[info["dtype"]]
        buf = torch.from_numpy(np.array(mm[base + s : base + e]))
        out[name] = buf.view(dt).reshape(info["shape"]).to(device)
    return out


def save_safetensors_dir(weights: dict[str, torch.Tensor], cfg: ModelConfig, path: str | Path,
                         max_shard_bytes: int = 5 << 30, metadata: dict | None = None) -> None:
    """Write an HF-style checkpoint directory (sharded when large)."""
    path = Path(path)
    cfg.save(path)
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name in sorted(weights):
        nbytes = weights[name].numel() * weights[name].element_size()
        if size + nbytes > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][name] = weights[name]
        size += nbytes
    if len(shards) == 1:
        save_safetensors(shards[0], path / "model.safetensors", {"format": "pt", **(metadata or {})})
        return
    index = {"metadata": {"total_size": sum(w.numel() * w.element_size() for w in weights.values())}, "weight_map": {}}
    for i, shard in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_safetensors(shard, path / fn, {"format": "pt", **(metadata or {})})
        for name in shard:
            index["weight_map"][name] = fn
    (path / "model.safetensors.index.json").write_text(json.dumps(index, indent=2))


def load_safetensors_dir(path: str | Path, device="cpu") -> tuple[dict[str, torch.Tensor], ModelConfig]:
    path = Path(path)
    cfg = ModelConfig.load(path)
    files = sorted(path.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files in {path}")
    weights: dict[str, torch.Tensor] = {}
    for f in files:
        weights.update(load_safetensors(f, device))
    return weights, cfg
