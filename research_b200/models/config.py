"""Decoder-only model configuration, readable from / writable to a HF ``config.json``.

Families covered (the ones the reference has functional oracles for,
rollouts/tools/functional_extractor/*_functional.py): Qwen2/2.5 (QKV bias, tied embeddings),
Qwen3 (per-head QK RMSNorm, no bias), Llama/SmolLM (no bias, untied head), and sparse
mixture-of-experts variants (Qwen3-MoE softmax-top-k router; GLM-4-MoE sigmoid router with
correction bias, shared expert and leading dense layers).
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field, replace
from pathlib import Path


@dataclass(frozen=True)
class ModelConfig:
    family: str = "qwen2"              # qwen2 | qwen3 | llama | qwen3_moe | glm4_moe
    vocab_size: int = 4096
    hidden_size: int = 256
    num_layers: int = 4
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 704
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e4
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = True
    attention_bias: bool = True        # QKV bias (Qwen2)
    qk_norm: bool = False              # Qwen3
    sliding_window: int = 0
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_type: str = "softmax"       # softmax (top-k then renormalise) | sigmoid (GLM-4)
    n_shared_experts: int = 0
    first_k_dense_replace: int = 0
    routed_scaling_factor: float = 1.0
    n_group: int = 1                   # group-limited routing (sigmoid router): expert groups ...
    topk_group: int = 1                # ... of which this many stay eligible per token
    eos_token_id: int = -1
    init_std: float = 0.02

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def num_params(self) -> int:
        d, L = self.hidden_size, self.num_layers
        attn = d * (self.q_size + 2 * self.kv_size) + self.q_size * d
        if self.attention_bias:
            attn += self.q_size + 2 * self.kv_size
        if self.is_moe:
            mlp = self.num_experts * 3 * d * self.moe_intermediate_size + self.num_experts * d
        else:
            mlp = 3 * d * self.intermediate_size
        emb = self.vocab_size * d * (1 if self.tie_word_embeddings else 2)
        return L * (attn + mlp + 2 * d) + emb + d

    # ---- HF config.json interop -----------------------------------------------------------
    def to_hf_dict(self) -> dict:
        arch = {"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "llama": "LlamaForCausalLM",
                "qwen3_moe": "Qwen3MoeForCausalLM", "glm4_moe": "Glm4MoeForCausalLM"}[self.family]
        d = {
            "architectures": [arch], "model_type": self.family, "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads, "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim, "intermediate_size": self.intermediate_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "attention_bias": self.attention_bias,
            "hidden_act": "silu", "torch_dtype": "bfloat16", "initializer_range": self.init_std,
            "use_sliding_window": self.sliding_window > 0, "sliding_window": self.sliding_window or None,
            "attention_dropout": 0.0, "use_cache": True,
        }
        if self.eos_token_id >= 0:
            d["eos_token_id"] = self.eos_token_id
        if self.is_moe:
            d.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob,
                     n_shared_experts=self.n_shared_experts, first_k_dense_replace=self.first_k_dense_replace,
                     routed_scaling_factor=self.routed_scaling_factor, n_routed_experts=self.num_experts,
                     n_group=self.n_group, topk_group=self.topk_group)
        return d

    @staticmethod
    def from_hf_dict(d: dict) -> "ModelConfig":
        mt = d.get("model_type", "qwen2")
        family = {"qwen2": "qwen2", "qwen3": "qwen3", "llama": "llama", "qwen3_moe": "qwen3_moe",
                  "glm4_moe": "glm4_moe"}.get(mt, "llama")
        heads = d["num_attention_heads"]
        return ModelConfig(
            family=family, vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
            num_layers=d["num_hidden_layers"], num_heads=heads,
            num_kv_heads=d.get("num_key_value_heads", heads),
            head_dim=d.get("head_dim") or d["hidden_size"] // heads,
            intermediate_size=d.get("intermediate_size", 0), rms_norm_eps=d.get("rms_norm_eps", 1e-6),
            rope_theta=d.get("rope_theta", 1e4), max_position_embeddings=d.get("max_position_embeddings", 8192),
            tie_word_embeddings=d.get("tie_word_embeddings", False),
            attention_bias=d.get("attention_bias", family == "qwen2"), qk_norm=family in ("qwen3", "qwen3_moe"),
            sliding_window=(d.get("sliding_window") or 0) if d.get("use_sliding_window") else 0,
            num_experts=d.get("num_experts", d.get("n_routed_experts", 0)) or 0,
            num_experts_per_tok=d.get("num_experts_per_tok", 0) or 0,
            moe_intermediate_size=d.get("moe_intermediate_size", 0) or 0,
            norm_topk_prob=d.get("norm_topk_prob", True),
            router_type="sigmoid" if family == "glm4_moe" else "softmax",
            n_shared_experts=d.get("n_shared_experts", 0) or 0,
            first_k_dense_replace=d.get("first_k_dense_replace", 0) or 0,
            routed_scaling_factor=d.get("routed_scaling_factor", 1.0) or 1.0,
            n_group=d.get("n_group", 1) or 1, topk_group=d.get("topk_group", 1) or 1,
            eos_token_id=d.get("eos_token_id", -1) if isinstance(d.get("eos_token_id", -1), int) else -1,
            init_std=d.get("initializer_range", 0.02),
        )

    def save(self, path: str | Path) -> None:
        Path(path).mkdir(parents=True, exist_ok=True)
        (Path(path) / "config.json").write_text(json.dumps(self.to_hf_dict(), indent=2))

    @staticmethod
    def load(path: str | Path) -> "ModelConfig":
        return ModelConfig.from_hf_dict(json.loads((Path(path) / "config.json").read_text()))

    def as_dict(self) -> dict:
        return asdict(self)


PRESETS: dict[str, ModelConfig] = {
    # tiny CPU plumbing model: Qwen2-style, vocab 4096, 4 layers, d 256, 4q/2kv heads
    "tiny-qwen2": ModelConfig(),
    "tiny-qwen3": ModelConfig(family="qwen3", attention_bias=False, qk_norm=True, tie_word_embeddings=False),
    "tiny-llama": ModelConfig(family="llama", attention_bias=False, tie_word_embeddings=False),
    "tiny-moe": ModelConfig(family="qwen3_moe", attention_bias=False, qk_norm=True, tie_word_embeddings=False,
                            num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128),
    "tiny-glm4-moe": ModelConfig(family="glm4_moe", attention_bias=True, tie_word_embeddings=False, num_experts=8,
                                 num_experts_per_tok=2, moe_intermediate_size=128, router_type="sigmoid",
                                 n_shared_experts=1, first_k_dense_replace=1, routed_scaling_factor=1.5),
    "qwen2.5-0.5b": ModelConfig(family="qwen2", vocab_size=151936, hidden_size=896, num_layers=24, num_heads=14,
                                num_kv_heads=2, head_dim=64, intermediate_size=4864, rope_theta=1e6,
                                max_position_embeddings=32768, tie_word_embeddings=True, attention_bias=True),
    "llama-3-8b": ModelConfig(family="llama", vocab_size=128256, hidden_size=4096, num_layers=32, num_heads=32,
                              num_kv_heads=8, head_dim=128, intermediate_size=14336, rms_norm_eps=1e-5,
                              rope_theta=5e5, max_position_embeddings=8192, tie_word_embeddings=False,
                              attention_bias=False),
    "qwen3-30b-a3b": ModelConfig(family="qwen3_moe", vocab_size=151936, hidden_size=2048, num_layers=48,
                                 num_heads=32, num_kv_heads=4, head_dim=128, intermediate_size=6144,
                                 rope_theta=1e6, max_position_embeddings=40960, tie_word_embeddings=False,
                                 attention_bias=False, qk_norm=True, num_experts=128, num_experts_per_tok=8,
                                 moe_intermediate_size=768, norm_topk_prob=True),
}


def get_preset(name: str, **overrides) -> ModelConfig:
    cfg = PRESETS[name]
    return replace(cfg, **overrides) if overrides else cfg


_ = field  # dataclasses.field kept for subclasses
