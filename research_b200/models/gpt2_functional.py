"""GPT-2 as pure functions with a functional KV cache (dev/nano-inference/jax: ``model.py:28-110``,
``layers.py:59-216``, ``kvcache.py:21-116``, ``generate.py``).

The reference writes this experiment in JAX, where arrays are immutable and the cache is a value passed in and
returned; the same style in PyTorch: ``KVCache`` is a frozen record, ``update_kv_cache`` returns a NEW record (the
buffers are written out of place with ``index_copy``), ``gpt2_forward`` takes and returns it. Weights use the Hugging
Face GPT-2 names (``wte.weight``, ``h.0.attn.c_attn.weight`` ... with ``Conv1D`` layout ``[in, out]``), optionally
prefixed by ``transformer.``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch
from torch import Tensor


@dataclass(frozen=True)
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    layer_norm_epsilon: float = 1e-5


@dataclass(frozen=True)
class KVCache:
    """``k`` / ``v``: ``[layers, batch, heads, max_len, head_dim]``; ``length``: tokens cached so far."""

    k: Tensor
    v: Tensor
    length: int = 0


def init_kv_cache(config: GPT2Config, batch: int, max_len: int | None = None, dtype=torch.float32, device="cpu") -> KVCache:
    shape = (config.n_layer, batch, config.n_head, max_len or config.n_positions, config.n_embd // config.n_head)
    return KVCache(torch.zeros(shape, dtype=dtype, device=device), torch.zeros(shape, dtype=dtype, device=device), 0)


def update_kv_cache(cache: KVCache, layer: int, k_new: Tensor, v_new: Tensor) -> KVCache:
    """New cache with ``k_new`` / ``v_new`` ``[B, H, T, D]`` written at positions ``length .. length + T`` of ``layer``;
    the argument is left untouched. ``length`` advances only in ``advance`` (every layer of a step writes the same span)."""
    T = k_new.shape[2]
    assert cache.length + T <= cache.k.shape[3], "KV cache is full"
    pos = torch.arange(cache.length, cache.length + T, device=cache.k.device)
    k = cache.k.clone()
    v = cache.v.clone()
    k[layer] = cache.k[layer].index_copy(2, pos, k_new.to(cache.k.dtype))
    v[layer] = cache.v[layer].index_copy(2, pos, v_new.to(cache.v.dtype))
    return replace(cache, k=k, v=v)


def get_kv_cache(cache: KVCache, layer: int, seq_len: int) -> tuple[Tensor, Tensor]:
    return cache.k[layer, :, :, :seq_len], cache.v[layer, :, :, :seq_len]


def advance(cache: KVCache, n: int) -> KVCache:
    return replace(cache, length=cache.length + n)


# ---------------------------------------------------------------------------------------------- layers
def gelu_new(x: Tensor) -> Tensor:
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x.pow(3))))


def layer_norm(x: Tensor, gamma: Tensor, beta: Tensor, eps: float) -> Tensor:
    mean = x.mean(-1, keepdim=True)
    var = (x - mean).pow(2).mean(-1, keepdim=True)
    return (x - mean) * torch.rsqrt(var + eps) * gamma + beta


def linear(x: Tensor, weight: Tensor, bias: Tensor) -> Tensor:
    """GPT-2's ``Conv1D``: ``weight`` is ``[in, out]``."""
    return x @ weight + bias


def _w(weights: dict[str, Tensor], name: str) -> Tensor:
    return weights[name] if name in weights else weights["transformer." + name]


def multi_head_attention(x: Tensor, weights: dict[str, Tensor], layer: int, config: GPT2Config, cache: KVCache | None):
    B, T, C = x.shape
    H, D = config.n_head, C // config.n_head
    p = f"h.{layer}.attn."
    qkv = linear(x, _w(weights, p + "c_attn.weight"), _w(weights, p + "c_attn.bias"))
    q, k, v = (t.view(B, T, H, D).transpose(1, 2) for t in qkv.split(C, dim=-1))
    past = 0
    if cache is not None:
        past = cache.length
        cache = update_kv_cache(cache, layer, k, v)
        k, v = get_kv_cache(cache, layer, past + T)
    scores = (q @ k.transpose(-1, -2)) / math.sqrt(D)
    qpos = torch.arange(past, past + T, device=x.device)[:, None]
    kpos = torch.arange(past + T, device=x.device)[None, :]
    scores = scores.masked_fill(kpos > qpos, float("-inf"))
    out = (torch.softmax(scores.float(), -1).to(x.dtype) @ v).transpose(1, 2).reshape(B, T, C)
    return linear(out, _w(weights, p + "c_proj.weight"), _w(weights, p + "c_proj.bias")), cache


def mlp_block(x: Tensor, weights: dict[str, Tensor], layer: int) -> Tensor:
    p = f"h.{layer}.mlp."
    return linear(gelu_new(linear(x, _w(weights, p + "c_fc.weight"), _w(weights, p + "c_fc.bias"))),
                  _w(weights, p + "c_proj.weight"), _w(weights, p + "c_proj.bias"))


def transformer_block(x: Tensor, weights: dict[str, Tensor], layer: int, config: GPT2Config, cache: KVCache | None):
    eps = config.layer_norm_epsilon
    a, cache = multi_head_attention(layer_norm(x, _w(weights, f"h.{layer}.ln_1.weight"), _w(weights, f"h.{layer}.ln_1.bias"), eps),
                                    weights, layer, config, cache)
    x = x + a
    x = x + mlp_block(layer_norm(x, _w(weights, f"h.{layer}.ln_2.weight"), _w(weights, f"h.{layer}.ln_2.bias"), eps), weights, layer)
    return x, cache


def gpt2_forward(input_ids: Tensor, weights: dict[str, Tensor], config: GPT2Config, cache: KVCache | None = None):
    """``input_ids [B, T]`` -> logits ``[B, T, V]``; with a cache, ``(logits, new_cache)`` and the tokens are taken to
    follow the ``cache.length`` tokens already cached."""
    B, T = input_ids.shape
    past = cache.length if cache is not None else 0
    pos = torch.arange(past, past + T, device=input_ids.device)
    x = _w(weights, "wte.weight")[input_ids] + _w(weights, "wpe.weight")[pos][None]
    for layer in range(config.n_layer):
        x, cache = transformer_block(x, weights, layer, config, cache)
    x = layer_norm(x, _w(weights, "ln_f.weight"), _w(weights, "ln_f.bias"), config.layer_norm_epsilon)
    logits = x @ _w(weights, "wte.weight").t()
    if cache is None:
        return logits
    return logits, advance(cache, T)


def generate(input_ids: Tensor, weights: dict[str, Tensor], config: GPT2Config, max_new_tokens: int, temperature: float = 0.0,
             generator: torch.Generator | None = None) -> Tensor:
    """Greedy (``temperature == 0``) or sampled continuation: one prefill, then one token per step through the cache."""
    B, T = input_ids.shape
    cache = init_kv_cache(config, B, T + max_new_tokens, _w(weights, "wte.weight").dtype, input_ids.device)
    logits, cache = gpt2_forward(input_ids, weights, config, cache)
    out = [input_ids]
    for _ in range(max_new_tokens):
        last = logits[:, -1].float()
        nxt = last.argmax(-1, keepdim=True) if temperature <= 0 else torch.multinomial(torch.softmax(last / temperature, -1), 1, generator=generator)
        out.append(nxt)
        logits, cache = gpt2_forward(nxt, weights, config, cache)
    return torch.cat(out, dim=1)
