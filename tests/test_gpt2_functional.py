"""Functional GPT-2 with a functional KV cache against Hugging Face GPT-2 (tiny, random init, CPU)."""

import pytest
import torch

transformers = pytest.importorskip("transformers")

from research_b200.models.gpt2_functional import (GPT2Config, generate, gpt2_forward, init_kv_cache, update_kv_cache)  # noqa: E402


def _tiny():
    torch.manual_seed(0)
    hf_cfg = transformers.GPT2Config(vocab_size=211, n_positions=64, n_embd=48, n_layer=3, n_head=4, attn_implementation="eager")
    model = transformers.GPT2LMHeadModel(hf_cfg).float().eval()
    cfg = GPT2Config(vocab_size=211, n_positions=64, n_embd=48, n_layer=3, n_head=4)
    return model, {k: v.detach() for k, v in model.state_dict().items()}, cfg


def test_forward_matches_hf_and_cache_matches_full_forward():
    model, w, cfg = _tiny()
    ids = torch.randint(0, 211, (2, 17))
    with torch.no_grad():
        ref = model(ids).logits
    full = gpt2_forward(ids, w, cfg)
    assert (full - ref).abs().max() < 2e-4
    # prefill 9 tokens, then 8 single-token steps: the same logits as the uncached forward
    cache = init_kv_cache(cfg, 2, 32)
    logits, cache = gpt2_forward(ids[:, :9], w, cfg, cache)
    assert cache.length == 9 and (logits - full[:, :9]).abs().max() < 2e-4
    for t in range(9, 17):
        step, cache = gpt2_forward(ids[:, t:t + 1], w, cfg, cache)
        assert (step[:, 0] - full[:, t]).abs().max() < 2e-4
    assert cache.length == 17


def test_cache_updates_are_out_of_place():
    cfg = GPT2Config(vocab_size=8, n_positions=8, n_embd=8, n_layer=2, n_head=2)
    c0 = init_kv_cache(cfg, 1, 8)
    k = torch.ones(1, 2, 3, 4)
    c1 = update_kv_cache(c0, 1, k, 2 * k)
    assert float(c0.k.abs().sum()) == 0.0 and float(c1.k[1, :, :, :3].sum()) == 24.0 and float(c1.v[1].sum()) == 48.0
    assert float(c1.k[0].abs().sum()) == 0.0 and c1.length == 0
    with pytest.raises(AssertionError):
        update_kv_cache(c0, 0, torch.ones(1, 2, 9, 4), torch.ones(1, 2, 9, 4))


def test_greedy_generation_matches_hf():
    model, w, cfg = _tiny()
    ids = torch.randint(0, 211, (1, 6))
    with torch.no_grad():
        ref = model.generate(ids, max_new_tokens=10, do_sample=False, pad_token_id=0)
    mine = generate(ids, w, cfg, 10)
    assert torch.equal(mine, ref)
    g = torch.Generator().manual_seed(3)
    sampled = generate(ids, w, cfg, 5, temperature=1.0, generator=g)
    assert sampled.shape == (1, 11) and torch.equal(sampled[:, :6], ids)
