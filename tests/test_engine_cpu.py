"""CPU tests of the engine: C++ scheduler / block manager / radix tree and end-to-end generation
against the functional oracle (greedy exact match, the reference's own correctness criterion)."""

import random

import pytest
import torch

from research_b200.inference import (EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig, Sequence,
                                     SequenceStatus, schedule)
from research_b200.inference.cache import PagedKVCache, RadixKVCache, compute_block_hash
from research_b200.inference.context import (allocate_and_build_context, build_decode_context,
                                             build_prefill_context, extend_and_build_context)
from research_b200.inference.scheduler import can_schedule_any, schedule_native
from research_b200.models import causal_lm_forward, get_preset, init_random_weights


def _seq(i, n, status):
    return Sequence(i, list(range(n)), [], n, status, 1.0, 8, frozenset())


def test_schedule_policy_matches_native():
    rng = random.Random(0)
    for _ in range(200):
        running = [_seq(i, rng.randint(1, 50), SequenceStatus.RUNNING) for i in range(rng.randint(0, 12))]
        waiting = [_seq(100 + i, rng.randint(1, 300), SequenceStatus.WAITING) for i in range(rng.randint(0, 12))]
        cfg = SchedulerConfig(rng.randint(1, 10), rng.randint(10, 600), 16)
        free = rng.randint(0, 40)
        assert schedule(waiting, running, free, cfg) == schedule_native(waiting, running, free, cfg)


def test_schedule_decode_first_and_limits():
    cfg = SchedulerConfig(max_batch_size=3, max_tokens_per_batch=100, block_size=16)
    running = [_seq(i, 5, SequenceStatus.RUNNING) for i in range(4)]
    waiting = [_seq(10, 20, SequenceStatus.WAITING)]
    out = schedule(waiting, running, 100, cfg)
    assert out.decode_seqs == (0, 1, 2) and out.preempted_seqs == (3,) and out.prefill_seqs == ()
    out = schedule([_seq(10, 40, SequenceStatus.WAITING), _seq(11, 70, SequenceStatus.WAITING)], [], 100, cfg)
    assert out.prefill_seqs == (10,)  # token budget stops the second
    out = schedule([_seq(10, 40, SequenceStatus.WAITING)], [], 2, cfg)
    assert out.prefill_seqs == ()  # needs 3 blocks
    assert can_schedule_any([], running, 0, cfg) and not can_schedule_any([], [], 5, cfg)


@pytest.mark.parametrize("cls", [PagedKVCache, RadixKVCache])
def test_prefix_hit_two_prompts(cls):
    cache = cls(num_blocks=32, block_size=4)
    a = list(range(100, 112))
    b = a[:8] + [7, 8, 9, 10, 11]
    blocks_a = cache.allocate(0, a)
    assert len(blocks_a) == 3 and cache.get_cached_tokens(0) == 0
    blocks_b = cache.allocate(1, b)
    assert cache.get_cached_tokens(1) == 8
    assert blocks_b[:2] == blocks_a[:2] and blocks_b[2] != blocks_a[2]
    assert cache.ref_count(blocks_a[0]) >= 2
    cache.deallocate(0)
    cache.deallocate(1)
    assert cache.check_invariants() == 0
    # the prefix survives its sequences
    cache.allocate(2, a[:8] + [1, 2])
    assert cache.get_cached_tokens(2) == 8


def test_fully_cached_prompt_recomputes_last_block():
    cache = PagedKVCache(16, 4)
    p = list(range(8))
    cache.allocate(0, p)
    cache.allocate(1, p)
    assert cache.get_cached_tokens(1) == 4  # never the whole prompt: the step needs logits


@pytest.mark.parametrize("cls", [PagedKVCache, RadixKVCache])
def test_append_token_grows_blocks_and_publishes(cls):
    cache = cls(16, 4)
    cache.allocate(0, [1, 2, 3])
    assert cache.append_token(0, 4) is None
    new = cache.append_token(0, 5)
    assert new is not None and cache.get_block_ids(0)[-1] == new
    for t in (6, 7, 8):
        cache.append_token(0, t)
    cache.deallocate(0)
    cache.allocate(1, [1, 2, 3, 4, 5, 6, 7, 8, 9])
    assert cache.get_cached_tokens(1) == 8  # generated blocks are reusable too


def test_radix_eviction_lru_and_pinning():
    cache = RadixKVCache(num_blocks=8, block_size=4)
    cache.allocate(0, list(range(0, 16)))      # 4 blocks
    cache.deallocate(0)
    cache.allocate(1, list(range(100, 116)))   # 4 blocks
    assert cache.num_free_blocks() == 4        # seq 0's blocks are cached but evictable
    cache.allocate(2, list(range(200, 212)))   # forces eviction of seq 0's leaf
    assert cache.stats()["evictions"] >= 3
    assert cache.check_invariants() == 0
    with pytest.raises(RuntimeError):
        cache.allocate(3, list(range(300, 340)))
    cache.deallocate(1)
    cache.deallocate(2)
    assert cache.check_invariants() == 0
    cache.flush()
    assert cache.num_free_blocks() == 8 and cache.stats()["evictable_blocks"] == 0


def test_radix_split_keeps_pins_consistent():
    cache = RadixKVCache(32, 4)
    long = list(range(24))
    cache.allocate(0, long)
    cache.allocate(1, long[:12] + [90, 91, 92, 93, 94])   # splits seq 0's edge while 0 is pinned
    assert cache.get_cached_tokens(1) == 12
    cache.deallocate(0)
    cache.deallocate(1)
    st = cache.stats()
    assert st["free_blocks"] + st["evictable_blocks"] == 32, st
    assert cache.check_invariants() == 0


def test_allocator_fuzz_invariants():
    rng = random.Random(1)
    for cls in (PagedKVCache, RadixKVCache):
        cache = cls(64, 4)
        live = {}
        for step in range(600):
            if live and rng.random() < 0.45:
                sid = rng.choice(list(live))
                if rng.random() < 0.5:
                    try:
                        cache.append_token(sid, rng.randint(0, 5))
                    except RuntimeError:
                        pass
                else:
                    cache.deallocate(sid)
                    del live[sid]
            else:
                toks = [rng.randint(0, 3) for _ in range(rng.randint(1, 30))]
                try:
                    cache.allocate(step, toks)
                    live[step] = True
                except RuntimeError:
                    pass
            assert cache.check_invariants() == 0
        for sid in list(live):
            cache.deallocate(sid)
        st = cache.stats()
        assert st["free_blocks"] + st["evictable_blocks"] == 64


def test_block_hash_chain():
    h1 = compute_block_hash([1, 2, 3, 4])
    assert h1 == compute_block_hash([1, 2, 3, 4]) and h1 != compute_block_hash([1, 2, 3, 5])
    assert compute_block_hash([5, 6, 7, 8], h1) != compute_block_hash([5, 6, 7, 8])


def test_context_builders():
    cache = PagedKVCache(16, 4)
    ctx, blocks = allocate_and_build_context(cache, 0, [1, 2, 3, 4, 5, 6])
    assert ctx.is_prefill and len(ctx.slot_mapping) == 6
    assert ctx.slot_mapping[0] == blocks[0] * 4 and ctx.slot_mapping[5] == blocks[1] * 4 + 1
    d = extend_and_build_context(cache, 0, 7, 6)
    assert not d.is_prefill and d.seq_lens == (7,) and d.slot_mapping == (blocks[1] * 4 + 2,)
    p = build_prefill_context(cache, [0], [6], [blocks], [4])
    assert p.query_lens == (2,) and len(p.slot_mapping) == 2
    assert build_decode_context(cache, [0], [5], [blocks]).slot_mapping == (blocks[1] * 4,)


# ------------------------------------------------------------------------------ engine end-to-end
def _prompts(cfg, n, seed=0, shared_len=24):
    g = torch.Generator().manual_seed(seed)
    shared = torch.randint(0, cfg.vocab_size, (shared_len,), generator=g).tolist()
    out = []
    for i in range(n):
        k = int(torch.randint(16, 64, (1,), generator=g))
        p = torch.randint(0, cfg.vocab_size, (k,), generator=g).tolist()
        out.append(shared + p if i % 2 == 0 else p)
    return out


def _oracle_greedy(w, cfg, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(causal_lm_forward(torch.tensor([ids]), w, cfg)[0, -1].argmax()))
    return tuple(ids[len(prompt):])


@pytest.mark.parametrize("preset", ["tiny-qwen2", "tiny-qwen3", "tiny-llama", "tiny-moe", "tiny-glm4-moe"])
@pytest.mark.parametrize("cache_type", ["radix", "paged", "none"])
def test_engine_greedy_matches_oracle(preset, cache_type):
    cfg = get_preset(preset, num_layers=2)
    w = init_random_weights(cfg, seed=0)
    eng = InferenceEngine(EngineConfig(cache_type=cache_type, max_batch_size=4, max_model_len=256, num_kv_blocks=96,
                                       ignore_eos=True), cfg, w, device="cpu")
    prompts = _prompts(cfg, 6)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    for p, s in zip(prompts, outs):
        assert s.prompt_tokens == tuple(p)
        assert s.completion_tokens == _oracle_greedy(w, cfg, p, 6)
        assert len(s.logprobs) == 6 and all(lp <= 0 for lp in s.logprobs) and s.finish_reason == "length"
    if cache_type != "none":
        assert eng.cache_stats()["hit_tokens"] > 0
    assert eng.check_invariants() == 0 and not eng.has_pending()


def test_engine_preemption_recomputes_and_finishes():
    cfg = get_preset("tiny-qwen2", num_layers=1)
    w = init_random_weights(cfg, seed=0)
    # pool so small that running sequences must be preempted while they grow
    eng = InferenceEngine(EngineConfig(cache_type="none", max_batch_size=4, max_model_len=128, num_kv_blocks=10,
                                       ignore_eos=True), cfg, w, device="cpu")
    prompts = [p[:30] for p in _prompts(cfg, 4, seed=3)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40))
    for p, s in zip(prompts, outs):
        assert s.completion_tokens == _oracle_greedy(w, cfg, p, 40)
    assert eng.check_invariants() == 0


def test_engine_sampling_seeded_stop_tokens_and_weight_update():
    cfg = get_preset("tiny-qwen2", num_layers=1)
    w = init_random_weights(cfg, seed=0)
    eng = InferenceEngine(EngineConfig(max_batch_size=4, max_model_len=128, num_kv_blocks=64, ignore_eos=True), cfg, w,
                          device="cpu")
    p = _prompts(cfg, 2)
    a = eng.generate(p, SamplingParams(temperature=1.0, max_tokens=5, seed=7))
    b = eng.generate(p, SamplingParams(temperature=1.0, max_tokens=5, seed=7))
    assert [s.completion_tokens for s in a] == [s.completion_tokens for s in b]
    first = a[0].completion_tokens[0]
    c = eng.generate(p[:1], SamplingParams(temperature=1.0, max_tokens=5, seed=7, stop_token_ids=frozenset({first})))
    assert c[0].completion_tokens == (first,) and c[0].finish_reason == "stop"
    # weight update bumps the version and invalidates cached prefixes
    assert eng.cache_stats()["hit_tokens"] > 0
    w2 = init_random_weights(cfg, seed=1)
    eng.update_weights(w2)
    assert eng.get_weight_version() == 1
    d = eng.generate(p[:1], SamplingParams(temperature=0.0, max_tokens=4))
    assert d[0].weight_version == 1 and d[0].cached_tokens == 0
    assert d[0].completion_tokens == _oracle_greedy(w2, cfg, p[0], 4)
    with pytest.raises(ValueError):
        eng.add_request([1] * 100, SamplingParams(max_tokens=100))


def test_folded_rmsnorm_matches_separate_norm(monkeypatch):
    """Norm weights folded into the projections + row statistics inside the GEMM give the same tokens and
    log-probabilities as separate RMSNorm calls (CPU twins of both paths)."""
    import torch

    from research_b200.inference import EngineConfig, InferenceEngine, SamplingParams
    from research_b200.models import get_preset, init_random_weights

    cfg = get_preset("tiny-qwen3", num_layers=2)
    w = init_random_weights(cfg, seed=3)
    for k in list(w):
        if k.endswith("layernorm.weight"):
            w[k] = 1 + 0.3 * torch.randn(w[k].shape, generator=torch.Generator().manual_seed(len(k)))
    ecfg = EngineConfig(max_batch_size=4, max_model_len=64, num_kv_blocks=32, use_cuda_graphs=False, ignore_eos=True)
    prompts = [[5, 6, 7, 8, 9], [11, 12, 13]]
    sp = SamplingParams(temperature=0.0, max_tokens=6)
    folded = InferenceEngine(ecfg, cfg, w, device="cpu")
    assert folded.runner.fold_norm
    a = folded.generate(prompts, sp)
    monkeypatch.setenv("RB_NO_NORM_FOLD", "1")
    plain = InferenceEngine(ecfg, cfg, w, device="cpu")
    assert not plain.runner.fold_norm
    b = plain.generate(prompts, sp)
    for x, y in zip(a, b):
        assert x.completion_tokens == y.completion_tokens
        assert max(abs(p - q) for p, q in zip(x.logprobs, y.logprobs)) < 1e-4
    # a second load must not fold twice
    folded.update_weights(w)
    assert folded.generate(prompts, sp)[0].completion_tokens == a[0].completion_tokens


def test_lazy_random_weights_and_split_chooser():
    import torch

    from research_b200.models import LazyRandomWeights, get_preset
    from research_b200.models.weights import param_shapes
    from research_b200.ops.gemm import _cluster_split_choice

    cfg = get_preset("tiny-moe", num_layers=2)
    lw = LazyRandomWeights(cfg, seed=1)
    assert set(lw) == set(param_shapes(cfg)) and len(lw) == len(param_shapes(cfg))
    n = "model.layers.1.mlp.experts.3.up_proj.weight"
    assert torch.equal(lw[n], lw[n]) and not torch.equal(lw[n], LazyRandomWeights(cfg, seed=2)[n])
    assert float(lw["model.norm.weight"].min()) == 1.0
    for M in (1, 64, 256):
        for N in (128, 896, 1152, 4096, 6144, 28672):
            for K in (768, 896, 2048, 4096, 14336):
                s, bn = _cluster_split_choice(M, N, K)
                if s > 1:
                    units = -(-M // 128) * -(-N // bn) * s
                    per = -(-(-(-K // 64)) // s)
                    assert s in (2, 4, 8) and bn // s >= 8 and units <= 148 - 148 % s and (s - 1) * per < -(-K // 64)
                else:
                    assert bn == 0
    assert _cluster_split_choice(256, 896, 896) == (1, 0) and _cluster_split_choice(256, 896, 4864)[0] > 1


def test_async_batcher_shares_batches():
    """Eight coroutines generating concurrently run in shared engine steps, not one after another."""
    import asyncio

    from research_b200.inference import EngineConfig, InferenceEngine, SamplingParams
    from research_b200.inference.async_engine import batcher_for
    from research_b200.models import get_preset, init_random_weights

    cfg = get_preset("tiny-qwen2", num_layers=2)
    eng = InferenceEngine(EngineConfig(max_batch_size=8, max_model_len=64, num_kv_blocks=64, use_cuda_graphs=False, ignore_eos=True),
                          cfg, init_random_weights(cfg, seed=0), device="cpu")
    sp = SamplingParams(temperature=0.0, max_tokens=6)
    prompts = [[3 + i, 4, 5, 6 + i] for i in range(8)]

    async def go():
        b = batcher_for(eng)
        outs = await asyncio.gather(*[b.generate(p, sp) for p in prompts])
        # a second wave from coroutines that continue after their first result (multi-turn agents)
        more = await asyncio.gather(*[b.generate(p + list(o.completion_tokens), SamplingParams(temperature=0.0, max_tokens=2))
                                      for p, o in zip(prompts[:3], outs[:3])])
        return b, outs, more

    b, outs, more = asyncio.run(go())
    ref = eng.generate(prompts, sp)
    assert [o.completion_tokens for o in outs] == [r.completion_tokens for r in ref]
    assert b.max_rows == 8 and b.steps <= 6 + 2 + 4, (b.max_rows, b.steps)   # ~one step per token, not per request
    assert all(len(m.completion_tokens) == 2 for m in more) and batcher_for(eng) is b


def test_group_limited_routing_oracle_and_config():
    import torch

    from research_b200.models import ModelConfig, get_preset, init_random_weights
    from research_b200.models.functional import causal_lm_forward, group_limited_choice, route
    from research_b200.parallel.moe import route_reference

    g = torch.Generator().manual_seed(0)
    E, ng, tg = 24, 4, 2
    choice = torch.rand(50, E, generator=g)
    got = group_limited_choice(choice, ng, tg)
    for r in range(50):                                                  # an independent restatement, row by row
        gs = [sum(sorted(choice[r, a * 6:(a + 1) * 6].tolist())[-2:]) for a in range(ng)]
        keep = sorted(range(ng), key=lambda a: -gs[a])[:tg]
        for e in range(E):
            assert float(got[r, e]) == (float(choice[r, e]) if e // 6 in keep else 0.0)
    assert group_limited_choice(choice, 1, 1) is choice and group_limited_choice(choice, 4, 4) is choice
    with pytest.raises(AssertionError):
        group_limited_choice(choice, 24, 2)                              # groups of one expert
    cfg = get_preset("tiny-glm4-moe", num_layers=2, num_experts=16, num_experts_per_tok=4, n_group=4, topk_group=2)
    back = ModelConfig.from_hf_dict(cfg.to_hf_dict())
    assert back.n_group == 4 and back.topk_group == 2
    w = init_random_weights(cfg, seed=0)
    x = torch.randn(40, cfg.hidden_size, generator=g)
    idx, wt = route(x, w, "model.layers.1.mlp.", cfg)
    assert max(len(set((row // 4).tolist())) for row in idx) <= 2        # at most two groups per token
    plain = route(x, w, "model.layers.1.mlp.", get_preset("tiny-glm4-moe", num_layers=2, num_experts=16, num_experts_per_tok=4))[0]
    assert not torch.equal(plain.sort(-1).values, idx.sort(-1).values)    # the limit changes some choices
    logits = x @ w["model.layers.1.mlp.gate.weight"].float().t()
    ridx, rw = route_reference(logits, 4, True, w["model.layers.1.mlp.gate.e_score_correction_bias"], cfg.norm_topk_prob,
                               cfg.routed_scaling_factor, 4, 2)
    assert torch.equal(ridx.long().sort(-1).values, idx.sort(-1).values) and torch.allclose(rw.sum(-1), wt.float().sum(-1), atol=1e-5)
    out = causal_lm_forward(torch.randint(0, cfg.vocab_size, (1, 12), generator=g), w, cfg)
    assert torch.isfinite(out).all()
