"""GPU tests of the engine: kernel-backed generation against the fp32 functional oracle, using the
reference's own criterion (exact greedy match, else the chosen token must be a near-top token
of the oracle and the reported log-probability must agree)."""

import pytest
import torch

from research_b200.inference import EngineConfig, InferenceEngine, SamplingParams
from research_b200.models import causal_lm_forward, get_preset, init_random_weights

pytestmark = pytest.mark.gpu


def _prompts(cfg, n, seed=0, shared_len=40):
    g = torch.Generator().manual_seed(seed)
    shared = torch.randint(0, cfg.vocab_size, (shared_len,), generator=g).tolist()
    out = []
    for i in range(n):
        k = int(torch.randint(16, 90, (1,), generator=g))
        p = torch.randint(0, cfg.vocab_size, (k,), generator=g).tolist()
        out.append(shared + p if i % 2 == 0 else p)
    return out


def _check_against_oracle(w32, cfg, prompt, sample, lp_tol=0.06, top_gap=0.25):
    ids = list(prompt) + list(sample.completion_tokens)
    logits = causal_lm_forward(torch.tensor([ids]), w32, cfg)[0].float()
    lps = torch.log_softmax(logits, -1)
    for j, (tok, lp) in enumerate(zip(sample.completion_tokens, sample.logprobs)):
        row = lps[len(prompt) + j - 1]
        assert row[tok].item() >= row.max().item() - top_gap, (j, row[tok].item(), row.max().item())
        assert abs(row[tok].item() - lp) < lp_tol, (j, row[tok].item(), lp)


@pytest.mark.parametrize("preset", ["tiny-qwen2", "tiny-qwen3", "tiny-llama"])
@pytest.mark.parametrize("graphs", [False, True])
def test_engine_gpu_greedy_vs_oracle(cuda_device, preset, graphs):
    cfg = get_preset(preset, num_layers=3, init_std=0.05)
    w32 = init_random_weights(cfg, seed=0)
    w32 = {k: v.bfloat16().float() for k, v in w32.items()}  # the oracle sees the same bf16-rounded weights
    eng = InferenceEngine(EngineConfig(max_batch_size=8, max_model_len=512, num_kv_blocks=256, ignore_eos=True,
                                       use_cuda_graphs=graphs, graph_batch_sizes=(2, 4, 8)),
                          cfg, {k: v.bfloat16() for k, v in w32.items()}, device=cuda_device)
    prompts = _prompts(cfg, 10)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for p, s in zip(prompts, outs):
        _check_against_oracle(w32, cfg, p, s)
    assert eng.cache_stats()["hit_tokens"] > 0 and eng.check_invariants() == 0
    eng.shutdown()


def test_engine_gpu_graph_equals_eager_and_seeded(cuda_device):
    cfg = get_preset("tiny-qwen2", num_layers=2, init_std=0.05)
    w = {k: v.bfloat16() for k, v in init_random_weights(cfg, seed=1).items()}
    prompts = _prompts(cfg, 6, seed=2)
    res = []
    for graphs in (False, True):
        eng = InferenceEngine(EngineConfig(max_batch_size=8, max_model_len=512, num_kv_blocks=256, ignore_eos=True,
                                           use_cuda_graphs=graphs, graph_batch_sizes=(8,)), cfg, w, device=cuda_device)
        res.append(eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=16, seed=5)))
        eng.shutdown()
    assert [s.completion_tokens for s in res[0]] == [s.completion_tokens for s in res[1]]
    assert max(abs(a - b) for x, y in zip(res[0], res[1]) for a, b in zip(x.logprobs, y.logprobs)) < 1e-3


def test_runner_score_logits_close_to_oracle(cuda_device):
    cfg = get_preset("tiny-qwen2", num_layers=4, init_std=0.05)
    w32 = {k: v.bfloat16().float() for k, v in init_random_weights(cfg, seed=3).items()}
    eng = InferenceEngine(EngineConfig(max_batch_size=2, max_model_len=256, num_kv_blocks=64, use_cuda_graphs=False),
                          cfg, {k: v.bfloat16() for k, v in w32.items()}, device=cuda_device)
    ids = torch.randint(0, cfg.vocab_size, (150,))
    got = eng.runner.score(ids).cpu()
    want = causal_lm_forward(ids[None], w32, cfg)[0]
    assert (got - want).abs().max().item() < 0.08, (got - want).abs().max().item()
    lp_g, lp_w = torch.log_softmax(got, -1), torch.log_softmax(want, -1)
    assert (lp_g - lp_w).abs().max().item() < 0.08
    eng.shutdown()
