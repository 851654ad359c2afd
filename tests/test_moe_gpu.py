"""GPU tests of the MoE path: router kernel, grouped tcgen05 GEMMs with fused combine, engine."""

import pytest
import torch

from research_b200 import ops
from research_b200.inference import EngineConfig, InferenceEngine, SamplingParams
from research_b200.models import causal_lm_forward, get_preset, init_random_weights
from research_b200.models.functional import moe_mlp
from research_b200.parallel.moe import MoELayerWeights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset,E,k,F,d", [("tiny-moe", 8, 2, 128, 256), ("tiny-glm4-moe", 8, 2, 128, 256),
                                            ("tiny-moe", 128, 8, 768, 2048)])
@pytest.mark.parametrize("T", [5, 300])
def test_moe_layer_matches_functional(cuda_device, preset, E, k, F, d, T):
    cfg = get_preset(preset, num_layers=2, num_experts=E, num_experts_per_tok=k, moe_intermediate_size=F, hidden_size=d,
                     init_std=0.05)
    w = {n: v.bfloat16().float() for n, v in init_random_weights(cfg, seed=0).items() if n.startswith("model.layers.1.mlp.")}
    layer = MoELayerWeights(cfg, cuda_device)
    layer.load(w, "model.layers.1.mlp.")
    h = (torch.randn(T, d) * 0.5).bfloat16()
    x0 = torch.randn(T, d).bfloat16()
    x = x0.clone().to(cuda_device)
    layer.forward(h.to(cuda_device), x)
    want = x0.float() + moe_mlp(h.float()[None], w, "model.layers.1.mlp.", cfg)[0]
    err = (x.float().cpu() - want).abs()
    assert err.max().item() < 0.06 + 0.02 * want.abs().max().item(), err.max().item()
    # a second call reuses the scratch and must give the same answer
    x2 = x0.clone().to(cuda_device)
    layer.forward(h.to(cuda_device), x2)
    assert torch.equal(x2, x)


@pytest.mark.parametrize("preset", ["tiny-moe", "tiny-glm4-moe"])
def test_moe_engine_vs_oracle(cuda_device, preset):
    cfg = get_preset(preset, num_layers=2, init_std=0.05)
    w32 = {k: v.bfloat16().float() for k, v in init_random_weights(cfg, seed=0).items()}
    eng = InferenceEngine(EngineConfig(max_batch_size=8, max_model_len=256, num_kv_blocks=128, ignore_eos=True,
                                       graph_batch_sizes=(8,)), cfg, {k: v.bfloat16() for k, v in w32.items()},
                          device=cuda_device)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (20, 33, 47)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    for p, s in zip(prompts, outs):
        ids = list(p) + list(s.completion_tokens)
        lps = torch.log_softmax(causal_lm_forward(torch.tensor([ids]), w32, cfg)[0].float(), -1)
        for j, (tok, lp) in enumerate(zip(s.completion_tokens, s.logprobs)):
            row = lps[len(p) + j - 1]
            assert row[tok].item() >= row.max().item() - 0.3 and abs(row[tok].item() - lp) < 0.08
    eng.shutdown()


@pytest.mark.parametrize("E,n_group,topk_group,k", [(64, 4, 2, 6), (256, 8, 4, 8), (16, 8, 3, 2), (96, 3, 1, 4), (64, 4, 4, 6)])
def test_group_limited_router_kernel(cuda_device, E, n_group, topk_group, k):
    import ctypes

    from research_b200.ops._util import check_rc, stream_handle
    from research_b200.parallel.moe import _lib, route_reference

    g = torch.Generator().manual_seed(E + n_group)
    T = 333
    logits = torch.randn(T, E, generator=g) * 2.0
    bias = torch.randn(E, generator=g) * 0.05
    want_idx, want_w = route_reference(logits, k, True, bias, True, 2.5, n_group, topk_group)
    lg, bs = logits.to(cuda_device), bias.to(cuda_device)
    idx = torch.empty(T, k, dtype=torch.int32, device=cuda_device)
    w = torch.empty(T, k, dtype=torch.float32, device=cuda_device)
    counts = torch.zeros(E, dtype=torch.int32, device=cuda_device)
    check_rc(_lib().rb_moe_route_groups(lg.data_ptr(), bs.data_ptr(), T, E, k, 1, ctypes.c_float(2.5), n_group, topk_group,
                                        idx.data_ptr(), w.data_ptr(), counts.data_ptr(), stream_handle(cuda_device)), "rb_moe_route_groups")
    got_idx, got_w = idx.cpu().long(), w.cpu()
    order_g, order_w = got_idx.argsort(-1), want_idx.long().argsort(-1)
    assert torch.equal(got_idx.gather(-1, order_g), want_idx.long().gather(-1, order_w))
    assert torch.allclose(got_w.gather(-1, order_g), want_w.gather(-1, order_w), rtol=1e-4, atol=1e-6)
    assert torch.equal(counts.cpu().long(), torch.bincount(want_idx.long().reshape(-1), minlength=E))
    if topk_group < n_group:                                     # every chosen expert lies in one of topk_group groups
        groups = got_idx // (E // n_group)
        assert max(len(set(r.tolist())) for r in groups) <= topk_group


def test_moe_layer_with_group_limited_routing(cuda_device):
    cfg = get_preset("tiny-glm4-moe", num_layers=2, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128, hidden_size=256,
                     init_std=0.05, n_group=4, topk_group=2)
    w = {n: v.bfloat16().float() for n, v in init_random_weights(cfg, seed=0).items() if n.startswith("model.layers.1.mlp.")}
    layer = MoELayerWeights(cfg, cuda_device)
    layer.load(w, "model.layers.1.mlp.")
    T = 200
    h = (torch.randn(T, 256) * 0.5).bfloat16()
    x0 = torch.randn(T, 256).bfloat16()
    x = x0.clone().to(cuda_device)
    layer.forward(h.to(cuda_device), x)
    want = x0.float() + moe_mlp(h.float()[None], w, "model.layers.1.mlp.", cfg)[0]
    err = (x.float().cpu() - want).abs()
    assert err.max().item() < 0.06 + 0.02 * want.abs().max().item(), err.max().item()


class _Sink:
    """Stand-in for the gradient bucket: the first write of a view stores, later writes add."""

    def __init__(self):
        self.seen = set()

    def accumulate_into(self, view) -> bool:
        key = view.data_ptr()
        hit = key in self.seen
        self.seen.add(key)
        return hit


@pytest.mark.parametrize("T,k,E,d,F", [(200, 2, 8, 256, 128), (1024, 4, 16, 512, 192), (96, 8, 64, 128, 64)])
def test_grouped_experts_training_vs_reference(cuda_device, T, k, E, d, F):
    """Forward, data gradient, weight gradients and combine-weight gradient of the grouped expert MLP against the fp32
    per-expert loop; a second backward pass must ADD to the weight gradients; experts without tokens get zeros."""
    from research_b200.ops.moe_train import GroupedExperts, GroupedPlan, grouped_experts_reference

    g = torch.Generator().manual_seed(T + E)
    h = (torch.randn(T, d, generator=g) * 0.5).bfloat16().to(cuda_device)
    wgu = (torch.randn(E * 2 * F, d, generator=g) * 0.05).bfloat16().to(cuda_device)
    wd = (torch.randn(E * d, F, generator=g) * 0.05).bfloat16().to(cuda_device)
    logits = torch.randn(T, E, generator=g)
    logits[:, E - 1] = -1e9                       # the last expert never gets a token
    wt, idx = logits.softmax(-1).topk(k, dim=-1)
    wt, idx = wt.to(cuda_device), idx.to(cuda_device)
    dout = (torch.randn(T, d, generator=g) * 0.1).bfloat16().to(cuda_device)

    hr, wtr = h.float().requires_grad_(True), wt.clone().requires_grad_(True)
    wgur, wdr = wgu.float().requires_grad_(True), wd.float().requires_grad_(True)
    ref = grouped_experts_reference(hr, idx, wtr, wgur, wdr)
    ref.backward(dout.float())

    plan = GroupedPlan(idx.to(torch.int32).contiguous(), E, d, F)
    offs = plan.offsets.cpu()
    counts = torch.bincount(idx.reshape(-1).cpu(), minlength=E)
    assert all(int(offs[e + 1] - offs[e]) == max(64, -(-int(counts[e]) // 64) * 64) for e in range(E))
    ggu, gd = torch.full_like(wgu, 7.0), torch.full_like(wd, 7.0)    # must be overwritten, not added to
    sink = _Sink()
    hk, wtk = h.clone().requires_grad_(True), wt.clone().requires_grad_(True)
    out = GroupedExperts.apply(hk, wtk, wgu, ggu, wd, gd, plan, sink)
    out.backward(dout)

    def rel(a, b):
        return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))

    assert rel(out, ref) < 2e-2, rel(out, ref)
    assert rel(hk.grad, hr.grad) < 3e-2, rel(hk.grad, hr.grad)
    assert rel(wtk.grad, wtr.grad) < 3e-2, rel(wtk.grad, wtr.grad)
    assert rel(ggu, wgur.grad) < 3e-2, rel(ggu, wgur.grad)
    assert rel(gd, wdr.grad) < 3e-2, rel(gd, wdr.grad)
    assert float(ggu[(E - 1) * 2 * F:].abs().max()) == 0.0 and float(gd[(E - 1) * d:].abs().max()) == 0.0
    # second pass of the same window: gradients add up
    out2 = GroupedExperts.apply(hk, wtk, wgu, ggu, wd, gd, plan, sink)
    out2.backward(dout)
    assert rel(ggu, 2 * wgur.grad) < 3e-2 and rel(gd, 2 * wdr.grad) < 3e-2
    ops.check_status()
