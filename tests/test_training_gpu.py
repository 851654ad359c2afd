"""GPU tests of the training kernels and the kernel-backed trainable model (vs PyTorch fp32)."""

import pytest
import torch

from research_b200 import ops
from research_b200.models import causal_lm_forward, get_preset, init_random_weights
from research_b200.ops import train as T
from research_b200.training import losses as L
from research_b200.training.backends import PyTorchTrainingBackend
from research_b200.training.types import TrainerConfig

pytestmark = pytest.mark.gpu


def test_logprob_entropy_fwd_bwd(cuda_device):
    R, V = 37, 4099
    logits = (torch.randn(R, V, device=cuda_device) * 2).contiguous()
    tg = torch.randint(0, V, (R,), dtype=torch.int32, device=cuda_device)
    tg[3] = -1
    lp, lse, ent = T.logprob_entropy_fwd(logits, tg, True)
    rl, rlse, rent = T.logprob_entropy_reference(logits.cpu(), tg.cpu(), True)
    assert (lp.cpu() - rl).abs().max() < 1e-4 and (lse.cpu() - rlse).abs().max() < 1e-4 and (ent.cpu() - rent).abs().max() < 1e-3
    g_lp, g_ent = torch.randn(R, device=cuda_device), torch.randn(R, device=cuda_device) * 0.1
    d = T.logprob_entropy_bwd(logits, tg, lse, ent, g_lp, g_ent)
    x = logits.cpu().clone().requires_grad_(True)
    a, _, c = T.logprob_entropy_reference(x, tg.cpu(), True)
    ((a * g_lp.cpu()).sum() + (c * g_ent.cpu()).sum()).backward()
    assert (d.float().cpu() - x.grad).abs().max() < 2e-2 * x.grad.abs().max() + 1e-4


def test_rmsnorm_bwd_and_rope(cuda_device):
    x = torch.randn(130, 896, device=cuda_device).bfloat16()
    w = (1 + 0.1 * torch.randn(896, device=cuda_device)).bfloat16()
    dy = torch.randn(130, 896, device=cuda_device).bfloat16()
    dx, dw = T.rmsnorm_bwd(x, w, dy, 1e-6)
    rdx, rdw = T.rmsnorm_bwd(x.cpu(), w.cpu(), dy.cpu(), 1e-6)
    assert (dx.float().cpu() - rdx.float()).abs().max() < 0.05
    assert (dw.cpu() - rdw).abs().max() < 0.02 * rdw.abs().max() + 0.05
    q = torch.randn(50, 4, 64, device=cuda_device).bfloat16()
    pos = torch.randint(0, 300, (50,), dtype=torch.int32, device=cuda_device)
    tab = ops.rope_table(512, 64, 1e4, device=cuda_device)
    y = T.rope(q, pos, tab)
    ry = T.rope(q.cpu(), pos.cpu(), tab.cpu())
    assert (y.float().cpu() - ry.float()).abs().max() < 0.02
    back = T.rope(y, pos, tab, backward=True)  # rotation by -angle undoes it
    assert (back.float() - q.float()).abs().max() < 0.03


@pytest.mark.parametrize("rows,d", [(1000, 64), (77, 256), (300, 512), (2049, 896), (65, 1024), (33, 4096)])
def test_rmsnorm_bwd_widths(cuda_device, rows, d):
    """Register-resident path (d <= 1024) and the generic one against the PyTorch twin."""
    g = torch.Generator().manual_seed(d)
    x = torch.randn(rows, d, generator=g).bfloat16().to(cuda_device)
    w = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16().to(cuda_device)
    dy = torch.randn(rows, d, generator=g).bfloat16().to(cuda_device)
    dx, dw = T.rmsnorm_bwd(x, w, dy, 1e-6)
    rdx, rdw = T.rmsnorm_bwd(x.cpu(), w.cpu(), dy.cpu(), 1e-6)
    assert (dx.float().cpu() - rdx.float()).abs().max() < 0.06
    assert (dw.cpu() - rdw).abs().max() < 0.02 * rdw.abs().max() + 0.05
    ops.check_status()


def test_adamw_kernel_matches_torch(cuda_device):
    n = 10007
    p0 = torch.randn(n)
    ref = p0.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    master = p0.clone().to(cuda_device)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    pb = master.bfloat16()
    for step in range(1, 4):
        g = torch.randn(n)
        ref.grad = g.clone()
        opt.step()
        T.adamw_step(master, m, v, g.to(cuda_device), pb, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
    assert (master.cpu() - ref.detach()).abs().max() < 1e-5
    assert (pb.float().cpu() - ref.detach()).abs().max() < 0.02
    assert abs(float(T.sumsq(master)) - float((master ** 2).sum())) < 1e-2 * float((master ** 2).sum())


@pytest.mark.parametrize("preset,ckpt", [("tiny-qwen2", False), ("tiny-qwen3", True), ("tiny-llama", False)])
def test_native_model_gradients_vs_oracle(cuda_device, preset, ckpt):
    cfg = get_preset(preset, num_layers=2, init_std=0.05)
    w = {k: v.bfloat16().float() for k, v in init_random_weights(cfg, seed=0).items()}
    be = PyTorchTrainingBackend(cfg, w, device=cuda_device, loss_fn="ce", lr=1e-3, activation_checkpointing=ckpt,
                                trainer_config=TrainerConfig(micro_batch_size=2))
    ids = torch.randint(0, cfg.vocab_size, (4, 32))
    m = be.forward_backward({"input_ids": ids, "labels": ids}).wait()
    leaves = {k: v.clone().requires_grad_(True) for k, v in w.items()}
    ref, _ = L.sft_loss(causal_lm_forward(ids, leaves, cfg), {"labels": ids})
    ref.backward()
    assert abs(m["loss"] - float(ref.detach())) < 0.03, (m["loss"], float(ref.detach()))
    for n in ("model.layers.1.mlp.down_proj.weight", "model.layers.0.self_attn.q_proj.weight",
              "model.layers.0.self_attn.k_proj.weight", "model.layers.1.mlp.gate_proj.weight",
              "model.embed_tokens.weight", "model.norm.weight", "model.layers.0.input_layernorm.weight"):
        got, want = be.buckets.grad_view(n).float().cpu(), leaves[n].grad
        rel = (got - want).norm() / (want.norm() + 1e-8)
        assert rel < 0.06, (n, float(rel))
    ops.check_status()


def test_backend_gpu_overfits_and_grpo_step(cuda_device, tmp_path):
    cfg = get_preset("tiny-qwen2", num_layers=2)
    be = PyTorchTrainingBackend(cfg, device=cuda_device, loss_fn="ce", lr=3e-3, checkpoint_dir=tmp_path)
    ids = torch.randint(0, cfg.vocab_size, (4, 48))
    first = last = None
    for _ in range(8):
        m = be.forward_backward({"input_ids": ids, "labels": ids}).wait()
        o = be.optim_step().wait()
        first = first if first is not None else m["loss"]
        last = m["loss"]
    assert last < first - 1.0 and o["grad_norm"] > 0
    be.save_checkpoint()
    assert (tmp_path / "step_0008" / "model.safetensors").exists()
    from research_b200.training.grpo import GRPOConfig, grpo_train

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 4096, (int(n),), generator=g).tolist() for n in torch.randint(20, 60, (8,), generator=g)]
    gcfg = GRPOConfig(model_name="tiny-qwen2", lr=1e-5, batch_size=2, n_samples_per_prompt=4, num_minibatches=2, max_tokens=8,
                      max_seq_len=128, temperature=1.0, num_steps=2, output_dir=str(tmp_path / "rl"), checkpoint_every=0,
                      max_batch_size=8, kv_blocks=128, loss="grpo_clipped")
    hist = grpo_train(gcfg, prompts, lambda s: float(sum(s.tokens[-s.response_length:]) % 2), device=cuda_device)
    assert len(hist) == 2 and hist[-1]["weight_version"] == 2.0 and "clipfrac" in hist[-1]
    ops.check_status()


def test_native_model_matches_oracle_layer_by_layer(cuda_device):
    """The kernel path (tcgen05 GEMMs, flash attention at head size 64) against the fp32 oracle, per layer."""
    from research_b200.models import get_preset
    from research_b200.models.debug import verify_against_oracle
    from research_b200.training.backends.native import NativeTrainingBackend

    cfg = get_preset("tiny-qwen2", num_layers=3, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=512)
    backend = NativeTrainingBackend(cfg, None, device=cuda_device, loss_fn="sft")
    ids = torch.randint(0, cfg.vocab_size, (2, 160), generator=torch.Generator().manual_seed(0))
    rep = verify_against_oracle(backend.model, ids, rel_tol=3e-2)
    assert rep.ok, rep.format()


@pytest.mark.parametrize("preset", ["tiny-moe", "tiny-glm4-moe"])
def test_native_moe_gradients_vs_oracle(cuda_device, preset):
    """Mixture-of-experts training on the kernel path: loss and expert / router gradients against the oracle."""
    cfg = get_preset(preset, num_layers=2, init_std=0.05)
    w = {k: v.bfloat16().float() for k, v in init_random_weights(cfg, seed=0).items()}
    be = PyTorchTrainingBackend(cfg, w, device=cuda_device, loss_fn="ce", lr=1e-3)
    ids = torch.randint(0, cfg.vocab_size, (4, 32), generator=torch.Generator().manual_seed(1))
    m = be.forward_backward({"input_ids": ids, "labels": ids}).wait()
    leaves = {k: v.clone().requires_grad_(True) for k, v in w.items()}
    ref, _ = L.sft_loss(causal_lm_forward(ids, leaves, cfg), {"labels": ids})
    ref.backward()
    assert abs(m["loss"] - float(ref.detach())) < 0.05, (m["loss"], float(ref.detach()))
    moe_layer = max(cfg.first_k_dense_replace, 1)
    used = [e for e in range(cfg.num_experts) if leaves[f"model.layers.{moe_layer}.mlp.experts.{e}.down_proj.weight"].grad.abs().sum() > 0]
    names = [f"model.layers.{moe_layer}.mlp.experts.{used[0]}.down_proj.weight", f"model.layers.{moe_layer}.mlp.experts.{used[-1]}.gate_proj.weight",
             f"model.layers.{moe_layer}.mlp.gate.weight", "model.layers.0.self_attn.q_proj.weight", "model.embed_tokens.weight"]
    if cfg.n_shared_experts > 0:
        names.append(f"model.layers.{moe_layer}.mlp.shared_experts.up_proj.weight")
    for n in names:
        got, want = be.buckets.grad_view(n).float().cpu(), leaves[n].grad
        rel = (got - want).norm() / (want.norm() + 1e-8)
        cos = torch.nn.functional.cosine_similarity(got.reshape(-1), want.reshape(-1), dim=0)
        if ".experts." in n or ".gate.weight" in n:
            # the kernel path routes on bf16 activations: a few near-tie tokens pick another expert than the
            # fp32 oracle, which moves whole rows of an expert's gradient; direction and scale must still agree
            assert cos > 0.93 and rel < 0.4, (n, float(rel), float(cos))
        else:
            assert rel < 0.1, (n, float(rel), float(cos))
    ops.check_status()


def test_small_activation_kernels(cuda_device):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 1024, generator=g).bfloat16().to(cuda_device)
    dy = torch.randn(64, 1024, generator=g).bfloat16().to(cuda_device)
    xf, df = x.float(), dy.float()
    assert torch.allclose(T.relu2(x).float(), torch.relu(xf) ** 2, atol=2e-2, rtol=1e-2)
    assert torch.allclose(T.relu2_backward(x, dy).float(), 2 * torch.relu(xf) * df, atol=3e-2, rtol=1e-2)
    assert torch.allclose(T.softcap(x, 15.0).float(), 15 * torch.tanh(xf / 15), atol=2e-2, rtol=1e-2)
    assert torch.allclose(T.softcap_backward(x, dy, 15.0).float(), (1 - torch.tanh(xf / 15) ** 2) * df, atol=2e-2, rtol=1e-2)
    z = torch.randn(33, 5001, generator=g).to(cuda_device)
    y = T.log_softmax(z)
    assert torch.allclose(y, torch.log_softmax(z, -1), atol=1e-4)
    w = torch.randn(33, 5001, generator=g).to(cuda_device)
    ref = torch.autograd.functional.vjp(lambda t: torch.log_softmax(t, -1), z, w)[1]
    assert torch.allclose(T.log_softmax_backward(y, w), ref, atol=1e-3)


@pytest.mark.parametrize("shape,out", [((2, 3, 17, 23), (5, 7)), ((1, 4, 8, 8), (1, 1)), ((3, 2, 10, 6), (10, 6)), ((2, 2, 5, 9), (7, 4)), ((1, 2, 3, 4), (13, 9))])
def test_adaptive_avg_pool2d_and_vec_add(cuda_device, shape, out):
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(shape, generator=g).to(cuda_device)
    y = T.adaptive_avg_pool2d(x, out)
    ref = torch.nn.functional.adaptive_avg_pool2d(x, out)
    assert torch.allclose(y, ref, atol=1e-5)
    dy = torch.randn(ref.shape, generator=g).to(cuda_device)
    xr = x.clone().requires_grad_(True)
    torch.nn.functional.adaptive_avg_pool2d(xr, out).backward(dy)
    assert torch.allclose(T.adaptive_avg_pool2d_backward(dy, shape[-2:]), xr.grad, atol=1e-5)
    a = torch.randn(1000, 8, generator=g).bfloat16().to(cuda_device)
    b = torch.randn(1000, 8, generator=g).bfloat16().to(cuda_device)
    assert torch.equal(T.vec_add(a, b), a + b)
    ops.check_status()


def test_sharded_adamw_single_gpu_matches_torch(cuda_device):
    """The optimizer path of a one-GPU backend (reduce + clip + fused AdamW with the bf16 write-back) against
    ``torch.optim.AdamW`` on fp32 copies; the fp32 master weights are compared tightly."""
    from research_b200.parallel.fsdp import FlatBuckets, ShardedAdamW
    from research_b200.parallel.symm import LocalComm

    comm = LocalComm(cuda_device)
    shapes = [("layers.0.a", (64, 48)), ("layers.0.b", (48,)), ("layers.1.a", (40, 64)), ("head", (1000, 64))]
    chunk_of = lambda n: 0 if n.startswith("layers.0") else (1 if n.startswith("layers.1") else 2)  # noqa: E731
    b = FlatBuckets(comm, shapes, chunk_of, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(0)
    init = {n: torch.randn(s, generator=g).bfloat16() for n, s in shapes}
    for n, _ in shapes:
        b.param_view(n).copy_(init[n])
    opt = ShardedAdamW(b, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0)
    ref = {n: init[n].float().clone().requires_grad_(True) for n, _ in shapes}
    ropt = torch.optim.AdamW(ref.values(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(4):
        grads = {n: (torch.randn(s, generator=g) * 0.5).bfloat16() for n, s in shapes}
        for n, _ in shapes:
            b.grad_view(n).copy_(grads[n])
            ref[n].grad = grads[n].float()
        norm = opt.step()
        ref_norm = torch.nn.utils.clip_grad_norm_(ref.values(), 1.0)
        ropt.step()
        assert abs(float(norm) - float(ref_norm)) < 1e-3 * float(ref_norm)
        for n, _ in shapes:
            assert (b.param_view(n).float().cpu() - ref[n].detach()).abs().max() < 2e-2, (step, n)
    for n, _ in shapes:                                                 # fp32 master state, parameter by parameter
        sp = b.specs[n]
        lo = sp.offset - b.chunks[sp.chunk][0]
        got = opt.master[sp.chunk][lo:lo + sp.numel].cpu()
        assert (got - ref[n].detach().reshape(-1)).abs().max() < 2e-5, n
    ops.check_status()
