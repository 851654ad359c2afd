"""tcgen05 flash attention (forward and backward) against fp32 PyTorch references."""

import math

import pytest
import torch

from research_b200 import ops
from research_b200.ops import flash

pytestmark = pytest.mark.gpu


def _rand(shape, device, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(device)


def _cu(lens, device):
    return torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=device)


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 14, 2), (128, 8, 2), (128, 4, 4)])
@pytest.mark.parametrize("causal,window", [(True, 0), (True, 100), (False, 0)])
def test_flash_varlen_forward(cuda_device, D, Hq, Hkv, causal, window):
    lens = [1, 127, 128, 129, 300, 517]
    T = sum(lens)
    # q, k, v as views of one fused projection output (row stride > H*D)
    qkv = _rand((T, (Hq + 2 * Hkv) * D), cuda_device, seed=1)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D :].view(T, Hkv, D)
    cu = _cu(lens, cuda_device)
    got, lse = flash.flash_attn_varlen(q, k, v, cu, cu, max(lens), causal=causal, window=window, return_lse=True)
    want, lse_ref = flash.flash_attn_varlen_reference(q, k, v, cu, cu, causal=causal, window=window)
    diff = (got.float() - want.float()).abs()
    assert diff.max().item() < 0.02 and diff.mean().item() < 0.001, (diff.max().item(), diff.mean().item())
    assert torch.allclose(lse, lse_ref, atol=2e-3, rtol=1e-4), (lse - lse_ref).abs().max().item()


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 14, 2), (128, 8, 2)])
def test_flash_cross_lengths(cuda_device, D, Hq, Hkv):
    """More keys than queries: the queries are the last positions (chunked prefill)."""
    q_lens, k_lens = [5, 64, 130, 1], [5, 200, 400, 77]
    q = _rand((sum(q_lens), Hq, D), cuda_device, seed=2)
    k = _rand((sum(k_lens), Hkv, D), cuda_device, seed=3)
    v = _rand((sum(k_lens), Hkv, D), cuda_device, seed=4)
    cu_q, cu_k = _cu(q_lens, cuda_device), _cu(k_lens, cuda_device)
    got = flash.flash_attn_varlen(q, k, v, cu_q, cu_k, max(q_lens))
    want, _ = flash.flash_attn_varlen_reference(q, k, v, cu_q, cu_k)
    diff = (got.float() - want.float()).abs()
    assert diff.max().item() < 0.02 and diff.mean().item() < 0.001, (diff.max().item(), diff.mean().item())


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 14, 2), (128, 32, 8)])
@pytest.mark.parametrize("window", [0, 48])
def test_flash_paged_prefill(cuda_device, D, Hq, Hkv, window):
    new = [5, 64, 65, 130, 1, 200]
    prefix = [0, 16, 3, 100, 40, 0]
    lens = [n + p for n, p in zip(new, prefix)]
    B, bs = len(lens), 16
    nblk = [(l + bs - 1) // bs for l in lens]
    total = sum(nblk) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(5))
    kc = _rand((total, Hkv, bs, D), cuda_device, seed=30)
    vc = _rand((total, Hkv, bs, D), cuda_device, seed=31)
    bt = torch.zeros(B, max(nblk) + 2, dtype=torch.int32)
    o = 0
    for b in range(B):
        bt[b, : nblk[b]] = perm[o : o + nblk[b]].to(torch.int32)
        o += nblk[b]
    bt = bt.to(cuda_device)
    cu = _cu(new, cuda_device)
    q = _rand((sum(new), Hq, D), cuda_device, seed=32)
    sl = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
    got = flash.flash_paged_prefill(q, kc, vc, bt, cu, sl, max(new), window=window)
    want = ops.paged_prefill_reference(q, kc, vc, bt, cu, sl, window=window)
    diff = (got.float() - want.float()).abs()
    assert diff.max().item() < 0.02 and diff.mean().item() < 0.001, (diff.max().item(), diff.mean().item())


def test_flash_large_scores(cuda_device):
    """Scores that grow along the sequence exercise the lazy rescale of the O accumulator."""
    D, H, T = 128, 2, 1024
    q = _rand((T, H, D), cuda_device, seed=7, scale=3.0)
    k = _rand((T, H, D), cuda_device, seed=8, scale=3.0)
    k = (k.float() * torch.linspace(0.2, 3.0, T, device=cuda_device)[:, None, None]).to(torch.bfloat16)
    v = _rand((T, H, D), cuda_device, seed=9)
    cu = _cu([T], cuda_device)
    got, lse = flash.flash_attn_varlen(q, k, v, cu, cu, T, return_lse=True)
    want, lse_ref = flash.flash_attn_varlen_reference(q, k, v, cu, cu)
    diff = (got.float() - want.float()).abs()
    assert diff.max().item() < 0.03 and diff.mean().item() < 0.002, (diff.max().item(), diff.mean().item())
    assert torch.allclose(lse, lse_ref, atol=5e-3, rtol=1e-4)


def _grad_check(got, want, what, tol_max=0.06, tol_rel=0.02):
    diff = (got.float() - want.float()).abs()
    rel = diff.sum().item() / max(want.float().abs().sum().item(), 1e-9)
    assert diff.max().item() < tol_max and rel < tol_rel, (what, diff.max().item(), rel)


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 14, 2), (128, 8, 2), (128, 4, 4)])
@pytest.mark.parametrize("causal,window", [(True, 0), (True, 100), (False, 0)])
def test_flash_varlen_backward(cuda_device, D, Hq, Hkv, causal, window):
    lens = [1, 63, 64, 129, 300, 517]
    T = sum(lens)
    qkv = _rand((T, (Hq + 2 * Hkv) * D), cuda_device, seed=11)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D :].view(T, Hkv, D)
    dout = _rand((T, Hq, D), cuda_device, seed=12)
    cu = _cu(lens, cuda_device)
    out, lse = flash.flash_attn_varlen(q, k, v, cu, cu, max(lens), causal=causal, window=window, return_lse=True)
    dq, dk, dv = flash.flash_attn_varlen_backward(q, k, v, out, dout, lse, cu, cu, max(lens), max(lens), causal, window)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o_ref, _ = flash.flash_attn_varlen_reference(qf, kf, vf, cu, cu, causal=causal, window=window)
    rq, rk, rv = torch.autograd.grad(o_ref, (qf, kf, vf), dout.float())
    _grad_check(dv, rv, "dv")
    _grad_check(dk, rk, "dk")
    _grad_check(dq, rq, "dq")


def test_flash_autograd_cross_lengths(cuda_device):
    D, Hq, Hkv = 128, 8, 2
    q_lens, k_lens = [5, 64, 130], [5, 200, 400]
    q = _rand((sum(q_lens), Hq, D), cuda_device, seed=13).requires_grad_(True)
    k = _rand((sum(k_lens), Hkv, D), cuda_device, seed=14).requires_grad_(True)
    v = _rand((sum(k_lens), Hkv, D), cuda_device, seed=15).requires_grad_(True)
    cu_q, cu_k = _cu(q_lens, cuda_device), _cu(k_lens, cuda_device)
    out = flash.flash_attention(q, k, v, cu_q, cu_k, max(q_lens), max(k_lens))
    w = _rand(out.shape, cuda_device, seed=16)
    (out.float() * w.float()).sum().backward()
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o_ref, _ = flash.flash_attn_varlen_reference(qf, kf, vf, cu_q, cu_k)
    rq, rk, rv = torch.autograd.grad(o_ref, (qf, kf, vf), w.float())
    _grad_check(v.grad, rv, "dv")
    _grad_check(k.grad, rk, "dk")
    _grad_check(q.grad, rq, "dq")


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 4, 2), (64, 4, 1)])
@pytest.mark.parametrize("causal,window", [(True, 0), (True, 300), (False, 0)])
def test_flash_long_sequences_two_tile_kernel(cuda_device, D, Hq, Hkv, causal, window):
    """Lengths around multiples of 256 exercise the two-query-tile kernel: tile b missing, tile b with more key
    tiles than tile a, window starting inside tile a's range."""
    lens = [255, 256, 257, 1000, 1281]
    T = sum(lens)
    q, k, v = _rand((T, Hq, D), cuda_device, seed=21), _rand((T, Hkv, D), cuda_device, seed=22), _rand((T, Hkv, D), cuda_device, seed=23)
    cu = _cu(lens, cuda_device)
    got, lse = flash.flash_attn_varlen(q, k, v, cu, cu, max(lens), causal=causal, window=window, return_lse=True)
    want, lse_ref = flash.flash_attn_varlen_reference(q, k, v, cu, cu, causal=causal, window=window)
    diff = (got.float() - want.float()).abs()
    assert diff.max().item() < 0.02 and diff.mean().item() < 0.001, (diff.max().item(), diff.mean().item())
    assert torch.allclose(lse, lse_ref, atol=2e-3, rtol=1e-4), (lse - lse_ref).abs().max().item()


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 8, 2), (64, 14, 2)])
def test_flash_backward_head_split(cuda_device, monkeypatch, D, Hq, Hkv):
    """dK/dV with one CTA per (key tile, query head) and a reduction over each group: same gradients as the
    per-kv-head form and as the fp32 reference; the automatic rule picks it only where the coarse grid has fewer CTAs than the GPU has SMs."""
    lens = [700, 129, 1]
    T = sum(lens)
    qkv = _rand((T, (Hq + 2 * Hkv) * D), cuda_device, seed=21)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D :].view(T, Hkv, D)
    dout = _rand((T, Hq, D), cuda_device, seed=22)
    cu = _cu(lens, cuda_device)
    out, lse = flash.flash_attn_varlen(q, k, v, cu, cu, max(lens), causal=True, return_lse=True)
    monkeypatch.setattr(flash, "_HEAD_SPLIT", "0")
    base = flash.flash_attn_varlen_backward(q, k, v, out, dout, lse, cu, cu, max(lens), max(lens), True, 0)
    monkeypatch.setattr(flash, "_HEAD_SPLIT", "1")
    split = flash.flash_attn_varlen_backward(q, k, v, out, dout, lse, cu, cu, max(lens), max(lens), True, 0)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o_ref, _ = flash.flash_attn_varlen_reference(qf, kf, vf, cu, cu, causal=True)
    rq, rk, rv = torch.autograd.grad(o_ref, (qf, kf, vf), dout.float())
    for got, want, what in zip(split, (rq, rk, rv), ("dq", "dk", "dv")):
        _grad_check(got, want, what + " (head split)")
    assert torch.equal(split[0], base[0])                       # dQ does not depend on the split
    for a, b in zip(split[1:], base[1:]):                       # fp32 sums over the group vs one accumulator: same to bf16 rounding
        assert (a.float() - b.float()).abs().max().item() < 0.02
    monkeypatch.setattr(flash, "_HEAD_SPLIT", "auto")
    assert flash.head_split_pays(1, 4096, 4096, 16, 2) and not flash.head_split_pays(1, 4096, 4096, 32, 8)
    assert not flash.head_split_pays(32, 512, 512, 14, 2) and not flash.head_split_pays(1, 4096, 4096, 8, 8)
    ops.check_status()
