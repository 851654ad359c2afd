"""GPU numerics: every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""

import math

import pytest
import torch

from research_b200 import ops

pytestmark = pytest.mark.gpu


def _rand(shape, device, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(device)


def _assert_close(got, want, atol, rtol, what=""):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{what}: {bad} of {err.numel()} off; max err {err.max().item():.4g}"


# ------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize(
    "M,N,K",
    [(128, 128, 64), (256, 256, 256), (384, 1152, 896), (256, 896, 4864), (1000, 520, 328), (64, 4096, 4096),
     (2048, 2048, 2048)],
)
@pytest.mark.parametrize("bn", [0, 32, 64, 128, 256])
def test_gemm_tn(cuda_device, M, N, K, bn):
    a = _rand((M, K), cuda_device, seed=1)
    b = _rand((N, K), cuda_device, seed=2)
    out = ops.gemm(a, b, bn=bn)
    ref = ops.gemm_reference(a, b, out_dtype=torch.float32)
    _assert_close(out, ref, atol=0.02 * math.sqrt(K), rtol=0.01, what=f"gemm {M}x{N}x{K} bn={bn}")


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (512, 896, 1152), (896, 4864, 512), (136, 264, 200)])
def test_gemm_majorness(cuda_device, a_mn, b_mn, M, N, K):
    a = _rand((K, M) if a_mn else (M, K), cuda_device, seed=3)
    b = _rand((K, N) if b_mn else (N, K), cuda_device, seed=4)
    out = ops.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    ref = ops.gemm_reference(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out_dtype=torch.float32)
    _assert_close(out, ref, atol=0.02 * math.sqrt(K), rtol=0.01, what=f"gemm mn {a_mn}{b_mn}")


def test_gemm_epilogue_bias_residual_f32(cuda_device):
    M, N, K = 300, 1152, 896
    a = _rand((M, K), cuda_device, seed=5)
    b = _rand((N, K), cuda_device, 0.05, seed=6)
    bias = _rand((N,), cuda_device, seed=7)
    res = _rand((M, N), cuda_device, seed=8)
    out = ops.gemm(a, b, bias=bias, residual=res)
    ref = ops.gemm_reference(a, b, bias, res, out_dtype=torch.float32)
    _assert_close(out, ref, atol=0.05, rtol=0.01, what="bias+residual")
    out32 = ops.gemm(a, b, out_f32=True)
    assert out32.dtype == torch.float32
    _assert_close(out32, ops.gemm_reference(a, b, out_dtype=torch.float32), atol=2e-3, rtol=1e-3, what="f32 out")
    # in-place residual (x += proj) as the decoder uses it
    x = res.clone()
    ops.gemm(a, b, residual=x, out=x)
    _assert_close(x, ops.gemm_reference(a, b, None, res, out_dtype=torch.float32), atol=0.05, rtol=0.01, what="inplace")


# two-CTA kernel (tcgen05.mma.cta_group::2, csrc/gemm2_sm100.cu): forward, dgrad and wgrad operand layouts, ragged M / N / K
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (1024, 768, 320), (600, 1000, 512), (256, 2048, 4096), (4096, 1024, 1088)])
@pytest.mark.parametrize("bn", [0, 128, 256])
def test_gemm_pair_kernel(cuda_device, a_mn, b_mn, M, N, K, bn):
    from research_b200.ops.gemm import gemm2

    a = _rand((K, M) if a_mn else (M, K), cuda_device, seed=11)
    b = _rand((K, N) if b_mn else (N, K), cuda_device, seed=12)
    out = gemm2(a, b, a_mn_major=a_mn, b_mn_major=b_mn, bn=bn)
    ref = ops.gemm_reference(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out_dtype=torch.float32)
    _assert_close(out, ref, atol=0.02 * math.sqrt(K), rtol=0.01, what=f"gemm2 {M}x{N}x{K} mn {a_mn}{b_mn} bn={bn}")


def test_gemm_pair_kernel_epilogues_and_dispatch(cuda_device):
    from research_b200.ops.gemm import _use_pair_kernel, gemm2

    M, N, K = 1024, 1152, 896
    a = _rand((M, K), cuda_device, seed=5)
    b = _rand((N, K), cuda_device, 0.05, seed=6)
    bias = _rand((N,), cuda_device, seed=7)
    res = _rand((M, N), cuda_device, seed=8)
    ref = ops.gemm_reference(a, b, bias, res, out_dtype=torch.float32)
    _assert_close(gemm2(a, b, bias=bias, residual=res), ref, atol=0.05, rtol=0.01, what="gemm2 bias+residual")
    out32 = gemm2(a, b, out_f32=True)
    assert out32.dtype == torch.float32
    _assert_close(out32, ops.gemm_reference(a, b, out_dtype=torch.float32), atol=2e-3, rtol=1e-3, what="gemm2 f32 out")
    x = res.clone()                                     # accumulate in place, as the weight-gradient GEMM does
    gemm2(a, b, residual=x, out=x)
    _assert_close(x, ops.gemm_reference(a, b, None, res, out_dtype=torch.float32), atol=0.05, rtol=0.01, what="gemm2 inplace")
    # strided output rows and operand rows (views of wider matrices)
    wide = torch.zeros(M, N + 64, dtype=torch.bfloat16, device=cuda_device)
    gemm2(a, b, out=wide[:, :N])
    _assert_close(wide[:, :N], ops.gemm_reference(a, b, out_dtype=torch.float32), atol=0.02 * math.sqrt(K), rtol=0.01, what="gemm2 ldc")
    assert float(wide[:, N:].abs().sum()) == 0.0
    # the public entry point sends training-sized problems here and keeps decode-sized ones on the one-CTA kernel
    assert _use_pair_kernel(4096, 6144, 4096, False, False) and _use_pair_kernel(28672, 4096, 4096, True, True)
    assert not _use_pair_kernel(256, 28672, 4096, False, False) and not _use_pair_kernel(4096, 4096, 4096, True, False)
    big_a, big_b = _rand((2048, 1024), cuda_device, seed=13), _rand((4736, 1024), cuda_device, 0.05, seed=14)
    _assert_close(ops.gemm(big_a, big_b), ops.gemm_reference(big_a, big_b, out_dtype=torch.float32), atol=0.1, rtol=0.01,
                  what="gemm dispatch to the pair kernel")


@pytest.mark.parametrize("M,F,K,bn", [(256, 4864, 896, 256), (70, 512, 256, 128), (300, 256, 320, 64)])
def test_gemm_fused_swiglu(cuda_device, M, F, K, bn):
    from research_b200.ops.gemm import interleave_gate_up

    x = _rand((M, K), cuda_device, seed=40)
    g = _rand((F, K), cuda_device, 0.05, seed=41)
    u = _rand((F, K), cuda_device, 0.05, seed=42)
    got = ops.gemm(x, interleave_gate_up(g, u, bn), bn=bn, swiglu=True)
    want = ops.swiglu_reference(torch.cat([x.float() @ g.float().t(), x.float() @ u.float().t()], -1).bfloat16())
    assert got.shape == (M, F)
    _assert_close(got, want, atol=0.02, rtol=0.03, what="fused swiglu")
    # programmatic dependent launch must not change results
    ops.set_pdl(True)
    again = ops.gemm(x, interleave_gate_up(g, u, bn), bn=bn, swiglu=True)
    y = ops.rmsnorm(again, _rand((F,), cuda_device, seed=43) * 0 + 1)
    ops.set_pdl(False)
    assert torch.equal(again, got) and torch.isfinite(y.float()).all()


@pytest.mark.parametrize("M,N,K,split", [(256, 896, 4864, 0), (256, 896, 4864, 5), (64, 4096, 14336, 0), (130, 520, 2056, 3)])
def test_gemm_split_k(cuda_device, M, N, K, split):
    a = _rand((M, K), cuda_device, seed=50)
    b = _rand((N, K), cuda_device, 0.05, seed=51)
    bias = _rand((N,), cuda_device, seed=52)
    res = _rand((M, N), cuda_device, seed=53)
    want = ops.gemm_reference(a, b, bias, res, out_dtype=torch.float32)
    got = ops.gemm(a, b, bias=bias, residual=res, split_k=split)
    _assert_close(got, want, atol=0.06, rtol=0.01, what=f"split-k {split}")
    again = ops.gemm(a, b, bias=bias, residual=res, split_k=split)   # tickets reset themselves; sums are deterministic
    assert torch.equal(got, again)
    x = res.clone()
    ops.gemm(a, b, residual=x, out=x, split_k=split)                  # in-place residual as the decoder uses it
    _assert_close(x, ops.gemm_reference(a, b, None, res, out_dtype=torch.float32), atol=0.06, rtol=0.01, what="split-k inplace")


@pytest.mark.parametrize("M,N,K,bn,split,max_ctas", [
    (256, 896, 4864, 64, 4, 0), (256, 896, 4864, 32, 4, 0), (256, 896, 4864, 32, 2, 0), (256, 4096, 14336, 128, 2, 0),
    (130, 520, 2056, 64, 2, 0), (256, 4096, 4096, 128, 8, 0), (384, 1024, 2048, 64, 4, 16), (8, 1152, 896, 32, 2, 0),
    (256, 4096, 14336, 256, 4, 0), (64, 4096, 4096, 256, 8, 0), (256, 6144, 4096, 256, 2, 0), (256, 1024, 2048, 256, 2, 4)])
def test_gemm_cluster_split_k(cuda_device, M, N, K, bn, split, max_ctas):
    """K slices are the CTAs of one thread-block cluster; partial tiles meet in distributed shared memory."""
    a = _rand((M, K), cuda_device, seed=60)
    b = _rand((N, K), cuda_device, 0.05, seed=61)
    bias = _rand((N,), cuda_device, seed=62)
    res = _rand((M, N), cuda_device, seed=63)
    want = ops.gemm_reference(a, b, bias, res, out_dtype=torch.float32)
    got = ops.gemm(a, b, bias=bias, residual=res, bn=bn, split_k=split, cluster_split=True, max_ctas=max_ctas)
    _assert_close(got, want, atol=0.06, rtol=0.01, what=f"cluster split-k bn={bn} s={split}")
    again = ops.gemm(a, b, bias=bias, residual=res, bn=bn, split_k=split, cluster_split=True, max_ctas=max_ctas)
    assert torch.equal(got, again)                                      # fixed slice order: bitwise repeatable
    f32 = ops.gemm(a, b, bn=bn, split_k=split, cluster_split=True, out_f32=True)
    _assert_close(f32, ops.gemm_reference(a, b, out_dtype=torch.float32), atol=0.02, rtol=0.005, what="cluster split-k fp32")
    x = res.clone()
    ops.gemm(a, b, residual=x, out=x, bn=bn, split_k=split, cluster_split=True)   # in-place residual
    _assert_close(x, ops.gemm_reference(a, b, None, res, out_dtype=torch.float32), atol=0.06, rtol=0.01, what="cluster inplace")
    ops.check_status()


@pytest.mark.parametrize("M,N,K,bn,max_ctas", [(256, 1152, 896, 0, 0), (8, 1152, 896, 32, 0), (300, 512, 904, 64, 0), (1000, 1024, 2048, 128, 5),
                                               (256, 6144, 4096, 0, 0)])
def test_gemm_folded_rmsnorm(cuda_device, M, N, K, bn, max_ctas):
    """rstd(row) * (A W'^T) + bias with W' = W * norm weight equals rmsnorm(A) W^T + bias; the row statistics come
    from the A tiles as they pass through shared memory."""
    a = _rand((M, K), cuda_device, 3.0, seed=70)
    w = _rand((N, K), cuda_device, 0.05, seed=71)
    ln = (1 + 0.2 * _rand((K,), cuda_device, seed=72).float()).bfloat16()
    bias = _rand((N,), cuda_device, seed=73)
    af = a.float()
    h = af * torch.rsqrt(af.pow(2).mean(-1, keepdim=True) + 1e-6) * ln.float()
    want = h @ w.float().T + bias.float()
    wf = (w.float() * ln.float()[None, :]).bfloat16()
    got = ops.gemm(a, wf, bias=bias, bn=bn, max_ctas=max_ctas, norm_eps=1e-6)
    _assert_close(got, want, atol=0.08, rtol=0.02, what="folded rmsnorm")
    assert torch.equal(got, ops.gemm(a, wf, bias=bias, bn=bn, max_ctas=max_ctas, norm_eps=1e-6))
    ops.check_status()


def test_gemm_folded_rmsnorm_swiglu(cuda_device):
    from research_b200.ops.gemm import interleave_gate_up

    M, F, K, bn = 256, 1024, 896, 256
    x = _rand((M, K), cuda_device, 2.0, seed=80)
    g = _rand((F, K), cuda_device, 0.05, seed=81)
    u = _rand((F, K), cuda_device, 0.05, seed=82)
    ln = (1 + 0.2 * _rand((K,), cuda_device, seed=83).float()).bfloat16()
    xf = x.float()
    h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * ln.float())
    want = torch.nn.functional.silu(h @ g.float().T) * (h @ u.float().T)
    fold = lambda t: (t.float() * ln.float()[None, :]).bfloat16()
    got = ops.gemm(x, interleave_gate_up(fold(g), fold(u), bn), bn=bn, swiglu=True, norm_eps=1e-6)
    _assert_close(got, want, atol=0.05, rtol=0.03, what="folded rmsnorm + swiglu")
    ops.check_status()


@pytest.mark.parametrize("K,M,N", [(16384, 128, 896), (16384, 896, 896), (4096, 1152, 896), (8192, 256, 520)])
def test_gemm_weight_gradient_shapes_split(cuda_device, K, M, N):
    """Weight-gradient GEMMs of narrow projections (both operands MN-major, few output tiles, K = tokens): the
    chooser cuts K over a cluster; accumulation into the gradient buffer happens in the epilogue."""
    from research_b200.ops.gemm import _auto_split_k

    dy = _rand((K, M), cuda_device, 0.3, seed=90)
    x = _rand((K, N), cuda_device, 0.3, seed=91)
    acc = _rand((M, N), cuda_device, seed=92)
    want = dy.float().T @ x.float() + acc.float()
    got = acc.clone()
    ops.gemm(dy, x, residual=got, out=got, a_mn_major=True, b_mn_major=True)
    rel = (got.float() - want).norm() / want.norm()
    assert rel < 5e-3, float(rel)
    again = acc.clone()
    ops.gemm(dy, x, residual=again, out=again, a_mn_major=True, b_mn_major=True)
    assert torch.equal(got, again)
    if K >= 16384:
        assert _auto_split_k(M, N, K, False, 64)[0] > 1     # these shapes are meant to take the split path
    ops.check_status()


def test_gemm_strided_views(cuda_device):
    big = _rand((256, 2048), cuda_device, seed=9)
    a = big[:, 512:1024]  # lda = 2048
    b = _rand((640, 512), cuda_device, seed=10)
    out = ops.gemm(a, b)
    _assert_close(out, ops.gemm_reference(a, b, out_dtype=torch.float32), atol=0.5, rtol=0.01, what="strided")


# ------------------------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("rows,d", [(7, 64), (300, 896), (33, 4096), (5, 128)])
def test_rmsnorm(cuda_device, rows, d):
    x = _rand((rows, d), cuda_device, 3.0, seed=11)
    w = _rand((d,), cuda_device, seed=12)
    got = ops.rmsnorm(x, w, 1e-6)
    want = ops.rmsnorm_reference(x.cpu(), w.cpu(), 1e-6)
    _assert_close(got.cpu(), want, atol=1e-2, rtol=1e-2, what="rmsnorm")
    # bit-level agreement with the same rounding points on almost every element
    exact = (got.cpu() == want).float().mean().item()
    assert exact > 0.98, exact


@pytest.mark.parametrize("D,Hq,Hkv,qknorm", [(64, 14, 2, False), (128, 32, 8, False), (128, 32, 4, True)])
def test_rope_kv_append(cuda_device, D, Hq, Hkv, qknorm):
    T, nb, bs = 37, 12, 16
    qkv = _rand((T, (Hq + 2 * Hkv) * D), cuda_device, seed=13)
    pos = torch.randint(0, 500, (T,), dtype=torch.int32)
    slots = torch.randperm(nb * bs)[:T].to(torch.int32)
    slots[5] = -1
    table = ops.rope_table(512, D, 1e4)
    qn = _rand((D,), cuda_device, seed=14) if qknorm else None
    kn = _rand((D,), cuda_device, seed=15) if qknorm else None
    kc = torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16, device=cuda_device)
    vc = torch.zeros_like(kc)
    q = ops.rope_kv_append(qkv, pos.to(cuda_device), slots.to(cuda_device), table.to(cuda_device), kc, vc, Hq, Hkv, D, qn, kn)
    kc_ref, vc_ref = torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16), torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16)
    q_ref = ops.rope_kv_append_reference(qkv.cpu(), pos, slots, table, kc_ref, vc_ref, Hq, Hkv, D,
                                         qn.cpu() if qknorm else None, kn.cpu() if qknorm else None)
    _assert_close(q.cpu(), q_ref, atol=2e-2, rtol=2e-2, what="rope q")
    _assert_close(kc.cpu(), kc_ref, atol=2e-2, rtol=2e-2, what="k cache")
    assert torch.equal(vc.cpu(), vc_ref)


def test_swiglu_and_backward(cuda_device):
    gu = _rand((130, 2 * 4864), cuda_device, 2.0, seed=16)
    got = ops.swiglu(gu)
    _assert_close(got.cpu(), ops.swiglu_reference(gu.cpu()), atol=2e-2, rtol=2e-2, what="swiglu")
    dout = _rand((130, 4864), cuda_device, seed=17)
    dgu = ops.swiglu_backward(gu, dout)
    guf = gu.float().cpu().requires_grad_(True)
    g, u = guf.chunk(2, -1)
    (torch.nn.functional.silu(g) * u).backward(dout.float().cpu())
    _assert_close(dgu.cpu(), guf.grad, atol=3e-2, rtol=2e-2, what="swiglu bwd")


def test_embedding_transpose(cuda_device):
    table = _rand((1000, 896), cuda_device, seed=18)
    ids = torch.randint(0, 1000, (77,), dtype=torch.int32, device=cuda_device)
    assert torch.equal(ops.embedding(ids, table), table[ids.long()])
    x = _rand((300, 520), cuda_device, seed=19)
    assert torch.equal(ops.transpose(x), x.t().contiguous())


# ------------------------------------------------------------------------------------ sampling
def test_sampling_greedy_and_logprob(cuda_device):
    B, V = 9, 151936
    logits = torch.randn(B, V, device=cuda_device) * 3
    temps = torch.zeros(B, device=cuda_device)
    tok, lp = ops.sample_with_logprobs(logits, temps)
    ref_lp = torch.log_softmax(logits, -1)
    assert torch.equal(tok.long(), logits.argmax(-1))
    _assert_close(lp, ref_lp.gather(-1, tok.long()[:, None]).squeeze(-1), atol=1e-4, rtol=1e-4, what="greedy lp")
    tl = ops.token_logprobs(logits, tok)
    _assert_close(tl, lp, atol=1e-4, rtol=1e-4, what="token_logprobs")


def test_sampling_distribution_and_seeding(cuda_device):
    V, B = 64, 4096
    base = torch.randn(V, device=cuda_device) * 2
    logits = base[None].repeat(B, 1).contiguous()
    temps = torch.full((B,), 0.7, device=cuda_device)
    seeds = torch.arange(B, dtype=torch.int64, device=cuda_device)
    tok, lp = ops.sample_with_logprobs(logits, temps, seeds, step=3)
    tok2, _ = ops.sample_with_logprobs(logits, temps, seeds, step=3)
    assert torch.equal(tok, tok2), "same seed and step must reproduce"
    tok3, _ = ops.sample_with_logprobs(logits, temps, seeds, step=4)
    assert not torch.equal(tok, tok3)
    # empirical distribution follows softmax(logits / T)
    p = torch.softmax(base / 0.7, -1)
    counts = torch.bincount(tok.long(), minlength=V).float() / B
    assert (counts - p).abs().max().item() < 0.03
    # logprob is of the unscaled logits
    want = torch.log_softmax(base, -1)[tok.long()]
    _assert_close(lp, want, atol=1e-4, rtol=1e-4, what="unscaled logprob")


# ------------------------------------------------------------------------------------ attention
def _make_paged(B, Hkv, D, lens, device, seed):
    bs = 16
    nblk = [(l + bs - 1) // bs for l in lens]
    total = sum(nblk) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed + 7))   # block placement is part of the case
    kc = _rand((total, Hkv, bs, D), device, seed=seed)
    vc = _rand((total, Hkv, bs, D), device, seed=seed + 1)
    max_blocks = max(nblk) + 2
    bt = torch.zeros(B, max_blocks, dtype=torch.int32)
    o = 0
    for b in range(B):
        bt[b, : nblk[b]] = perm[o : o + nblk[b]].to(torch.int32)
        o += nblk[b]
    return kc, vc, bt.to(device)


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 14, 2), (128, 32, 8), (128, 32, 4)])
@pytest.mark.parametrize("splits", [1, 4])
def test_paged_decode(cuda_device, D, Hq, Hkv, splits):
    lens = [1, 15, 16, 17, 100, 333, 1024, 777]
    B = len(lens)
    kc, vc, bt = _make_paged(B, Hkv, D, lens, cuda_device, seed=20)
    q = _rand((B, Hq, D), cuda_device, seed=22)
    sl = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
    got = ops.paged_decode(q, kc, vc, bt, sl, num_splits=splits)
    want = ops.paged_decode_reference(q, kc, vc, bt, sl)
    diff = (got.float() - want.float()).abs()
    assert diff.max().item() < 0.01 and diff.mean().item() < 0.001, (diff.max().item(), diff.mean().item())


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 14, 2), (128, 32, 8)])
@pytest.mark.parametrize("window", [0, 48])
def test_paged_prefill(cuda_device, D, Hq, Hkv, window):
    new = [5, 64, 65, 130, 1, 200]
    prefix = [0, 16, 3, 100, 40, 0]
    lens = [n + p for n, p in zip(new, prefix)]
    B = len(lens)
    kc, vc, bt = _make_paged(B, Hkv, D, lens, cuda_device, seed=30)
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=cuda_device)
    q = _rand((sum(new), Hq, D), cuda_device, seed=32)
    sl = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
    got = ops.paged_prefill(q, kc, vc, bt, cu, sl, max(new), window=window)
    want = ops.paged_prefill_reference(q, kc, vc, bt, cu, sl, window=window)
    diff = (got.float() - want.float()).abs()
    # rows that attend to one or two keys return |v| ~ 2-4, where one bf16 ulp is 0.0156
    assert diff.max().item() < 0.02 and diff.mean().item() < 0.001, (diff.max().item(), diff.mean().item())


# ------------------------------------------------------------------------------------ NVFP4 GEMV
@pytest.mark.parametrize("L,M,K", [(2, 256, 512), (1, 128, 256), (3, 77, 2048), (1, 1024, 7168)])
def test_nvfp4_gemv(cuda_device, L, M, K):
    from research_b200.ops import nvfp4

    g = torch.Generator().manual_seed(5)
    a, sfa = nvfp4.quantize_nvfp4(torch.randn(L, M, K, generator=g))
    b, sfb = nvfp4.quantize_nvfp4(torch.randn(L, K, generator=g))
    want = nvfp4.nvfp4_gemv_reference(a, b, sfa, sfb).float()
    got = nvfp4.nvfp4_gemv(a.to(cuda_device), b.to(cuda_device), sfa.to(cuda_device), sfb.to(cuda_device)).float().cpu()
    # fp16 output: one ulp of the result magnitude
    assert torch.allclose(got, want, rtol=2e-3, atol=2e-3 * want.abs().max().item()), (got - want).abs().max().item()


# ------------------------------------------------------------------------------------ symmetric GEMM / Muon
@pytest.mark.parametrize("M,K", [(256, 512), (136, 72), (1024, 256)])
def test_gemm_symmetric_and_scaled_epilogue(cuda_device, M, K):
    a = _rand((M, K), cuda_device, seed=41) * 0.2
    got = ops.gemm_symmetric(a).float()
    want = a.float() @ a.float().T
    _assert_close(got, want, atol=0.06, rtol=0.02, what="A A^T")
    assert torch.equal(got, got.T), "mirrored store must give an exactly symmetric matrix"
    sym = (want * 0.1).to(torch.bfloat16)
    got2 = ops.gemm_symmetric(sym, alpha=0.5, beta=-1.5, residual=sym).float()
    want2 = 0.5 * sym.float() @ sym.float().T - 1.5 * sym.float()
    _assert_close(got2, want2, atol=0.08, rtol=0.03, what="b A + c A A")
    x = _rand((M, 192), cuda_device, seed=42)
    got3 = ops.gemm(sym, x, residual=x, b_mn_major=True, alpha=1.0, beta=2.5).float()
    _assert_close(got3, sym.float() @ x.float() + 2.5 * x.float(), atol=0.08, rtol=0.03, what="a X + B X")


def test_polar_express_gpu(cuda_device):
    from research_b200.training.muon import polar_express, polar_express_reference

    G = torch.randn(256, 640, generator=torch.Generator().manual_seed(3)).to(cuda_device)
    X = polar_express(G).float()
    ref = polar_express_reference(G)
    assert (X - ref).abs().max().item() < 0.05
    s = torch.linalg.svdvals(X)
    assert s.min().item() > 0.6 and s.max().item() < 1.25


# ------------------------------------------------------------------------------------ FP8 GEMM
@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (130, 264, 80), (4096, 1024, 768)])
@pytest.mark.parametrize("a_dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_gemm_fp8(cuda_device, M, N, K, a_dtype):
    g = torch.Generator().manual_seed(6)
    x = torch.randn(M, K, generator=g).to(cuda_device)
    w = torch.randn(N, K, generator=g).to(cuda_device)
    xq, sx = ops.quantize_fp8(x, a_dtype)
    wq, sw = ops.quantize_fp8(w)
    got = ops.gemm_fp8(xq, wq, scale=sx * sw, out_f32=True)
    want = (xq.float() @ wq.float().T) * (sx * sw)          # exact product of the quantised operands
    _assert_close(got, want, atol=2e-3 * want.abs().max().item(), rtol=1e-3, what="fp8 gemm")
    got16 = ops.gemm_fp8(xq, wq, scale=sx * sw)
    assert got16.dtype == torch.bfloat16 and (got16.float() - want).abs().max().item() < 0.02 * want.abs().max().item()


# ------------------------------------------------------------------------------------ fused lm_head + sampling
@pytest.mark.parametrize("M,V,K", [(256, 151936, 896), (7, 1000, 64), (130, 32000, 256)])
def test_lm_head_sample_matches_two_step(cuda_device, M, V, K):
    h = _rand((M, K), cuda_device, seed=51)
    w = _rand((V, K), cuda_device, seed=52) * 0.2
    temps = torch.ones(M, device=cuda_device)
    temps[::3] = 0.0                                     # greedy rows
    temps[1::3] = 0.7
    seeds = torch.arange(M, device=cuda_device, dtype=torch.int64) * 7919 + 1
    step_t = torch.tensor([5], dtype=torch.int64, device=cuda_device)
    logits = ops.gemm(h, w, out_f32=True)
    tok_ref, lp_ref = ops.sample_with_logprobs(logits, temps, seeds, step=3, step_tensor=step_t)
    tok, lp = ops.lm_head_sample(h, w, temps, seeds, step=3, step_tensor=step_t)
    assert torch.equal(tok, tok_ref), (tok != tok_ref).sum().item()
    assert torch.allclose(lp, lp_ref, atol=2e-4, rtol=1e-4), (lp - lp_ref).abs().max().item()
    greedy = logits.argmax(-1).to(torch.int32)
    assert torch.equal(tok[::3], greedy[::3])
    tok2, _ = ops.lm_head_sample(h, w, temps, seeds, step=4, step_tensor=step_t)
    assert (tok2[1::3] != tok[1::3]).any(), "another step must draw other noise"


# ------------------------------------------------------------------------------------ bounded waits
def test_bounded_flag_wait_runs_out_and_the_device_stays_usable(cuda_device):
    """The failure branch of the cross-GPU flag wait: a wait on a flag that nothing sets, with a budget of one
    millisecond, returns on its own, records its status code for the host, and the next kernel runs normally."""
    import time

    from research_b200.ops._util import KernelStatusError, check_status, status_tensor, stream_handle
    from research_b200.parallel.symm import LocalComm, _lib

    comm = LocalComm(cuda_device)
    slot = comm.new_slot()
    st = status_tensor(cuda_device)
    torch.cuda.synchronize()
    check_status(cuda_device)
    t0 = time.perf_counter()
    rc = _lib().rb_symm_wait_budget(comm.flags.local.data_ptr(), 1, slot, 1, st.data_ptr(), 1_000_000,
                                    stream_handle(cuda_device))
    assert rc == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0, "the wait did not honour its budget"
    with pytest.raises(KernelStatusError, match="flag written by another GPU"):
        check_status(cuda_device)
    # the status word was reset by the failed check; the context is intact
    a, b = _rand((256, 128), cuda_device, seed=1), _rand((192, 128), cuda_device, 0.1, seed=2)
    _assert_close(ops.gemm(a, b), a.float() @ b.float().t(), 0.05, 0.02, "gemm after a timed-out wait")
    # a flag that IS set lets the same wait through
    comm.signal(slot)
    rc = _lib().rb_symm_wait_budget(comm.flags.local.data_ptr(), 1, slot, 1, st.data_ptr(), 1_000_000,
                                    stream_handle(cuda_device))
    assert rc == 0
    torch.cuda.synchronize()
    check_status(cuda_device)


def test_wait_budget_is_a_launch_setting(cuda_device):
    """The library-wide budget of the flag waits can be set and restored from the host."""
    from research_b200.parallel.symm import _lib

    lib = _lib()
    default = lib.rb_comm_get_wait_budget_ns()
    lib.rb_comm_set_wait_budget_ns(5_000_000)
    assert lib.rb_comm_get_wait_budget_ns() == 5_000_000
    lib.rb_comm_set_wait_budget_ns(0)
    assert lib.rb_comm_get_wait_budget_ns() == default


def test_gemm_waits_for_a_flag_inside_the_launch(cuda_device):
    """``wait_flag``: the tile producers compare a device flag with a device value before their first load (the
    tensor-parallel all-reduce uses it to wait for the peers' acknowledgements). Satisfied flag: normal result, on the
    plain and on the cluster split-K path."""
    g = torch.Generator().manual_seed(5)
    flag = torch.tensor([3, 3], dtype=torch.int32, device=cuda_device)      # [0] flag, [1] value it must reach
    for M, N, K in ((64, 1024, 4096), (256, 512, 256)):
        a = torch.randn(M, K, generator=g).bfloat16().to(cuda_device)
        w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(cuda_device)
        out = ops.gemm(a, w, wait_flag=(flag.data_ptr(), flag.data_ptr() + 4))
        want = a.float() @ w.float().t()
        assert (out.float() - want).abs().max().item() < 0.02 * K ** 0.5
    ops.check_status()
