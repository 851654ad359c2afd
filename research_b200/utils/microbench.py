"""Kernel micro-benchmarks with roofline fractions: ``python -m research_b200.utils.microbench``.

Prints one JSON object per kernel/shape: device time (CUDA events, L2 flushed between
iterations), achieved TFLOP/s or GB/s and the fraction of the measured peaks passed with
``--peak-tflops`` / ``--peak-gbs``.
"""

from __future__ import annotations

import argparse
import json

import torch

from .. import ops
from .timing import time_cuda


def bench_gemm(M, N, K, peak_tflops, iters=10, **kw):
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    t = time_cuda(lambda: ops.gemm(a, b, out=out, **kw), iters=iters)
    tl = time_cuda(lambda: torch.matmul(a, b.t(), out=out), iters=iters)
    flops = 2.0 * M * N * K
    byts = 2.0 * (M * K + N * K + M * N)
    ach = flops / (t["median_ms"] * 1e-3) / 1e12
    return {"kernel": "gemm_bf16_tcgen05", "M": M, "N": N, "K": K, **kw, "ms": round(t["median_ms"], 4),
            "tflops": round(ach, 1), "frac_of_measured_peak": round(ach / peak_tflops, 3),
            "gbs": round(byts / (t["median_ms"] * 1e-3) / 1e9, 1),
            "library_matmul_ms": round(tl["median_ms"], 4)}


def bench_decode_attention(B, ctx, Hq, Hkv, D, peak_gbs, iters=10):
    bs = 16
    nblk = (ctx + bs - 1) // bs
    total = B * nblk
    kc = torch.randn(total, Hkv, bs, D, device="cuda").bfloat16()
    vc = torch.randn(total, Hkv, bs, D, device="cuda").bfloat16()
    bt = torch.randperm(total, device="cuda").to(torch.int32).reshape(B, nblk).contiguous()
    sl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    out = torch.empty_like(q)
    splits = ops.decode_num_splits(B, Hkv, ctx, head_dim=D)
    t = time_cuda(lambda: ops.paged_decode(q, kc, vc, bt, sl, num_splits=splits, out=out), iters=iters)
    byts = 2.0 * B * ctx * Hkv * D * 2
    ach = byts / (t["median_ms"] * 1e-3) / 1e9
    return {"kernel": "paged_decode", "B": B, "ctx": ctx, "Hq": Hq, "Hkv": Hkv, "D": D, "splits": splits,
            "ms": round(t["median_ms"], 4), "gbs": round(ach, 1), "frac_of_measured_peak": round(ach / peak_gbs, 3)}


def bench_prefill_attention(B, n, Hq, Hkv, D, peak_tflops, iters=5):
    bs = 16
    nblk = (n + bs - 1) // bs
    kc = torch.randn(B * nblk, Hkv, bs, D, device="cuda").bfloat16()
    vc = torch.randn(B * nblk, Hkv, bs, D, device="cuda").bfloat16()
    bt = torch.arange(B * nblk, device="cuda", dtype=torch.int32).reshape(B, nblk).contiguous()
    cu = (torch.arange(B + 1, device="cuda") * n).to(torch.int32)
    sl = torch.full((B,), n, dtype=torch.int32, device="cuda")
    q = torch.randn(B * n, Hq, D, device="cuda").bfloat16()
    out = torch.empty_like(q)
    t = time_cuda(lambda: ops.paged_prefill(q, kc, vc, bt, cu, sl, n, out=out), iters=iters)
    flops = 4.0 * B * Hq * D * n * n / 2
    ach = flops / (t["median_ms"] * 1e-3) / 1e12
    return {"kernel": "paged_prefill", "B": B, "n": n, "Hq": Hq, "Hkv": Hkv, "D": D, "ms": round(t["median_ms"], 4),
            "tflops": round(ach, 1), "frac_of_measured_peak": round(ach / peak_tflops, 3)}


def bench_flash_forward(B, n, Hq, Hkv, D, peak_tflops, iters=5, paged=False):
    """tcgen05 flash attention forward, causal, B sequences of n tokens (dense or paged K/V)."""
    from ..ops import flash

    q = torch.randn(B * n, Hq, D, device="cuda").bfloat16()
    cu = (torch.arange(B + 1, device="cuda") * n).to(torch.int32)
    out = torch.empty_like(q)
    if paged:
        bs = 16
        nblk = (n + bs - 1) // bs
        kc = torch.randn(B * nblk, Hkv, bs, D, device="cuda").bfloat16()
        vc = torch.randn(B * nblk, Hkv, bs, D, device="cuda").bfloat16()
        bt = torch.arange(B * nblk, device="cuda", dtype=torch.int32).reshape(B, nblk).contiguous()
        sl = torch.full((B,), n, dtype=torch.int32, device="cuda")
        fn = lambda: flash.flash_paged_prefill(q, kc, vc, bt, cu, sl, n, out=out)  # noqa: E731
    else:
        k = torch.randn(B * n, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(B * n, Hkv, D, device="cuda").bfloat16()
        fn = lambda: flash.flash_attn_varlen(q, k, v, cu, cu, n, out=out)  # noqa: E731
    t = time_cuda(fn, iters=iters)
    flops = 4.0 * B * Hq * D * n * n / 2
    ach = flops / (t["median_ms"] * 1e-3) / 1e12
    return {"kernel": "flash_fwd_paged" if paged else "flash_fwd", "B": B, "n": n, "Hq": Hq, "Hkv": Hkv, "D": D,
            "ms": round(t["median_ms"], 4), "tflops": round(ach, 1), "frac_of_measured_peak": round(ach / peak_tflops, 3)}


def bench_flash_backward(B, n, Hq, Hkv, D, peak_tflops, iters=5):
    """tcgen05 flash attention backward (prep + dK/dV + dQ kernels), causal. FLOPs counted as 2.5x forward."""
    from ..ops import flash

    q = torch.randn(B * n, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B * n, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B * n, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B * n, Hq, D, device="cuda").bfloat16()
    cu = (torch.arange(B + 1, device="cuda") * n).to(torch.int32)
    out, lse = flash.flash_attn_varlen(q, k, v, cu, cu, n, return_lse=True)
    t = time_cuda(lambda: flash.flash_attn_varlen_backward(q, k, v, out, do, lse, cu, cu, n, n), iters=iters)
    flops = 2.5 * 4.0 * B * Hq * D * n * n / 2
    ach = flops / (t["median_ms"] * 1e-3) / 1e12
    return {"kernel": "flash_bwd", "B": B, "n": n, "Hq": Hq, "Hkv": Hkv, "D": D, "ms": round(t["median_ms"], 4),
            "tflops": round(ach, 1), "frac_of_measured_peak": round(ach / peak_tflops, 3)}


def bench_nvfp4_gemv(M, K, L, peak_gbs, launches=50):
    """NVFP4 block-scaled GEMV; timed as one CUDA graph of `launches` back-to-back launches so that the
    figure is device time per launch, not host launch overhead."""
    from ..ops import nvfp4

    a = torch.randint(0, 256, (L, M, K // 2), dtype=torch.uint8, device="cuda")
    b = torch.randint(0, 256, (L, K // 2), dtype=torch.uint8, device="cuda")
    sfa = torch.randint(40, 72, (L, M, K // 16), dtype=torch.uint8, device="cuda")
    sfb = torch.randint(40, 72, (L, K // 16), dtype=torch.uint8, device="cuda")
    out = torch.empty(L, M, dtype=torch.float16, device="cuda")
    nvfp4.nvfp4_gemv(a, b, sfa, sfb, out=out)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(launches):
            nvfp4.nvfp4_gemv(a, b, sfa, sfb, out=out)
    t = time_cuda(g.replay, iters=10)
    us = t["median_ms"] * 1e3 / launches
    byts = L * (M * K / 2 + M * K / 16 + K / 2 + K / 16 + 2 * M)
    ach = byts / (us * 1e-6) / 1e9
    return {"kernel": "nvfp4_gemv", "M": M, "K": K, "L": L, "us_per_launch": round(us, 2), "gbs": round(ach, 1),
            "frac_of_measured_peak": round(ach / peak_gbs, 3)}


def bench_rmsnorm(rows, d, peak_gbs):
    x = torch.randn(rows, d, device="cuda").bfloat16()
    w = torch.randn(d, device="cuda").bfloat16()
    out = torch.empty_like(x)
    t = time_cuda(lambda: ops.rmsnorm(x, w, 1e-6, out=out))
    ach = 2.0 * rows * d * 2 / (t["median_ms"] * 1e-3) / 1e9
    return {"kernel": "rmsnorm", "rows": rows, "d": d, "ms": round(t["median_ms"], 4), "gbs": round(ach, 1),
            "frac_of_measured_peak": round(ach / peak_gbs, 3)}


def bench_sampling(B, V, peak_gbs):
    logits = torch.randn(B, V, device="cuda")
    temps = torch.ones(B, device="cuda")
    t = time_cuda(lambda: ops.sample_with_logprobs(logits, temps))
    ach = B * V * 4.0 / (t["median_ms"] * 1e-3) / 1e9
    return {"kernel": "sample_logprob", "B": B, "V": V, "ms": round(t["median_ms"], 4), "gbs": round(ach, 1),
            "frac_of_measured_peak": round(ach / peak_gbs, 3)}


def sweep_decode_gemm(shapes=((256, 896, 4864), (256, 896, 896), (256, 4096, 14336), (256, 4096, 4096), (256, 6144, 4096),
                              (64, 4096, 14336)), launches: int = 60) -> list[dict]:
    """Decode-sized GEMMs (x += a @ W^T) over tile widths and K splits: unsplit, split inside a thread-block cluster
    (``c<S>``) and split through the global workspace (``l2_<S>``). Weights rotate through a ring larger than L2, so
    every launch streams them from HBM. Times are microseconds per launch, back to back on one stream."""
    import itertools

    from research_b200.ops.gemm import _auto_split_k

    dev = torch.device("cuda")
    rows = []
    for M, N, K in shapes:
        nw = max(2, int(400e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device=dev).bfloat16() * 0.05 for _ in range(nw)]
        a = torch.randn(M, K, device=dev).bfloat16()
        x = torch.zeros(M, N, device=dev).bfloat16()
        it = itertools.cycle(range(nw))

        def run(**kw):
            def once():
                ops.gemm(a, ws[next(it)], residual=x, out=x, **kw)

            for _ in range(10):
                once()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(launches):
                once()
            e1.record()
            torch.cuda.synchronize()
            return round(e0.elapsed_time(e1) / launches * 1e3, 1)

        res = {"kernel": "decode_gemm_sweep", "M": M, "N": N, "K": K, "chosen": _auto_split_k(M, N, K, False),
               "auto_us": run(), "unsplit_us": run(split_k=1)}
        for bn in (32, 64, 128, 256):
            if bn > N:
                continue
            res[f"bn{bn}"] = run(split_k=1, bn=bn)
            for s in (2, 4, 8):
                units = -(-M // 128) * -(-N // bn) * s
                if bn // s < 8 or K // 64 < 4 * s or units > 148 - 148 % s:
                    continue
                res[f"bn{bn}_c{s}"] = run(split_k=s, bn=bn, cluster_split=True)
                if bn < 256:
                    res[f"bn{bn}_l2_{s}"] = run(split_k=s, bn=bn, cluster_split=False)
        ops.check_status()
        rows.append(res)
    return rows


# GEMMs of one training step on the Llama-3-8B shape with 4096 tokens: (role, M, N, K, A MN-major, B MN-major)
TRAIN_GEMMS_8B = (
    ("qkv forward", 4096, 6144, 4096, False, False), ("o forward", 4096, 4096, 4096, False, False),
    ("gate|up forward", 4096, 28672, 4096, False, False), ("down forward", 4096, 4096, 14336, False, False),
    ("lm_head forward chunk", 2048, 128256, 4096, False, False),
    ("qkv dgrad", 4096, 4096, 6144, False, True), ("gate|up dgrad", 4096, 4096, 28672, False, True),
    ("down dgrad", 4096, 14336, 4096, False, True), ("lm_head dgrad chunk", 2048, 4096, 128256, False, True),
    ("qkv wgrad", 6144, 4096, 4096, True, True), ("o wgrad", 4096, 4096, 4096, True, True),
    ("gate|up wgrad", 28672, 4096, 4096, True, True), ("down wgrad", 4096, 14336, 4096, True, True),
)


def sweep_train_gemm(peak_tflops: float, iters: int = 10, shapes=TRAIN_GEMMS_8B):
    """Every GEMM of a training step three ways on identical operands: the one-CTA kernel, the two-CTA
    (``cta_group::2``) kernel at both tile widths, and the library (``torch.matmul``). L2 is flushed between launches."""
    from ..ops import gemm_mod as G

    rows = []
    for role, M, N, K, a_mn, b_mn in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        b = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.05).bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        la, lb = (a.t() if a_mn else a), (b if b_mn else b.t())
        flops = 2.0 * M * N * K

        def tf(fn):
            return round(flops / (time_cuda(fn, iters=iters)["median_ms"] * 1e-3) / 1e12, 1)

        saved = G._GEMM2
        G._GEMM2 = False
        one = tf(lambda: ops.gemm(a, b, out=out, a_mn_major=a_mn, b_mn_major=b_mn))
        G._GEMM2 = saved
        p256 = tf(lambda: G.gemm2(a, b, out=out, a_mn_major=a_mn, b_mn_major=b_mn, bn=256))
        p128 = tf(lambda: G.gemm2(a, b, out=out, a_mn_major=a_mn, b_mn_major=b_mn, bn=128))
        auto = tf(lambda: G.gemm2(a, b, out=out, a_mn_major=a_mn, b_mn_major=b_mn))
        lib = tf(lambda: torch.matmul(la, lb, out=out))
        ops.check_status()
        rows.append({"gemm": role, "M": M, "N": N, "K": K, "one_cta_tflops": one, "pair_bn256_tflops": p256,
                     "pair_bn128_tflops": p128, "pair_auto_tflops": auto, "library_tflops": lib,
                     "pair_vs_library": round(auto / lib, 3), "pair_frac_of_measured_peak": round(auto / peak_tflops, 3)})
    return rows


def bench_moe_train(T, k, E, d, F, peak_tflops, iters=5):
    """Forward + backward of one layer's routed experts in training: the grouped launches against a loop over the
    experts with one library GEMM triple each (what a module-per-expert model runs)."""
    from ..ops.moe_train import GroupedExperts, GroupedPlan

    class Sink:
        def accumulate_into(self, view):
            return False

    g = torch.Generator(device="cuda").manual_seed(0)
    h = (torch.randn(T, d, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True)
    wgu = (torch.randn(E * 2 * F, d, device="cuda", generator=g) * 0.02).bfloat16()
    wd = (torch.randn(E * d, F, device="cuda", generator=g) * 0.02).bfloat16()
    ggu, gd = torch.empty_like(wgu), torch.empty_like(wd)
    wt, idx = torch.randn(T, E, device="cuda", generator=g).softmax(-1).topk(k, dim=-1)
    wt = wt.contiguous().requires_grad_(True)
    idx32 = idx.to(torch.int32).contiguous()
    dout = (torch.randn(T, d, device="cuda", generator=g) * 0.1).bfloat16()
    sink = Sink()

    def grouped():
        plan = GroupedPlan(idx32, E, d, F)
        GroupedExperts.apply(h, wt, wgu, ggu, wd, gd, plan, sink).backward(dout)
        h.grad = wt.grad = None

    wl = [(wgu[e * 2 * F:(e + 1) * 2 * F].clone().requires_grad_(True), wd[e * d:(e + 1) * d].clone().requires_grad_(True)) for e in range(E)]

    def loop():
        flat = idx.reshape(-1)
        order = flat.argsort(stable=True)
        counts = torch.bincount(flat, minlength=E).tolist()
        tok = order // k
        xs = h.index_select(0, tok)
        ws = wt.reshape(-1).index_select(0, order).to(h.dtype)
        outs, off = [], 0
        for e, n in enumerate(counts):
            if n:
                gu = xs[off:off + n] @ wl[e][0].t()
                outs.append((torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]) @ wl[e][1].t())
                off += n
        out = torch.zeros_like(h).index_add(0, tok, torch.cat(outs) * ws[:, None])
        out.backward(dout)
        h.grad = wt.grad = None
        for a, b in wl:
            a.grad = b.grad = None

    tg = time_cuda(grouped, iters=iters)
    tl = time_cuda(loop, iters=iters)
    flops = 18.0 * T * k * F * d
    ach = flops / (tg["median_ms"] * 1e-3) / 1e12
    return {"kernel": "moe_grouped_experts_fwd_bwd", "T": T, "k": k, "E": E, "d": d, "F": F, "ms": round(tg["median_ms"], 3),
            "tflops": round(ach, 1), "frac_of_measured_peak": round(ach / peak_tflops, 3),
            "per_expert_library_loop_ms": round(tl["median_ms"], 3), "speedup": round(tl["median_ms"] / tg["median_ms"], 2)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--moe-train", action="store_true", help="only the grouped expert MLP of training (Qwen3-30B-A3B and a small shape)")
    ap.add_argument("--decode-gemm-sweep", action="store_true", help="only the tile-width / split-K sweep of decode GEMMs")
    ap.add_argument("--train-gemm-sweep", action="store_true",
                    help="only the GEMMs of a Llama-3-8B training step: one-CTA kernel, two-CTA kernel, library")
    ap.add_argument("--peak-tflops", type=float, default=1688.4)
    ap.add_argument("--peak-gbs", type=float, default=6453.4)
    ap.add_argument("--quick", action="store_true")
    args = ap.parse_args()
    if args.decode_gemm_sweep:
        for r in sweep_decode_gemm():
            print(json.dumps(r))
        return
    if args.train_gemm_sweep:
        for r in sweep_train_gemm(args.peak_tflops):
            print(json.dumps(r))
        return
    if args.moe_train:
        for shape in ((4096, 8, 128, 2048, 768), (8192, 8, 128, 2048, 768), (4096, 2, 8, 4096, 14336 // 4)):
            print(json.dumps(bench_moe_train(*shape, args.peak_tflops)), flush=True)
        return
    rows = []
    shapes = [(8192, 8192, 8192), (4096, 14336, 4096), (8192, 4096, 14336), (256, 1152, 896), (256, 9728, 896),
              (256, 896, 4864), (256, 151936, 896)]
    if args.quick:
        shapes = shapes[:1] + shapes[3:5]
    for M, N, K in shapes:
        rows.append(bench_gemm(M, N, K, args.peak_tflops))
    for bn in (128, 256):
        rows.append(bench_gemm(8192, 8192, 8192, args.peak_tflops, bn=bn))
    rows.append(bench_decode_attention(256, 832, 14, 2, 64, args.peak_gbs))
    rows.append(bench_decode_attention(64, 2304, 32, 8, 128, args.peak_gbs))
    rows.append(bench_decode_attention(4, 8192, 32, 8, 128, args.peak_gbs))
    rows.append(bench_prefill_attention(8, 2048, 32, 8, 128, args.peak_tflops))
    rows.append(bench_prefill_attention(16, 1024, 14, 2, 64, args.peak_tflops))
    rows.append(bench_flash_forward(8, 2048, 32, 8, 128, args.peak_tflops))
    rows.append(bench_flash_forward(8, 2048, 32, 8, 128, args.peak_tflops, paged=True))
    rows.append(bench_flash_forward(4, 8192, 32, 8, 128, args.peak_tflops))
    rows.append(bench_flash_forward(16, 1024, 14, 2, 64, args.peak_tflops))
    for M, K, L in ((256, 512, 2), (128, 256, 1), (7168, 16384, 1), (4096, 7168, 8), (7168, 2048, 4)):
        rows.append(bench_nvfp4_gemv(M, K, L, args.peak_gbs))
    rows.append(bench_flash_backward(8, 2048, 32, 8, 128, args.peak_tflops))
    rows.append(bench_flash_backward(4, 8192, 32, 8, 128, args.peak_tflops))
    rows.append(bench_rmsnorm(16384, 4096, args.peak_gbs))
    rows.append(bench_sampling(256, 151936, args.peak_gbs))
    for r in rows:
        print(json.dumps(r))


if __name__ == "__main__":
    main()
