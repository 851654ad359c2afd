"""Small, fixed workloads for Nsight Compute captures: ``python -m research_b200.utils.profile_cases <case>``.

Each case holds well under a few GB on the device, uses inputs larger than the 126 MB L2 where
DRAM figures matter, and launches the kernel of interest a handful of times so a
``--set full`` capture of 1-3 launches ends by itself in a minute or two.
"""

from __future__ import annotations

import sys

import torch

from .. import ops


def case_decode_attn() -> None:
    """paged_decode at the flagship decode shape: 256 sequences x 832 tokens, 14q/2kv heads, D=64."""
    from .microbench import bench_decode_attention

    print(bench_decode_attention(256, 832, 14, 2, 64, 6453.4, iters=3))


def case_decode_attn_d128() -> None:
    from .microbench import bench_decode_attention

    print(bench_decode_attention(64, 2304, 32, 8, 128, 6453.4, iters=3))


def case_gemm_down() -> None:
    """Decode-time down projection of the 0.5B shape: M=256, N=896, K=4864."""
    from .microbench import bench_gemm

    print(bench_gemm(256, 896, 4864, 1688.4, iters=3))


def case_gemm_gateup_8b() -> None:
    """Decode-time gate|up projection of the 8B shape: M=256, N=28672, K=4096 (weights 235 MB, streamed from HBM)."""
    from .microbench import bench_gemm

    print(bench_gemm(256, 28672, 4096, 1688.4, iters=3, bn=256))


def case_gemm_down_8b_cluster() -> None:
    """Decode-time down projection of the 8B shape with split-K over a thread-block cluster: M=256, N=4096, K=14336
    (weights 117 MB per launch, four copies rotated so that every launch streams them from HBM)."""
    import itertools

    ws = [torch.randn(4096, 14336, device="cuda").bfloat16() * 0.05 for _ in range(4)]
    a = torch.randn(256, 14336, device="cuda").bfloat16()
    x = torch.zeros(256, 4096, device="cuda").bfloat16()
    it = itertools.cycle(range(4))
    for _ in range(6):
        ops.gemm(a, ws[next(it)], residual=x, out=x)       # the chooser takes bn 256, 4 slices
    torch.cuda.synchronize()
    ops.check_status()
    print("ok")


def case_gemm_qkv_folded_norm() -> None:
    """qkv projection of the 0.5B shape with the RMSNorm folded in: M=256, N=1152, K=896."""
    a = torch.randn(256, 896, device="cuda").bfloat16()
    w = torch.randn(1152, 896, device="cuda").bfloat16() * 0.05
    b = torch.zeros(1152, device="cuda").bfloat16()
    for _ in range(6):
        ops.gemm(a, w, bias=b, norm_eps=1e-6)
    torch.cuda.synchronize()
    ops.check_status()
    print("ok")


def case_gemm_large() -> None:
    from .microbench import bench_gemm

    print(bench_gemm(4096, 14336, 4096, 1688.4, iters=3))


def case_flash_fwd() -> None:
    """tcgen05 flash attention forward: 8 x 2048 tokens, 32q/8kv heads, D=128, causal."""
    from .microbench import bench_flash_forward

    print(bench_flash_forward(8, 2048, 32, 8, 128, 1688.4, iters=3))


def case_flash_fwd_short() -> None:
    """Flash attention forward at training-rollout lengths: 32 x 512 tokens, 14q/2kv heads, D=64, causal."""
    from .microbench import bench_flash_forward

    print(bench_flash_forward(32, 512, 14, 2, 64, 1688.4, iters=3))


def case_flash_bwd() -> None:
    """tcgen05 flash attention backward: 8 x 2048 tokens, 32q/8kv heads, D=128, causal."""
    from .microbench import bench_flash_backward

    print(bench_flash_backward(8, 2048, 32, 8, 128, 1688.4, iters=3))


def case_decode_step() -> None:
    """Two eager decode steps at batch 256 (for a per-launch time list); the model preset comes from
    RB_PROFILE_MODEL (default: the 0.5B flagship shape), optionally cut to RB_PROFILE_LAYERS layers."""
    from ..inference import EngineConfig, InferenceEngine, SamplingParams
    from ..models import get_preset, init_random_weights

    import os

    over = {"num_layers": int(os.environ["RB_PROFILE_LAYERS"])} if os.environ.get("RB_PROFILE_LAYERS") else {}
    cfg = get_preset(os.environ.get("RB_PROFILE_MODEL", "qwen2.5-0.5b"), **over)   # fewer layers keep big models small
    dev = torch.device("cuda:0")
    w = init_random_weights(cfg, seed=0, dtype=torch.bfloat16, device=dev)
    eng = InferenceEngine(EngineConfig(max_batch_size=256, max_model_len=2048, num_kv_blocks=20000, ignore_eos=True,
                                       use_cuda_graphs=False, max_tokens_per_batch=16384), cfg, w, device=dev)
    g = torch.Generator().manual_seed(0)
    for i in range(256):
        n = int(torch.randint(600, 1000, (1,), generator=g))
        eng.add_request(torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(), SamplingParams(1.0, 64, seed=i))
    while eng.last_step_rows != (0, 256):
        eng.step()
    torch.cuda.synchronize()
    ops.set_pdl(False)
    # with `ncu --profile-from-start off` only the launches between start() and stop() are captured
    torch.cuda.profiler.start()
    for _ in range(2):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print("ok")


def case_gemm_pair() -> None:
    """Two-CTA (``cta_group::2``) GEMM at a training shape: the o projection forward, 4096 x 4096 x 4096, and the gate|up
    projection forward, 4096 x 28672 x 4096 (weights 235 MB: streamed from HBM)."""
    from ..ops.gemm import gemm2

    a = torch.randn(4096, 4096, device="cuda").bfloat16()
    wo = torch.randn(4096, 4096, device="cuda").bfloat16() * 0.05
    wgu = torch.randn(28672, 4096, device="cuda").bfloat16() * 0.05
    out_o = torch.empty(4096, 4096, device="cuda", dtype=torch.bfloat16)
    out_gu = torch.empty(4096, 28672, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        gemm2(a, wo, out=out_o)
        gemm2(a, wgu, out=out_gu)
    torch.cuda.synchronize()
    ops.check_status()
    print("ok")


def _optimizer_case(n_params: int):
    """One rank's sharded-optimizer state over ``n_params`` parameters in three chunks (this GPU is its only peer)."""
    from ..parallel.fsdp import FlatBuckets, ShardedAdamW
    from ..parallel.symm import LocalComm

    dev = torch.device("cuda", torch.cuda.current_device())
    comm = LocalComm(dev)
    rows = n_params // 3 // 4096
    shapes = [(f"w{i}", (rows, 4096)) for i in range(3)]
    fb = FlatBuckets(comm, shapes, lambda n: int(n[1:]))
    fb.params.normal_(0, 0.02)
    fb.grads.normal_(0, 0.01)
    return fb, ShardedAdamW(fb, lr=1e-5, max_grad_norm=1.0)


def case_rs_reduce() -> None:
    """Gradient reduce kernel on one GPU: 96 Mi bf16 gradients (192 MB, larger than L2) in three chunks; with one rank
    the launch reads the bucket once and produces the sum of squares (the norm pass of a single-GPU step)."""
    fb, opt = _optimizer_case(96 * 1024 * 1024)
    for _ in range(3):
        for c in range(3):
            opt.reduce_chunk(c)
        opt._reduced.clear()
        opt._passes.clear()
    torch.cuda.synchronize()
    ops.check_status()
    print("ok")


def case_adamw_allgather() -> None:
    """Sharded AdamW + parameter write-back on one GPU: 96 Mi parameters (fp32 master and both moments 1.1 GB, bf16
    gradients and parameters 192 MB each), three steps of three chunk launches."""
    fb, opt = _optimizer_case(96 * 1024 * 1024)
    for _ in range(3):
        opt.step()
        fb.grads.normal_(0, 0.01)
    torch.cuda.synchronize()
    ops.check_status()
    print("ok")


def case_moe_train() -> None:
    """Grouped expert MLP of training, forward + backward, at the Qwen3-30B-A3B layer shape: 4096 tokens, top-8 of 128
    experts, d = 2048, F = 768 (two warm-up passes, then one pass for the launch list)."""
    from ..ops.moe_train import GroupedExperts, GroupedPlan

    class Sink:
        def accumulate_into(self, view):
            return False

    T, k, E, d, F = 4096, 8, 128, 2048, 768
    g = torch.Generator(device="cuda").manual_seed(0)
    h = (torch.randn(T, d, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True)
    wgu = (torch.randn(E * 2 * F, d, device="cuda", generator=g) * 0.02).bfloat16()
    wd = (torch.randn(E * d, F, device="cuda", generator=g) * 0.02).bfloat16()
    ggu, gd = torch.empty_like(wgu), torch.empty_like(wd)
    wt, idx = torch.randn(T, E, device="cuda", generator=g).softmax(-1).topk(k, dim=-1)
    wt = wt.contiguous().requires_grad_(True)
    idx32 = idx.to(torch.int32).contiguous()
    dout = (torch.randn(T, d, device="cuda", generator=g) * 0.1).bfloat16()
    for _ in range(3):
        plan = GroupedPlan(idx32, E, d, F)
        GroupedExperts.apply(h, wt, wgu, ggu, wd, gd, plan, Sink()).backward(dout)
        h.grad = wt.grad = None
    torch.cuda.synchronize()
    ops.check_status()
    print("ok")


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}

if __name__ == "__main__":
    name = sys.argv[1] if len(sys.argv) > 1 else "decode_attn"
    CASES[name]()
