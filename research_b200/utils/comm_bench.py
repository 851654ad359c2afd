"""Roofline fractions of the fused compute + collective kernels, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29551 \\
        -m research_b200.utils.comm_bench [--link-gbs 770] [--peak-tflops 1688.4] [--hbm-gbs 6453.4]

Every kernel is timed with CUDA events on the launching stream after warm-up, four calls back to back per sample (the
tensor-parallel launches replayed from a CUDA graph, as in an engine step), a device barrier before each sample (so that
no rank starts early), median over the samples, maximum over ranks. The target time of a fused kernel is the slower of its FLOPs at the
measured GEMM peak and the bytes that must cross NVLink (per direction, per GPU) at the measured peer-copy bandwidth;
the line reports achieved = target / measured. One JSON object per kernel on rank 0.

Covered: fused GEMM + all-reduce / reduce-scatter (tensor-parallel row-parallel projections), all-gather fused into the
GEMM (tensor-parallel column-parallel projections, decode and prefill sizes), parameter all-gather fused into the GEMM
(sharded-parameter training: forward launch that consumes the gather, weight-gradient launch that carries it), gradient
reduce-scatter, sharded AdamW + parameter all-gather, trainer -> engine reshard copy.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--link-gbs", type=float, default=770.0, help="measured peer-copy bandwidth per direction per GPU")
    ap.add_argument("--peak-tflops", type=float, default=1688.4, help="measured cuBLAS bf16 burst throughput")
    ap.add_argument("--hbm-gbs", type=float, default=6453.4)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()

    from .. import ops
    from ..ops.gemm import gemm2
    from ..parallel.fsdp import FlatBuckets, ShardedAdamW
    from ..parallel.symm import PeerComm
    from ..parallel.tp import TensorParallel

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    comm = PeerComm(device=dev)
    W, r = comm.world, comm.rank
    link, peak, hbm = args.link_gbs * 1e9, args.peak_tflops * 1e12, args.hbm_gbs * 1e9
    bar_slot = comm.new_slot()
    rows_out = []

    def timed(fn, graph=False, reps=4, iters=args.iters, warm=3):
        """Seconds per call: `reps` calls back to back between two events (so that the host's launch work hides behind
        the previous call), replayed from a CUDA graph for the launches that an engine step captures too."""
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(reps):
                    fn()
            run = g.replay
        else:
            def run():
                for _ in range(reps):
                    fn()
        run()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            comm.barrier(bar_slot)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e-3 / reps)
        t = torch.tensor([statistics.median(ts)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def report(name, seconds, flops=0.0, link_bytes=0.0, hbm_bytes=0.0, **extra):
        target = max(flops / peak, link_bytes / link, hbm_bytes / hbm)
        bound = "compute" if target == flops / peak else ("nvlink" if target == link_bytes / link else "hbm")
        row = {"kernel": name, "ranks": W, "us": round(seconds * 1e6, 1), "target_us": round(target * 1e6, 1), "bound": bound,
               "fraction_of_roofline": round(target / seconds, 3), **extra}
        if flops:
            row["tflops"] = round(flops / seconds / 1e12, 1)
        if link_bytes:
            row["link_gbs"] = round(link_bytes / seconds / 1e9, 1)
        rows_out.append(row)
        if r == 0:
            print(json.dumps(row), flush=True)

    g = torch.Generator(device=dev).manual_seed(1 + r)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).bfloat16()

    # ------------------------------------------------------------------ tensor-parallel GEMMs (Llama-3-8B shape)
    d, F, Hd = 4096, 14336, 4096
    tp = TensorParallel(comm, max_rows=4096, max_cols=d)
    for M, tag in ((64 * W if 64 % (8 * W) else 64, "decode batch 64"), (256, "decode batch 256"), (4096, "prefill 4096 tokens")):
        M = -(-M // (8 * W)) * 8 * W
        rpr = M // W
        # row-parallel: o projection (K = Hd / W) and down projection (K = F / W)
        for K, what in ((Hd // W, "o"), (F // W, "down")):
            a, w = rnd(M, K), rnd(d, K, scale=0.05)
            x = tp.alloc((M, d))
            flops = 2.0 * M * d * K
            t = timed(lambda: tp.gemm_all_reduce(a, w, x), graph=True)
            report(f"gemm_all_reduce {what} ({tag})", t, flops, 2.0 * (W - 1) / W * M * d * 2, M=M, N=d, K=K)
            out, res = torch.zeros(rpr, d, dtype=torch.bfloat16, device=dev), rnd(rpr, d)
            t = timed(lambda: tp.gemm_reduce_scatter(a, w, out, residual=res), graph=True)
            report(f"gemm_reduce_scatter {what} ({tag})", t, flops, (W - 1) / W * M * d * 2, M=M, N=d, K=K)
            del a, w, x
        # column-parallel: q|k|v (N = 6144 / W) and gate|up (N = 2 F / W), activations gathered inside the launch
        xs = tp.alloc((rpr, d))
        xs.copy_(rnd(rpr, d))
        for N, what in ((6144 // W, "q|k|v"), (2 * F // W, "gate|up")):
            w = rnd(N, d, scale=0.05)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

            def ag():
                tp.publish_device()
                tp.all_gather_gemm(xs, w, out, ready_epoch="device")

            t = timed(ag, graph=True)
            report(f"all_gather_gemm {what} ({tag})", t, 2.0 * M * N * d, (W - 1) * rpr * d * 2, M=M, N=N, K=d)
            del w, out
    comm.barrier_host()

    # ------------------------------------------------------------------ sharded-parameter GEMMs (training, 4096 tokens)
    T = 4096
    shapes = [("model.layers.0.mlp.gate_proj.weight", (2 * F, d)), ("model.layers.0.self_attn.o_proj.weight", (d, d))]
    fb = FlatBuckets(comm, shapes, lambda n: 0, shard_rule=lambda n, s: True)
    fb.params.normal_(0, 0.02)
    comm.barrier_host()
    x = rnd(T, d)
    for name, (N, K) in shapes:
        h = fb.sharded_weight(name)
        flops = 2.0 * T * N * K
        remote = (W - 1) / W * N * K * 2
        full = fb.full_param(name).contiguous()
        out = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
        t_plain1 = timed(lambda: ops.gemm(x, full, out=out, bn=256))
        t_pair = timed(lambda: gemm2(x, full, out=out))
        t = timed(lambda: ops.gemm(x, None, out=out, b_gather=h))
        report(f"gather + GEMM forward {N}x{K} (consumed by the launch)", t, flops, remote, M=T, N=N, K=K,
               same_gemm_without_gather_us=round(t_plain1 * 1e6, 1), pair_kernel_local_weights_us=round(t_pair * 1e6, 1))
        dy = rnd(T, N, scale=0.1)
        gw = torch.zeros(N, K, dtype=torch.bfloat16, device=dev)
        t0 = timed(lambda: ops.gemm(dy, x, out=gw, a_mn_major=True, b_mn_major=True, bn=256))
        t = timed(lambda: ops.gemm(dy, x, out=gw, a_mn_major=True, b_mn_major=True, carry_gather=h))
        report(f"weight-gradient GEMM {N}x{K} carrying the gather for the data-gradient GEMM", t, flops, remote, M=N, N=K, K=T,
               same_gemm_without_gather_us=round(t0 * 1e6, 1))
        del full, out, dy, gw
    del fb
    comm.barrier_host()

    # ------------------------------------------------------------------ optimizer collectives (one 8B layer = 218 M parameters)
    n_layer = 218_112_000 // (8 * W) * (8 * W)
    rows = n_layer // 4096
    fb = FlatBuckets(comm, [("w", (rows, 4096))], lambda n: 0)
    fb.params.normal_(0, 0.02)
    fb.grads.normal_(0, 0.01)
    opt = ShardedAdamW(fb, lr=1e-5, max_grad_norm=1.0)
    n = rows * 4096
    shard = n // W

    def rs():
        opt.reduce_chunk(0)
        opt._reduced.clear()
        opt._passes.clear()

    t = timed(rs)
    report("rs_reduce (one layer's gradients: pull my slice from every peer, fp32 sum, scale, norm partial)", t, 0.0,
           (W - 1) * shard * 2, shard * 2 + shard * 4, elements=n)

    def adamw():
        opt._update_chunk(0, 0.9, 0.95)

    opt.step_count = 1
    t = timed(adamw)
    report("adamw_allgather (one layer: AdamW on my slice, bf16 values pushed to every peer)", t, 0.0, (W - 1) * shard * 2,
           shard * 30, elements=n)
    comm.barrier_host()

    # ------------------------------------------------------------------ trainer -> engine reshard copy (peer read of a flat bucket)
    from ..parallel.symm import _lib as comm_lib, ptr_array
    from ..ops._util import check_rc, stream_handle
    import numpy as np

    from ..parallel.weight_sync import SEG_DTYPE

    src = fb.params_buf.peer_ptrs[(r + 1) % W]
    dst = torch.empty(n, dtype=torch.bfloat16, device=dev)
    seg_rows = 1024
    segs = np.zeros(rows // seg_rows, dtype=SEG_DTYPE)
    for j in range(len(segs)):
        segs[j] = (src + j * seg_rows * 4096 * 2, dst.data_ptr() + j * seg_rows * 4096 * 2, 4096, 4096, seg_rows, 4096, j * seg_rows * 4096 // 8)
    table = torch.from_numpy(segs.view(np.uint8).copy()).to(dev)
    total = len(segs) * seg_rows * 4096 // 8

    def reshard():
        check_rc(comm_lib().rb_reshard_copy(table.data_ptr(), len(segs), total, stream_handle(dev)), "rb_reshard_copy")

    t = timed(reshard)
    moved = len(segs) * seg_rows * 4096 * 2
    report("reshard_copy (engine pulls a layer's parameters out of a peer's bucket)", t, 0.0, moved, moved, bytes=moved)
    ops.check_status(dev)
    _ = ptr_array
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
