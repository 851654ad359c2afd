"""Worker run by the multi-rank tests: ``torchrun --nproc-per-node N multi_rank_worker.py <device> <cases>``.

Each case checks a fused compute+collective path against a plain PyTorch fp32 reference built
from all ranks' data (every rank regenerates every rank's inputs from seeds). With ``cpu`` the
ranks are gloo processes and the host-side logic runs on the collective fallbacks.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from research_b200.parallel.fsdp import FlatBuckets, ShardedAdamW  # noqa: E402
from research_b200.parallel.symm import PeerComm  # noqa: E402
from research_b200.parallel.tp import TensorParallel  # noqa: E402


def rnd(shape, seed, dev, dtype, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(dev)


def close(got, want, atol, rtol, what):
    err = (got.float().cpu() - want.float().cpu()).abs()
    tol = atol + rtol * want.float().cpu().abs()
    assert (err <= tol).all(), f"{what}: max err {err.max().item():.4g}"


def case_barrier(comm, dev, dt):
    for _ in range(5):
        comm.barrier()
    ep = comm.signal(comm.new_slot())
    assert ep == 1


def case_tp_gemms(comm, dev, dt):
    W = comm.world
    tp = TensorParallel(comm, max_rows=512, max_cols=1024)
    # the last two shapes (few rows, K >= 2048) take the split-K GEMM + pull-sum path on a GPU
    for (M, N, K) in [(64 * W, 256, 128), (128 * W, 896, 512), (256, 1024, 320), (64, 1024, 4096), (256, 896, 2048)]:
        if M % (8 * W):
            continue
        a_all = [rnd((M, K), 100 + r, dev, dt) for r in range(W)]
        w_all = [rnd((N, K), 200 + r, dev, dt, 0.1) for r in range(W)]
        full = sum(a.float() @ w.float().t() for a, w in zip(a_all, w_all))
        # all-reduce into a symmetric residual stream
        x = tp.alloc((512, N), dt)
        x0 = rnd((M, N), 7, dev, dt)
        x[:M].copy_(x0)
        comm.barrier()
        tp.gemm_all_reduce(a_all[comm.rank], w_all[comm.rank], x[:M])
        close(x[:M], full + x0.float(), 0.08 * K ** 0.5 / 4 + 0.05, 0.02, f"gemm_all_reduce {M}x{N}x{K}")
        # twice in a row exercises the double-buffered staging
        tp.gemm_all_reduce(a_all[comm.rank], w_all[comm.rank], x[:M])
        close(x[:M], 2 * full + x0.float(), 0.15 * K ** 0.5 / 4 + 0.1, 0.02, "gemm_all_reduce x2")
        # reduce-scatter
        rpr = M // W
        out = torch.zeros(rpr, N, dtype=dt, device=dev)
        res = rnd((rpr, N), 9 + comm.rank, dev, dt)
        tp.gemm_reduce_scatter(a_all[comm.rank], w_all[comm.rank], out, residual=res)
        close(out, full[comm.rank * rpr:(comm.rank + 1) * rpr] + res.float(), 0.08 * K ** 0.5 / 4 + 0.05, 0.02,
              f"gemm_reduce_scatter {M}x{N}x{K}")
        comm.barrier()
    if comm.on_gpu:
        # the split path from a CUDA graph: three calls per replay, two replays; the epochs, the block ticket and the
        # acknowledgement counts of the slab all live on the device, so the replays must keep adding correctly
        M, N, K = 64, 1024, 4096
        a_all = [rnd((M, K), 100 + r, dev, dt) for r in range(W)]
        w_all = [rnd((N, K), 200 + r, dev, dt, 0.1) for r in range(W)]
        full = sum(a.float() @ w.float().t() for a, w in zip(a_all, w_all))
        x = tp.alloc((M, N), dt)
        tp.gemm_all_reduce(a_all[comm.rank], w_all[comm.rank], x)          # eager once: work buffers exist before the capture
        comm.barrier_host()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(3):
                tp.gemm_all_reduce(a_all[comm.rank], w_all[comm.rank], x)
        x.zero_()
        g.replay()
        g.replay()
        torch.cuda.synchronize()
        close(x, 6 * full, 0.5 * K ** 0.5 / 4 + 0.3, 0.03, "gemm_all_reduce split path, graph replays")
        comm.barrier_host()
    # all-gather -> GEMM (activation shards) and FSDP weight shards read from peers in the GEMM
    rows, K, N = 128, 256, 384
    xs = tp.alloc((rows, K), dt)
    shards = [rnd((rows, K), 300 + r, dev, dt) for r in range(W)]
    xs.copy_(shards[comm.rank])
    w = rnd((N, K), 5, dev, dt, 0.1)
    ep = tp.publish()
    out = torch.empty(rows * W, N, dtype=dt, device=dev)
    tp.all_gather_gemm(xs, w, out, ready_epoch=ep)
    close(out, torch.cat(shards).float() @ w.float().t(), 0.1, 0.02, "all_gather_gemm")
    ws = tp.alloc((N // W if N % W == 0 else N, K), dt)
    wsh = [rnd((ws.shape[0], K), 400 + r, dev, dt, 0.1) for r in range(W)]
    ws.copy_(wsh[comm.rank])
    xin = rnd((192, K), 6, dev, dt)
    ep = tp.publish()
    out2 = torch.empty(192, ws.shape[0] * W, dtype=dt, device=dev)
    tp.fsdp_gemm(xin, ws, out2, ready_epoch=ep)
    close(out2, xin.float() @ torch.cat(wsh).float().t(), 0.1, 0.02, "fsdp_gemm")
    comm.barrier()


def case_sharded_adamw(comm, dev, dt):
    W = comm.world
    shapes = [("layers.0.a", (64, 48)), ("layers.0.b", (48,)), ("layers.1.a", (40, 64)), ("head", (128, 64))]
    chunk_of = lambda n: 0 if n.startswith("layers.0") else (1 if n.startswith("layers.1") else 2)  # noqa: E731
    b = FlatBuckets(comm, shapes, chunk_of, dtype=dt)
    init = {n: rnd(s, 10 + i, dev, dt) for i, (n, s) in enumerate(shapes)}
    for n, _ in shapes:
        b.param_view(n).copy_(init[n])
    comm.barrier()
    opt = ShardedAdamW(b, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0)
    # reference: torch AdamW on fp32 copies with the rank-averaged gradient and the same clipping
    ref = {n: init[n].float().cpu().clone().requires_grad_(True) for n, _ in shapes}
    ropt = torch.optim.AdamW(ref.values(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(3):
        grads_all = [{n: rnd(s, 1000 * step + 50 * r + i, dev, dt, 0.5) for i, (n, s) in enumerate(shapes)} for r in range(W)]
        for n, _ in shapes:
            b.grad_view(n).copy_(grads_all[comm.rank][n])
        opt.reduce_chunk(2)  # chunks may be reduced early, in any order (overlap with backward)
        norm = opt.step()
        for n, _ in shapes:
            ref[n].grad = sum(g[n].float().cpu() for g in grads_all) / W
        ref_norm = torch.nn.utils.clip_grad_norm_(ref.values(), 1.0)
        ropt.step()
        assert abs(float(norm) - float(ref_norm)) < 2e-2 * float(ref_norm) + 1e-3, (float(norm), float(ref_norm))
        for n, _ in shapes:
            close(b.param_view(n), ref[n].detach(), 2e-2, 2e-2, f"adamw step {step} {n}")
        assert float(b.grads.abs().sum()) == 0.0
    sd = opt.state_dict()
    opt.load_state_dict(sd)


def case_weight_sync_and_tp_engine(comm, dev, dt):
    from research_b200.inference import EngineConfig, InferenceEngine, SamplingParams
    from research_b200.models import get_preset, init_random_weights
    from research_b200.models.weights import param_shapes
    from research_b200.parallel.weight_sync import sync_engine_from_buckets

    W = comm.world
    cfg = get_preset("tiny-qwen2", num_layers=2, init_std=0.05)
    w0 = {k: v.to(dt) for k, v in init_random_weights(cfg, seed=0).items()}
    w1 = {k: v.to(dt) for k, v in init_random_weights(cfg, seed=1).items()}
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (33, 50, 18, 64)]
    ecfg = EngineConfig(max_batch_size=8, max_model_len=256, num_kv_blocks=128, ignore_eos=True, graph_batch_sizes=(8,))
    # single-rank engine as the oracle for the TP engine
    solo = InferenceEngine(ecfg, cfg, w0, device=dev)
    want = solo.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    # ---- weight sync: rank 0's flat bucket is the trainer; every rank's engine pulls from it ----
    b = FlatBuckets(comm, list(param_shapes(cfg).items()), dtype=dt)
    if comm.rank == 0:
        for n in b.specs:
            b.param_view(n).copy_(w1[n])
    comm.barrier()
    if dev.type == "cuda":
        sync_engine_from_buckets(solo, b, src_rank=0, comm=comm)  # every rank pulls rank 0's bucket over NVLink
    else:
        sync_engine_from_buckets(solo, _bcast_buckets(b, comm))
    assert solo.get_weight_version() == 1
    oracle1 = InferenceEngine(ecfg, cfg, w1, device=dev)
    a = solo.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    c = oracle1.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    assert [s.completion_tokens for s in a] == [s.completion_tokens for s in c], "synced engine differs from fresh engine"
    assert all(s.weight_version == 1 and s.cached_tokens == 0 for s in a)
    solo.shutdown()
    oracle1.shutdown()
    # ---- tensor-parallel engine over the fused GEMM + all-reduce kernel ----
    tp = TensorParallel(comm, max_rows=2048, max_cols=max(cfg.hidden_size, 1024))
    tcfg = EngineConfig(max_batch_size=16, max_model_len=256, num_kv_blocks=128, ignore_eos=True, graph_batch_sizes=(16,))
    eng = InferenceEngine(tcfg, cfg, w0, device=dev, tp=tp)
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    # Criterion of the reference's correctness harness: exact greedy match, else every chosen token must be a near-top
    # token of the fp32 oracle and the reported log-prob must agree with it. Expected bf16 error: activations carry 8
    # mantissa bits (relative rounding 2^-9), logits of magnitude 5-10 come out of two layers and a 256-wide product with
    # an absolute error of 0.01-0.04, and the tensor-parallel engine sums its partial products in a different order than
    # one GPU does. So two tokens closer than about 0.1 nats may swap (margin 0.15 = three times the typical error) and a
    # reported log-prob may be off by the same amount (0.05); a wrong shard, mask or position shows as errors of 0.5 and up.
    from research_b200.models import causal_lm_forward

    w32 = {k: v.float().cpu() for k, v in w0.items()}
    for p_, x, y in zip(prompts, got, want):
        if x.completion_tokens == y.completion_tokens:
            assert max(abs(a_ - b_) for a_, b_ in zip(x.logprobs, y.logprobs)) < 0.05
            continue
        ids = list(p_) + list(x.completion_tokens)
        lps = torch.log_softmax(causal_lm_forward(torch.tensor([ids]), w32, cfg)[0].float(), -1)
        for j, (tok, lp) in enumerate(zip(x.completion_tokens, x.logprobs)):
            row = lps[len(p_) + j - 1]
            assert row[tok].item() >= row.max().item() - 0.15, ("not a near-top token", j, row[tok].item(), row.max().item())
            assert abs(row[tok].item() - lp) < 0.05, ("log-prob mismatch", j, row[tok].item(), lp)
    eng.shutdown()
    _ = W


def case_fsdp_backend_and_grpo(comm, dev, dt):
    """Two ranks train on different data: parameters stay identical across ranks and equal a
    single-process run on the concatenated batch; then the full GRPO loop runs sharded."""
    import tempfile

    from research_b200.models import get_preset, init_random_weights
    from research_b200.training.backends import FSDPTrainingBackend, PyTorchTrainingBackend
    from research_b200.training.grpo import GRPOConfig, grpo_train

    W = comm.world
    cfg = get_preset("tiny-qwen2", num_layers=2)
    w = init_random_weights(cfg, seed=0)
    be = FSDPTrainingBackend(cfg, w, device=dev, loss_fn="ce", lr=1e-2)
    g = torch.Generator().manual_seed(0)
    all_ids = torch.randint(0, cfg.vocab_size, (2 * W, 16), generator=g)
    mine = all_ids[comm.rank * 2:(comm.rank + 1) * 2]
    for _ in range(2):
        be.forward_backward({"input_ids": mine, "labels": mine}).wait()
        be.optim_step().wait()
    flat = be.buckets.params.float()
    gathered = [torch.empty_like(flat) for _ in range(W)]
    dist.all_gather(gathered, flat)
    for other in gathered:
        assert torch.equal(other, gathered[0]), "ranks diverged"
    if dev.type == "cpu":
        solo = PyTorchTrainingBackend(cfg, w, device=dev, loss_fn="ce", lr=1e-2)
        for _ in range(2):
            solo.forward_backward({"input_ids": all_ids, "labels": all_ids}).wait()
            solo.optim_step().wait()
        for n in ("model.layers.1.mlp.down_proj.weight", "model.embed_tokens.weight"):
            close(be.buckets.param_view(n), solo.buckets.param_view(n), 5e-4, 1e-3, f"fsdp vs single {n}")
    prompts = [torch.randint(0, 4096, (int(n),), generator=g).tolist() for n in torch.randint(16, 64, (16,), generator=g)]
    with tempfile.TemporaryDirectory() as d:
        gcfg = GRPOConfig(model_name="tiny-qwen2", lr=1e-5, batch_size=4, n_samples_per_prompt=4, num_minibatches=2,
                          max_tokens=6, max_seq_len=128, temperature=1.0, num_steps=1, output_dir=d, checkpoint_every=1,
                          max_batch_size=8, kv_blocks=128, experiment_name="mr")
        import os
        os.environ["ROLLOUTS_RUN_NAME"] = "mr_run"
        hist = grpo_train(gcfg, prompts, lambda s: float(sum(s.tokens[-s.response_length:]) % 2), device=dev)
        assert len(hist) == 1 and hist[0]["weight_version"] == 1.0
        dist.barrier()


def case_fsdp_full_shard(comm, dev, dt):
    """Sharded parameters (layer matrices split by rows, gathered inside the consuming GEMM launches) against the
    replicated-parameter mode: same data, same steps, same weights afterwards."""
    from research_b200.models import get_preset, init_random_weights
    from research_b200.training.backends import FSDPTrainingBackend
    from research_b200.training.backends.fsdp import FSDPConfig

    W = comm.world
    # head size 64: the flash kernels run on a GPU; 512 tokens per rank: the GEMMs have several tiles per part
    cfg = get_preset("tiny-qwen2", num_layers=2, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64,
                     intermediate_size=512 * W if dev.type == "cuda" else 256 * W, vocab_size=1024)
    w = init_random_weights(cfg, seed=3)
    g = torch.Generator().manual_seed(1)
    T = 256 if dev.type == "cuda" else 24
    all_ids = torch.randint(0, cfg.vocab_size, (2 * W, T), generator=g)
    mine = all_ids[comm.rank * 2:(comm.rank + 1) * 2]
    results = {}
    for mode in ("shard_optimizer_and_grads", "full_shard"):
        # a small learning rate: AdamW moves every weight by about lr per step whatever the gradient's size, so where
        # the two modes' bf16 GEMMs round a tiny gradient to opposite signs the weights part by 2 lr per step
        be = FSDPTrainingBackend(cfg, w, device=dev, loss_fn="ce", lr=2e-3, comm=comm, config=FSDPConfig(sharding_strategy=mode))
        assert be.buckets.any_sharded == (mode == "full_shard")
        losses = []
        for _ in range(3):
            losses.append(be.forward_backward({"input_ids": mine, "labels": mine}).wait()["loss"])
            be.optim_step().wait()
        results[mode] = (losses, {n: be.buckets.full_param(n).float().cpu() for n in
                                  ("model.layers.1.mlp.down_proj.weight", "model.layers.0.self_attn.q_proj.weight",
                                   "model.layers.0.self_attn.k_proj.weight", "model.layers.1.mlp.gate_proj.weight",
                                   "model.embed_tokens.weight", "model.layers.0.input_layernorm.weight")})
        if mode == "full_shard":
            sp = be.buckets.specs["model.layers.0.mlp.up_proj.weight"]
            assert sp.sharded and be.buckets.param_view(sp.name).shape[0] == sp.shape[0] // W
            assert be.buckets.p_numel < be.buckets.numel
            sd = be.get_weights().wait()
            assert sd["model.layers.0.mlp.up_proj.weight"].shape == sp.shape
        comm.barrier_host()
    (la, pa), (lb, pb) = results["shard_optimizer_and_grads"], results["full_shard"]
    tol = 1.5e-2 if dev.type == "cuda" else 2e-4
    for x, y in zip(la, lb):
        assert abs(x - y) < tol * max(1.0, abs(x)), (la, lb)
    assert lb[-1] < lb[0], lb
    for n in pa:
        close(pb[n], pa[n], tol, tol, f"full_shard vs replicated {n}")


def case_ep_training(comm, dev, dt):
    """Expert-parallel training against data-parallel training with replicated experts: same data, same steps, same
    losses and weights afterwards; every rank keeps only its own experts (parameters, gradients, optimizer state)."""
    from research_b200.models import get_preset, init_random_weights
    from research_b200.training.backends import FSDPTrainingBackend
    from research_b200.training.backends.fsdp import FSDPConfig

    W = comm.world
    E = 4 * W
    cfg = get_preset("tiny-moe", num_layers=2, num_experts=E, num_experts_per_tok=2, init_std=0.05)
    w = init_random_weights(cfg, seed=5)
    g = torch.Generator().manual_seed(2)
    T = 128 if dev.type == "cuda" else 24
    all_ids = torch.randint(0, cfg.vocab_size, (2 * W, T), generator=g)
    mine = all_ids[comm.rank * 2:(comm.rank + 1) * 2]
    results = {}
    for ep in (False, True):
        be = FSDPTrainingBackend(cfg, w, device=dev, loss_fn="ce", lr=2e-3, comm=comm, config=FSDPConfig(expert_parallel=ep))
        assert be.buckets.any_owned == ep
        if ep:
            mine_e = sorted({int(n.split(".experts.")[1].split(".")[0]) for n in be.buckets.specs if ".experts." in n})
            assert mine_e == list(range(comm.rank * 4, comm.rank * 4 + 4)), mine_e
            assert be.buckets.numel < results[False][2]
        losses = []
        for _ in range(3):
            losses.append(be.forward_backward({"input_ids": mine, "labels": mine}).wait()["loss"])
            be.optim_step().wait()
        sd = be.get_weights().wait()
        assert len(sd) == len(w), (len(sd), len(w))
        if ep:      # a checkpoint holds the whole model (every rank's experts) and loads back into the expert-parallel layout
            import tempfile

            from research_b200.models.weights import load_safetensors_dir

            with tempfile.TemporaryDirectory() as d:
                path = [d]
                dist.broadcast_object_list(path, src=0)
                be.save_checkpoint_to_path(path[0], 3)
                if comm.rank == 0:
                    saved, _ = load_safetensors_dir(path[0])
                    assert {n for n in w if ".experts." in n} <= set(saved), "a checkpoint must hold every rank's experts"
                    close(saved[f"model.layers.1.mlp.experts.{E - 1}.down_proj.weight"], sd[f"model.layers.1.mlp.experts.{E - 1}.down_proj.weight"],
                          1e-6, 0, "checkpointed expert of the last rank")
                be.load_checkpoint(path[0])
                comm.barrier_host()
        results[ep] = (losses, {n: sd[n].float().cpu() for n in
                                (f"model.layers.1.mlp.experts.{E - 1}.down_proj.weight", "model.layers.1.mlp.experts.0.gate_proj.weight",
                                 f"model.layers.0.mlp.experts.{W * 4 // 2}.up_proj.weight", "model.layers.1.mlp.gate.weight",
                                 "model.layers.0.self_attn.q_proj.weight", "model.embed_tokens.weight")}, be.buckets.numel)
        comm.barrier_host()
    (la, pa, _), (lb, pb, _) = results[False], results[True]
    tol = 2e-2 if dev.type == "cuda" else 2e-4
    for x, y in zip(la, lb):
        assert abs(x - y) < tol * max(1.0, abs(x)), (la, lb)
    assert lb[-1] < lb[0], lb
    for n in pa:
        close(pb[n], pa[n], 2e-2 if dev.type == "cuda" else 2e-4, 1e-3, f"expert parallel vs replicated experts: {n}")


def case_grpo_expert_parallel(comm, dev, dt):
    """The whole GRPO loop on a mixture-of-experts model with the experts split over the ranks for rollouts (lock-step
    engines) AND for the update; the weight sync moves each rank's own experts into its engine."""
    import tempfile

    from research_b200.training.grpo import GRPOConfig, grpo_train

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 4096, (int(n),), generator=g).tolist() for n in torch.randint(16, 40, (16,), generator=g)]
    with tempfile.TemporaryDirectory() as d:
        os.environ["ROLLOUTS_RUN_NAME"] = "ep_run"
        gcfg = GRPOConfig(model_name="tiny-moe", lr=1e-4, batch_size=2 * comm.world, n_samples_per_prompt=4, num_minibatches=2, max_tokens=6,
                          max_seq_len=96, temperature=1.0, num_steps=2, output_dir=d, checkpoint_every=0, max_batch_size=16,
                          kv_blocks=128, expert_parallel=True)
        hist = grpo_train(gcfg, prompts, lambda s: float(sum(s.tokens[-s.response_length:]) % 2), device=dev)
        assert len(hist) == 2 and hist[-1]["weight_version"] == 2.0, hist[-1]
        dist.barrier()


def case_grpo_disjoint(comm, dev, dt):
    """Trainers and engine on different ranks: the last rank only serves, the others only train; samples travel to the
    trainers, the new parameters travel back into the engine's packed layout."""
    import tempfile

    from research_b200.training.grpo import GRPOConfig, device_roles, grpo_train

    W = comm.world
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 4096, (int(n),), generator=g).tolist() for n in torch.randint(16, 48, (12,), generator=g)]
    with tempfile.TemporaryDirectory() as d:
        os.environ["ROLLOUTS_RUN_NAME"] = "disjoint_run"
        gcfg = GRPOConfig(model_name="tiny-qwen2", lr=1e-4, batch_size=4, n_samples_per_prompt=4, num_minibatches=2, max_tokens=6,
                          max_seq_len=96, temperature=1.0, num_steps=2, output_dir=d, checkpoint_every=0, max_batch_size=16,
                          kv_blocks=128, trainer_cuda_device_ids=tuple(range(W - 1)), inference_cuda_device_ids=(W - 1,))
        assert device_roles(gcfg, W) == (list(range(W - 1)), [W - 1])
        assert device_roles(GRPOConfig(), W) is None
        hist = grpo_train(gcfg, prompts, lambda s: float(sum(s.tokens[-s.response_length:]) % 2), device=dev)
        assert len(hist) == 2 and hist[-1]["weight_version"] == 2.0 and hist[0]["num_samples"] == 16.0
        if comm.rank < W - 1:
            assert "loss" in hist[-1] or "pg_loss" in hist[-1], hist[-1]
        # every rank saw the same samples and the same reward statistics
        t = torch.tensor([hist[-1]["mean_reward"]], dtype=torch.float64, device=dev)
        ref = t.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(t, ref)
        dist.barrier()


def case_grpo_disjoint_tp_engine(comm, dev, dt):
    """Disjoint placement with ONE tensor-parallel engine over the serving ranks (needs at least 3 ranks: the last two
    serve): both engine ranks generate the same samples in step, one of them reports, the trainers' new parameters
    reach both engine shards."""
    import tempfile

    from research_b200.training.grpo import GRPOConfig, grpo_train

    W = comm.world
    if W < 3:
        return
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 4096, (int(n),), generator=g).tolist() for n in torch.randint(16, 48, (12,), generator=g)]
    with tempfile.TemporaryDirectory() as d:
        os.environ["ROLLOUTS_RUN_NAME"] = "disjoint_tp_run"
        gcfg = GRPOConfig(model_name="tiny-qwen2", lr=1e-4, batch_size=4, n_samples_per_prompt=4, num_minibatches=2, max_tokens=6,
                          max_seq_len=96, temperature=1.0, num_steps=2, output_dir=d, checkpoint_every=0, max_batch_size=16,
                          kv_blocks=128, trainer_cuda_device_ids=tuple(range(W - 2)), inference_cuda_device_ids=(W - 2, W - 1),
                          inference_parallelism="tensor")
        hist = grpo_train(gcfg, prompts, lambda s: float(sum(s.tokens[-s.response_length:]) % 2), device=dev)
        # 4 prompt groups x 4 samples from the one engine (not once per engine rank)
        assert len(hist) == 2 and hist[-1]["weight_version"] == 2.0 and hist[0]["num_samples"] == 16.0, hist[0]
        t = torch.tensor([hist[-1]["mean_reward"]], dtype=torch.float64, device=dev)
        ref = t.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(t, ref)
        dist.barrier()


def case_moe_expert_parallel(comm, dev, dt):
    """Each rank routes its own tokens; experts are split over the ranks; dispatch and combine
    travel through peer memory. Checked against the single-process functional MoE."""
    from research_b200.models import get_preset, init_random_weights
    from research_b200.models.functional import moe_mlp
    from research_b200.parallel.moe import MoELayerWeights

    cfg = get_preset("tiny-moe", num_layers=2, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128,
                     init_std=0.05)
    w = {n: v.to(dt).float() for n, v in init_random_weights(cfg, seed=0).items() if n.startswith("model.layers.1.mlp.")}
    tp = TensorParallel(comm, max_rows=512, max_cols=1024, expert_parallel=True)
    layer = MoELayerWeights(cfg, dev, ep=tp)
    layer.load(w, "model.layers.1.mlp.")
    for T in (7, 200):
        h = rnd((T, cfg.hidden_size), 500 + comm.rank + T, dev, dt, 0.5)
        x0 = rnd((T, cfg.hidden_size), 600 + comm.rank + T, dev, dt)
        x = x0.clone()
        layer.forward(h, x)
        want = x0.float().cpu() + moe_mlp(h.float().cpu()[None], w, "model.layers.1.mlp.", cfg)[0]
        close(x, want, 0.08, 0.02, f"expert-parallel MoE T={T}")
    comm.barrier()


def _bcast_buckets(b, comm):
    dist.broadcast(b.params, src=0, group=comm.group)
    return b


def case_ep_agree(comm, dev, dt):
    """Per-step agreement of the expert-parallel engines: element-wise maximum over the ranks. On GPUs it travels through
    peer memory with a bounded wait: one rank arrives late ON THE HOST (nothing of it is in flight), its peers' wait
    runs out after a second and reports the failure, the context stays usable and the retry succeeds."""
    import time

    from research_b200.parallel.ep import ExpertParallel, PeerFailure

    W, r = comm.world, comm.rank
    ep = ExpertParallel(comm, timeout_s=1.0 if comm.on_gpu else 30.0)
    assert ep.agree(r, 5 - r, 0) == (W - 1, 5, 0)
    assert ep.agree(0) == (0,) and ep.agree(int(r == 0)) == (1,)
    if comm.on_gpu:
        assert ep.device_agree
        dist.barrier()
        late = r == W - 1
        if late:
            time.sleep(2.5)
        try:
            got, failed = ep.agree(1), False
        except PeerFailure:
            got, failed = None, True
        assert failed == (not late), (r, failed)
        if late:
            assert got == (1,)        # the peers' values of this epoch were already in its buffer
        dist.barrier()
        if failed:                    # the ranks that gave up did not advance their epoch: they ask again
            assert ep.agree(1) == (1,)
        x = torch.ones(4, device=dev)                 # the device still runs ordinary work
        assert float((x * 2).sum()) == 8.0
        assert ep.agree(r) == (W - 1,)


def case_tp_training(comm, dev, dt):
    """Tensor-parallel (x data-parallel) training against the single-process functional model: same loss, same full
    gradient, same weights after two AdamW steps, for a tied and an untied head, with QK-norm, and for the GRPO loss
    with its entropy term. World 2: tp 2. World 4: tp 2 x dp 2 (each data-parallel half has its own batch)."""
    from research_b200.models import causal_lm_forward, get_preset, init_random_weights
    from research_b200.training.backends.tensor_parallel import TensorParallelTrainingBackend, shard_weights, unshard_weights
    from research_b200.training.backends.torch_func import TorchFuncTrainingBackend
    from research_b200.training.types import TrainerConfig

    W, r = comm.world, comm.rank
    tp = 2
    dp = W // tp
    tol = dict(atol=2e-5, rtol=2e-4) if dev.type == "cpu" else dict(atol=3e-2, rtol=5e-2)
    for preset, kw, loss in (("tiny-qwen2", {}, "ce"), ("tiny-llama", {}, "grpo"), ("tiny-qwen3", {}, "ce")):
        try:
            cfg = get_preset(preset, num_layers=2, **kw)
        except (KeyError, AssertionError):
            continue
        full = init_random_weights(cfg, seed=3)
        parts = [shard_weights(full, i, tp) for i in range(tp)]
        back = unshard_weights(parts)
        assert all(torch.equal(back[k], full[k]) for k in full) and parts[0]["model.layers.0.self_attn.o_proj.weight"].shape[1] * tp == cfg.num_heads * cfg.head_dim
        tc = TrainerConfig(max_grad_norm=0.5)
        be = TensorParallelTrainingBackend(cfg, full, tp_size=tp, device=dev, dtype=dt if dev.type == "cuda" else torch.float32, loss_fn=loss, lr=1e-2, trainer_config=tc)
        assert (be.tp_rank, be.dp_rank, be.dp_size) == (r % tp, r // tp, dp)
        ref = TorchFuncTrainingBackend(cfg, full, device="cpu", loss_fn=loss, lr=1e-2, trainer_config=tc)

        def batch_of(group: int, step: int):
            g = torch.Generator().manual_seed(100 * step + group)
            ids = torch.randint(0, cfg.vocab_size, (4, 12), generator=g)
            mask = torch.ones(4, 12)
            mask[:, :3] = 0
            b = {"input_ids": ids, "labels": ids.clone(), "loss_mask": mask}
            if loss == "grpo":
                b["advantages"] = torch.randn(4, generator=g)
            return b

        for step in range(2):
            m = be.forward_backward(batch_of(r // tp, step)).wait()
            losses = []
            for grp in range(dp):                       # the oracle sees every data-parallel group's batch
                losses.append(ref.forward_backward(batch_of(grp, step)).wait()["loss"])
            assert abs(m["loss"] - losses[r // tp]) < (1e-4 if dev.type == "cpu" else 5e-2), (preset, step, m["loss"], losses)
            got = be.gathered_grads()
            for k, g in ref.grads.items():
                # after a step the two sets of weights differ in single entries (see below), and so do the gradients
                close(got[k], g / dp, what=f"{preset} step {step} grad {k}", atol=tol["atol"] * (1 if step == 0 else 20), rtol=tol["rtol"] * (1 if step == 0 else 20))
            ref_g = {k: (g / dp).float().cpu() for k, g in ref.grads.items()}
            n_be = be.optim_step().wait()["grad_norm"]
            n_ref = ref.optim_step().wait()["grad_norm"]
            assert abs(n_be - n_ref) <= (1e-3 if dev.type == "cpu" else 0.05) * max(n_ref, 1.0), (preset, n_be, n_ref)
            assert all(v.dtype == be.dtype for v in be.get_weights().wait().values())
            w = be._gather(be.master)             # the fp32 masters: the working copies add bf16 rounding (0.4 % of a norm weight)
            for k, v in ref.params.items():
                # Adam divides by the root of the second moment: where a gradient is almost zero, rounding differences move
                # single entries by a visible fraction of the learning rate (1e-2). On CPU (fp32 on both sides) that leaves
                # very few outliers and a tiny mean error. With bf16 gradients every near-zero entry is noise (a whole key
                # bias is), so there the comparison looks at entries with a gradient worth the name, after the first step
                err = (w[k].float().cpu() - v.float().cpu()).abs()
                if dev.type == "cpu":
                    off = (err > 0.05 * 1e-2).float().mean()
                    assert off < 1e-3 and err.mean() < 1e-4, f"{preset} step {step} weight {k}: {off:.2%} off, mean {err.mean():.3g}"
                elif step == 0:
                    strong = ref_g[k].abs() > 0.2 * ref_g[k].abs().max().clamp_min(1e-12)
                    if strong.any():
                        off = (err[strong] > 0.5 * 1e-2).float().mean()
                        assert off < 0.05, f"{preset} weight {k}: {off:.2%} of the {int(strong.sum())} entries with a clear gradient moved differently"
        # ranks of one tensor-parallel group must be fed the same tokens
        if dev.type == "cpu":
            bad = batch_of(r // tp, 7)
            bad["input_ids"] = bad["input_ids"] + (r % tp)
            try:
                be.forward_backward(bad)
                raise SystemExit("different batches inside a tensor-parallel group went unnoticed")
            except AssertionError as e:
                assert "different batches" in str(e)
    # checkpoint: the full model once, optimizer shards per tensor-parallel rank; a fresh backend resumes from it
    import tempfile

    box = [tempfile.mkdtemp() if r == 0 else None]
    dist.broadcast_object_list(box, src=0)
    cfg = get_preset("tiny-qwen2", num_layers=1)
    full = init_random_weights(cfg, seed=5)
    a = TensorParallelTrainingBackend(cfg, full, tp_size=tp, device=dev, checkpoint_dir=box[0], lr=1e-2)
    ids = torch.randint(0, cfg.vocab_size, (2, 8), generator=torch.Generator().manual_seed(r // tp))
    a.forward_backward({"input_ids": ids, "labels": ids})
    a.optim_step()
    path = a.save_checkpoint()
    b = TensorParallelTrainingBackend(cfg, init_random_weights(cfg, seed=6), tp_size=tp, device=dev, checkpoint_dir=box[0], lr=1e-2)
    b.load_checkpoint(path)
    assert b.current_step == 1 and all(torch.equal(b.master[k], a.master[k]) for k in a.master) and b.opt_state.step == 1
    from research_b200.models.weights import load_safetensors_dir

    saved, saved_cfg = load_safetensors_dir(path / "hf")
    wa = a.get_weights().wait()
    assert saved_cfg.hidden_size == cfg.hidden_size and all(torch.allclose(saved[k].float(), wa[k].float().cpu()) for k in wa)
    for be2 in (a, b):
        be2.forward_backward({"input_ids": ids, "labels": ids})
        be2.optim_step()
    assert all(torch.equal(b.master[k], a.master[k]) for k in a.master)


CASES = {"tp_training": case_tp_training, "ep_agree": case_ep_agree, "barrier": case_barrier, "tp_gemms": case_tp_gemms, "sharded_adamw": case_sharded_adamw,
         "weight_sync_tp_engine": case_weight_sync_and_tp_engine, "fsdp_backend_grpo": case_fsdp_backend_and_grpo,
         "fsdp_full_shard": case_fsdp_full_shard, "ep_training": case_ep_training, "grpo_expert_parallel": case_grpo_expert_parallel, "grpo_disjoint": case_grpo_disjoint, "grpo_disjoint_tp_engine": case_grpo_disjoint_tp_engine,
         "moe_ep": case_moe_expert_parallel}


def main():
    device = sys.argv[1]
    cases = sys.argv[2].split(",") if len(sys.argv) > 2 else list(CASES)
    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", "0"))
    if os.environ.get("RB_TEST_DUMP_AFTER"):
        import faulthandler

        faulthandler.dump_traceback_later(int(os.environ["RB_TEST_DUMP_AFTER"]), exit=True)
    if device == "cuda":
        torch.cuda.set_device(local)
        dev, dt = torch.device("cuda", local), torch.bfloat16
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev, dt = torch.device("cpu"), torch.float32
        dist.init_process_group("gloo")
    comm = PeerComm(device=dev)
    for name in cases:
        CASES[name](comm, dev, dt)
        if device == "cuda":
            from research_b200.ops import check_status

            torch.cuda.synchronize()
            check_status(dev)
        dist.barrier()
        if rank == 0:
            print(f"CASE_OK {name}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
