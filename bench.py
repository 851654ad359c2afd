"""Headline benchmark: sharded-data-parallel training throughput (tokens/s) on the Llama-3-8B shape.

Default workload ``train`` (BASELINE.json, "Llama-3-8B-shaped FSDP training ... bf16 params/grads with fp32
AdamW master state ... sequence length 4096 ... measured at 1/2/4/8 GPUs"): 32 layers, d 4096, 32 query / 8 KV
heads (head_dim 128), ffn 14336, vocab 128256, random init; one sequence of 4096 uniform-random token ids per
GPU per step (weak scaling), next-token cross-entropy. One step = forward + backward + optimizer step
(gradient reduce-scatter overlapped with backward, clip, sharded AdamW, parameter all-gather), all on this
repository's kernels over NVLink peer memory.

  value      : device time of K steps whose token batch already lies on the device (kernel-only)
  e2e.value  : the same K steps through the public backend API, ``forward_backward(batch).wait()`` +
               ``optim_step().wait()``, with the host batch staged through pinned memory and copied to the device
               every step and the step's loss / token count / gradient norm read back to the host every step

At N >= 2 every fused multi-GPU kernel the step depends on is first checked once against a ``torch.distributed``
oracle (``selfcheck`` in the JSON line); a mismatch ends the run with a non-zero exit code.

``--workload rollout`` / ``serving`` run the inference-engine workloads (Qwen2.5-0.5B-shaped rollout decode with
data-parallel replicas; Llama-3-8B-shaped serving, ``--tp`` for one tensor-parallel engine, ``--ep`` for MoE).

``--impl reference`` drives the unmodified reference package from ``baseline/_ref`` through its own public API:
for ``train`` its ``FSDPTrainingBackend`` on a random-init HF Llama of the same shape; for ``rollout`` its
``InferenceEngine``. ``--impl library`` is a same-box library baseline that does not import the reference
package: HF ``LlamaForCausalLM`` from config + ``torch.distributed.fsdp.fully_shard`` per decoder layer +
``torch.optim.AdamW`` + full-logits cross-entropy, i.e. what the reference backend does
(rollouts/training/backends/fsdp.py:253-479).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

MODEL = dict(vocab=151936, layers=24, d=896, heads=14, kv_heads=2, head_dim=64, ffn=4864)
N_REQUESTS, PROMPT_LO, PROMPT_HI, SHARED_PREFIX, NEW_TOKENS, MAX_BATCH = 1024, 128, 1024, 512, 512, 256


MAX_MODEL_LEN = 2048
SEQ_DESC = "prompt U[128,1024] (50% share a 512-token prefix) + 512 new"


def set_workload(name: str) -> None:
    """``rollout``: the flagship workload above. ``serving``: the tensor-parallel serving case (batch 64, random-token
    prompts of 2048 tokens, 256 decoded tokens each, no shared prefix)."""
    global N_REQUESTS, PROMPT_LO, PROMPT_HI, SHARED_PREFIX, NEW_TOKENS, MAX_BATCH, MAX_MODEL_LEN, SEQ_DESC
    if name == "serving":
        N_REQUESTS, PROMPT_LO, PROMPT_HI, SHARED_PREFIX, NEW_TOKENS, MAX_BATCH = 256, 2048, 2048, 0, 256, 64
        MAX_MODEL_LEN, SEQ_DESC = 2560, "prompt 2048 random tokens + 256 new"


def make_workload(seed: int, vocab: int):
    import torch

    g = torch.Generator().manual_seed(seed)
    shared = torch.randint(0, vocab, (SHARED_PREFIX,), generator=g).tolist()
    lens = torch.randint(PROMPT_LO, PROMPT_HI + 1, (N_REQUESTS,), generator=g).tolist()
    share = (torch.rand(N_REQUESTS, generator=g) < (0.5 if SHARED_PREFIX > 0 else -1.0)).tolist()
    prompts = []
    for n, s in zip(lens, share):
        if s:
            n = max(n, SHARED_PREFIX + 1)
            p = shared + torch.randint(0, vocab, (n - SHARED_PREFIX,), generator=g).tolist()
        else:
            p = torch.randint(0, vocab, (n,), generator=g).tolist()
        prompts.append(p)
    return prompts


def dist_setup(n_gpus: int):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
    assert world == n_gpus or world == 1, f"--gpus {n_gpus} but WORLD_SIZE={world}"
    return rank, world, local


def barrier(world: int):
    import torch
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    import torch
    import torch.distributed as dist

    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int) -> float:
    import torch
    import torch.distributed as dist

    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def engine_config(model: str, workload: str, global_batch: int, parallelism: str) -> dict:
    """The ``config`` dict of an engine line: the same keys and values for every arm of one workload."""
    from research_b200.models import get_preset

    cfg = get_preset(model)
    return {"model": (f"{model}-shaped ({cfg.num_layers}L d{cfg.hidden_size} {cfg.num_heads}q/{cfg.num_kv_heads}kv "
                      f"hd{cfg.head_dim} ffn{cfg.intermediate_size} vocab{cfg.vocab_size})"),
            "global_batch": global_batch, "seq_len": SEQ_DESC, "workload": workload, "parallelism": parallelism,
            "requests_per_replica": N_REQUESTS, "temperature": 1.0,
            "l2": "inputs larger than L2 (weights + KV read per step exceed 126 MB)"}


# ------------------------------------------------------------------------------------ native arm
def run_engine(args) -> dict:
    import torch

    from research_b200.inference import EngineConfig, InferenceEngine, SamplingParams
    from research_b200.models import LazyRandomWeights, get_preset, init_random_weights
    from research_b200.ops import check_status
    from research_b200.utils.timing import ClockSampler

    rank, world, local = dist_setup(args.gpus)
    dev = torch.device(f"cuda:{local}")
    cfg = get_preset(args.model)
    if cfg.num_params() > 12e9:   # tens of GB: build each tensor when the engine asks for it instead of a second full copy
        weights = LazyRandomWeights(cfg, seed=0, dtype=torch.bfloat16, device=dev)
    else:
        weights = init_random_weights(cfg, seed=0, dtype=torch.bfloat16, device=dev)
    tp = None
    if args.tp and world > 1:
        # one engine over all ranks: fused GEMM + all-reduce kernels over NVLink peer memory; every rank
        # runs the same schedule on the same requests, so the workload seed is shared
        from research_b200.parallel.symm import PeerComm
        from research_b200.parallel.tp import TensorParallel

        tp = TensorParallel(PeerComm(device=dev), max_rows=16384 + 64, max_cols=max(cfg.hidden_size, 1024))
    ep = None
    if args.ep and world > 1:
        # one engine per rank on its own requests (data-parallel attention), experts split over the ranks;
        # dispatch and combine are peer stores from inside the MoE kernels, the engines step in lock step
        from research_b200.parallel import ExpertParallel
        from research_b200.parallel.symm import PeerComm

        assert cfg.is_moe and tp is None, "--ep needs a mixture-of-experts model and excludes --tp"
        ep = ExpertParallel(PeerComm(device=dev))
    wl_rank = 0 if tp is not None else rank
    # KV pool: 640k tokens, or what 80 GB hold (large models)
    per_block = cfg.num_layers * 2 * (cfg.num_kv_heads // (world if tp is not None else 1)) * 16 * cfg.head_dim * 2
    KV_BLOCKS = int(min(40000, 80e9 // per_block))
    eng = InferenceEngine(
        EngineConfig(cache_type="radix", max_batch_size=MAX_BATCH, max_model_len=MAX_MODEL_LEN, ignore_eos=True,
                     max_tokens_per_batch=16384, num_kv_blocks=KV_BLOCKS, seed=wl_rank),
        cfg, weights, device=dev, tp=tp, ep=ep)
    del weights
    rank_for_seeds, rank = rank, wl_rank
    prompts = make_workload(rank, cfg.vocab_size)
    params = SamplingParams(temperature=1.0, max_tokens=NEW_TOKENS)
    for i, p in enumerate(prompts):
        eng.add_request(p, SamplingParams(temperature=1.0, max_tokens=NEW_TOKENS, seed=rank * 100003 + i))
    _ = params
    # ramp (untimed): admit and prefill until the running batch is full and a pure decode step ran
    ramp_steps = 0
    while True:
        eng.step()
        ramp_steps += 1
        n_prefill, n_decode = eng.last_step_rows
        full = n_prefill == 0 and n_decode == MAX_BATCH
        if ep is not None:       # lock step: every rank leaves the ramp in the same iteration
            full = not ep.agree(int(not full))[0]
        if full:
            break
        assert ramp_steps < 64, "engine did not reach a full running batch"
    K, W = args.steps, max(args.warmup, 3)

    def refill():
        # continuous batching: keep the queue non-empty if K outlasts the 1024 requests
        if eng.num_waiting() == 0 and eng.num_running() < MAX_BATCH:
            for i, p in enumerate(prompts):
                eng.add_request(p, SamplingParams(temperature=1.0, max_tokens=NEW_TOKENS, seed=rank * 100003 + i + 7919))

    # ---- end-to-end: K calls of the public step() ----
    for _ in range(W):
        eng.step()
    r = eng.runner
    bt_cols = max(1, eng._max_blocks_in(r.meta_host[3 * MAX_BATCH:4 * MAX_BATCH]))
    h2d = r.meta_host.numel() * 4 + MAX_BATCH * bt_cols * 4
    d2h = r.out_host.numel() * 4
    sampler = ClockSampler(local).start()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    toks_e2e = 0
    for _ in range(K):
        refill()
        eng.step()
        toks_e2e += eng.last_step_rows[0] + eng.last_step_rows[1]  # every scheduled row yields one token
    e1.record()
    barrier(world)
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world)
    toks_e2e_total = sum_over_ranks(float(toks_e2e), world)

    # ---- kernel-only: the same decode graph replayed K times (inputs: weights 0.99 GB + KV > L2) ----
    g = r.graphs[MAX_BATCH]
    for _ in range(W):
        g.replay()
    barrier(world)
    e0.record()
    for _ in range(K):
        g.replay()
    e1.record()
    barrier(world)
    dev_ms = max_over_ranks(e0.elapsed_time(e1), world)
    clocks = sampler.stop()
    check_status(dev)
    launches = r.launches_per_graph.get(MAX_BATCH, 0) * K

    rows_replayed = int((r.meta_host[3 * MAX_BATCH:4 * MAX_BATCH] > 0).sum())  # live rows in the replayed batch
    replicas = 1 if tp is not None else world
    value = sum_over_ranks(float(rows_replayed * K), world) / max(world // replicas, 1) / (dev_ms * 1e-3)
    e2e = toks_e2e_total / max(world // replicas, 1) / (e2e_ms * 1e-3)
    rank = rank_for_seeds
    out = {
        "metric": ("ep_rollout_decode_tokens_per_s" if ep is not None else
                   "rollout_decode_tokens_per_s" if tp is None else "tp_serving_decode_tokens_per_s"),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True,
        "scaling": "weak" if tp is None else "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform-random token ids, random-init weights)",
        "impl": "native",
        "config": engine_config(args.model, args.workload, MAX_BATCH * replicas,
                                f"dp{world}+ep{world}" if ep is not None else f"dp{world}" if tp is None else f"tp{world}"),
        "engine": {"cuda_graph_decode": True, "kv_cache": "paged, radix prefix reuse"},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / K, 4),
                "wall_ms_per_step": round(wall_ms / K, 4), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
        "cache": eng.cache_stats(), "ramp_steps": ramp_steps,
    }
    eng.shutdown()
    return out if rank == 0 else {}


# --------------------------------------------------------------------------------- reference arm
def build_reference_model_dir(path: str) -> None:
    """HF checkpoint of the benchmark shape with random weights plus a minimal tokenizer."""
    import torch

    from research_b200.models import get_preset, init_random_weights
    from research_b200.models.weights import save_safetensors_dir

    cfg = get_preset("qwen2.5-0.5b")
    w = init_random_weights(cfg, seed=0, dtype=torch.bfloat16)
    save_safetensors_dir(w, cfg, path)
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    vocab = {"<eos>": 0, "<unk>": 1, "a": 2, "b": 3}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<eos>", unk_token="<unk>").save_pretrained(path)


def run_reference_engine(args) -> dict:
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "rollouts")):
        return {"impl": "reference", "unavailable": "baseline/_ref/rollouts is absent (reference not installed on this box)"}
    sys.path.insert(0, ref_dir)
    try:
        import torch
        from rollouts.inference.engine import InferenceEngine as RefEngine
        from rollouts.inference.types import EngineConfig as RefConfig
        from rollouts.inference.types import SamplingParams as RefParams
    except Exception as e:  # missing dependency of the reference package
        return {"impl": "reference", "unavailable": f"reference import failed: {type(e).__name__}: {e}"[:300]}
    rank, world, local = dist_setup(args.gpus)
    tmp = tempfile.mkdtemp(prefix=f"ref_model_r{rank}_")
    build_reference_model_dir(tmp)
    eng = RefEngine(RefConfig(model_path=tmp, max_batch_size=MAX_BATCH))
    prompts = make_workload(rank, MODEL["vocab"])
    torch.manual_seed(rank)
    for p in prompts:
        eng.add_request(p, RefParams(temperature=1.0, max_tokens=NEW_TOKENS))
    K, W = args.steps, max(args.warmup, 3)
    # ramp: the reference admits up to max_batch_size sequences under its token budget per step
    ramp = 0
    while len(eng.running) < MAX_BATCH:
        eng.step()
        ramp += 1
        assert ramp < 16
    for _ in range(W):
        eng.step()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    toks = 0
    for _ in range(K):
        before = sum(s.num_generated for s in eng.running)
        n_running = len(eng.running)
        eng.step()
        toks += n_running
        _ = before
    e1.record()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    total = sum_over_ranks(float(toks), world)
    value = total / (ms * 1e-3)
    out = {
        "metric": "rollout_decode_tokens_per_s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": round(ms / K, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform-random token ids, random-init weights)",
        "impl": "reference",
        "config": engine_config("qwen2.5-0.5b", "rollout", MAX_BATCH * world, f"dp{world}"),
        "engine": "rollouts.inference.InferenceEngine (unmodified; no KV cache, one sequence per forward)",
        "e2e": {"value": round(value, 2), "unit": "tokens/s",
                "note": "the reference's step() is already end to end: it builds inputs on the host and reads .item() per token"},
    }
    return out if rank == 0 else {}


# ------------------------------------------------------------------------------------ training
TRAIN_SEQ, TRAIN_BATCH_PER_GPU = 4096, 1


def train_config(model: str, world: int, seq: int, batch: int) -> dict:
    """The ``config`` dict of a training line: identical for every arm so that the lines can be compared."""
    from research_b200.models import get_preset

    cfg = get_preset(model)
    return {"model": (f"{model}-shaped ({cfg.num_layers}L d{cfg.hidden_size} {cfg.num_heads}q/{cfg.num_kv_heads}kv "
                      f"hd{cfg.head_dim} ffn{cfg.intermediate_size} vocab{cfg.vocab_size})"),
            "global_batch": batch * world, "seq_len": seq, "workload": "train", "parallelism": f"fsdp{world}",
            "batch_per_gpu": batch, "optimizer": "AdamW lr 1e-5 betas (0.9, 0.95), clip 1.0", "loss": "next-token cross-entropy",
            "activation_checkpointing": False,
            "l2": "inputs larger than L2 (every step streams 16 GB of weights and more of activations)"}


def train_flops_per_token(cfg, seq: int) -> float:
    """6 x matmul parameters + causal attention (12 L Hq D seq / 2 per token)."""
    d, L, F = cfg.hidden_size, cfg.num_layers, cfg.intermediate_size
    qkv = d * (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim
    matmul_params = L * (qkv + cfg.num_heads * cfg.head_dim * d + 3 * d * F) + cfg.vocab_size * d
    return 6.0 * matmul_params + 12.0 * L * cfg.num_heads * cfg.head_dim * seq / 2


def host_batches(cfg, rank: int, n: int, batch: int, seq: int):
    """``n`` different host-side token batches (uniform random ids, seeded per rank), the same for every arm. Every
    step of a run gets its own batch: a batch seen twice would be half memorised after one AdamW step of 8 B
    parameters, and the loss printed beside the timing would no longer say "random tokens"."""
    import torch

    g = torch.Generator().manual_seed(1234 + rank)
    out = []
    for _ in range(n):
        ids = torch.randint(0, cfg.vocab_size, (batch, seq), generator=g)
        out.append({"input_ids": ids, "labels": ids.clone(), "loss_mask": torch.ones(batch, seq)})
    return out


def selfcheck_fused(comm, dev) -> dict:
    """Each fused multi-GPU kernel of the training step, once, against a ``torch.distributed`` oracle.
    Returns ``{name: max abs error}``; raises on a mismatch."""
    import torch
    import torch.distributed as dist

    from research_b200.parallel.fsdp import FlatBuckets, ShardedAdamW
    from research_b200.parallel.tp import TensorParallel

    W, r = comm.world, comm.rank
    out = {}
    # (1) reduce-scatter + clip + AdamW + all-gather kernels vs all_reduce + torch.optim.AdamW
    shapes = [("a", (256, 512)), ("b", (512,)), ("c", (384, 256))]
    fb = FlatBuckets(comm, shapes, lambda n: {"a": 0, "b": 0, "c": 1}[n])
    g = torch.Generator().manual_seed(5)
    init = {n: torch.randn(sh, generator=g).bfloat16() for n, sh in shapes}
    for n, _ in shapes:
        fb.param_view(n).copy_(init[n])
    comm.barrier()
    opt = ShardedAdamW(fb, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0)
    ref = {n: init[n].float().to(dev).requires_grad_(True) for n, _ in shapes}
    ropt = torch.optim.AdamW(ref.values(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    err = 0.0
    for step in range(2):
        gr = torch.Generator().manual_seed(100 * step + r)
        mine = {n: (torch.randn(sh, generator=gr) * 0.5).bfloat16().to(dev) for n, sh in shapes}
        for n, _ in shapes:
            fb.grad_view(n).copy_(mine[n])
            avg = mine[n].float()
            dist.all_reduce(avg)
            ref[n].grad = avg / W
        opt.reduce_chunk(1, overlapped=True)
        norm = opt.step()
        ref_norm = torch.nn.utils.clip_grad_norm_(ref.values(), 1.0)
        ropt.step()
        err = max(err, abs(float(norm) - float(ref_norm)) / float(ref_norm))
        for n, _ in shapes:
            err = max(err, float((fb.param_view(n).float() - ref[n].detach()).abs().max()))
    assert err < 3e-2, f"selfcheck rs_reduce + adamw_allgather: error {err}"
    out["rs_reduce+clip+adamw_allgather"] = round(err, 5)
    # (2) fused GEMM + all-reduce vs matmul + all_reduce
    tp = TensorParallel(comm, max_rows=512, max_cols=1024)
    M, N, K = 256, 1024, 512
    ga = torch.Generator().manual_seed(7 + r)
    a = torch.randn(M, K, generator=ga).bfloat16().to(dev)
    w = (torch.randn(N, K, generator=ga) * 0.1).bfloat16().to(dev)
    x = tp.alloc((512, N), torch.bfloat16)
    x.zero_()
    comm.barrier()
    tp.gemm_all_reduce(a, w, x[:M])
    want = a.float() @ w.float().t()
    dist.all_reduce(want)
    torch.cuda.synchronize()
    err2 = float((x[:M].float() - want).abs().max())
    assert err2 < 0.5, f"selfcheck gemm_all_reduce: error {err2}"
    out["gemm_all_reduce"] = round(err2, 4)
    from research_b200.ops import check_status

    check_status(dev)
    comm.barrier_host()
    return out


def run_train(args) -> dict:
    import torch
    import torch.distributed as dist

    from research_b200.models import get_preset
    from research_b200.ops import check_status
    from research_b200.ops._util import LAUNCH_COUNT
    from research_b200.training.types import TrainerConfig
    from research_b200.utils.timing import ClockSampler

    rank, world, local = dist_setup(args.gpus)
    dev = torch.device(f"cuda:{local}")
    cfg = get_preset(args.model)
    seq, batch = args.seq, args.batch
    K, W = args.steps, max(args.warmup, 3)
    kw = dict(loss_fn="sft", lr=1e-5, trainer_config=TrainerConfig(micro_batch_size=args.micro_batch or batch),
              activation_checkpointing=False, need_entropy=False)
    checks = None
    if world > 1:
        from research_b200.parallel.symm import PeerComm
        from research_b200.training.backends.fsdp import FSDPConfig, FSDPTrainingBackend

        comm = PeerComm(device=dev)
        checks = selfcheck_fused(comm, dev)
        backend = FSDPTrainingBackend(cfg, None, comm=comm, device=dev,
                                      config=FSDPConfig(sharding_strategy=args.sharding), **kw)
    else:
        from research_b200.training.backends.native import NativeTrainingBackend

        backend = NativeTrainingBackend(cfg, None, device=dev, **kw)
    batches = host_batches(cfg, rank, W + K, batch, seq)
    dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in host_batches(cfg, rank + 7919, K + 2, batch, seq)]

    def e2e_step(i):
        m = backend.forward_backward(batches[i % len(batches)]).wait()      # pinned staging + H2D, loss read back
        o = backend.optim_step().wait()
        return m, o

    def dev_step(i):
        backend.forward_backward(dev_batches[i % len(dev_batches)]).wait()  # the batch is already on the device
        backend.optim_step(read_back=False).wait()

    for i in range(W):
        m, o = e2e_step(i)
    float(o["grad_norm"])
    sampler = ClockSampler(local).start()
    # ---- end to end through the public API ----
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(K):
        m, o = e2e_step(W + i)
    backend.buckets.finish_pending()       # the K-th step's parameter update (second stream) ends inside the timed region
    e1.record()
    barrier(world)
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world)
    h2d = backend.last_h2d_bytes
    d2h = 4 * (len(m) + 1)     # the scalars of the step's metrics and the gradient norm
    # ---- device-timed: same steps, inputs resident on the device ----
    for i in range(2):
        dev_step(i)
    barrier(world)
    l0 = LAUNCH_COUNT[0]
    e0.record()
    for i in range(K):
        dev_step(2 + i)
    backend.buckets.finish_pending()
    e1.record()
    barrier(world)
    dev_ms = max_over_ranks(e0.elapsed_time(e1), world)
    launches = LAUNCH_COUNT[0] - l0
    clocks = sampler.stop()
    check_status(dev)
    tokens = batch * seq * world
    value = tokens * K / (dev_ms * 1e-3)
    e2e = tokens * K / (e2e_ms * 1e-3)
    peak = args.peak_tflops * 1e12
    out = {
        "metric": "fsdp_train_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 (fp32 AdamW master weights and moments)",
        "data": "synthetic (uniform-random token ids, random-init weights)", "impl": "native",
        "config": train_config(args.model, world, seq, batch),
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / K, 3),
                "wall_ms_per_step": round(wall_ms / K, 3), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
        "mfu_of_sustained_cublas": round(value / world * train_flops_per_token(cfg, seq) / peak, 3),
        "loss": round(float(m.get("loss", 0.0)), 4), "grad_norm": round(float(o["grad_norm"]), 4),
        "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1),
        "sharding": getattr(getattr(backend, "fsdp_config", None), "sharding_strategy", "single"),
        "comm_overlap": bool(getattr(backend, "overlap_comm", False)),
    }
    if checks is not None:
        out["selfcheck"] = checks
    _ = dist
    if world == 1 and args.extras and args.model == "llama-3-8b":
        # the same shape's rollout decode rate, outside the timed region, in a child process (a failure there cannot
        # take this line with it): the trainer's memory goes back to the driver first
        del backend, batches, dev_batches, m, o
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        out["extras"] = _rollout_decode_extra(args.model)
    return out if rank == 0 else {}


def _rollout_decode_extra(model: str) -> dict:
    """``bench.py --workload rollout --model <model>`` on this GPU as a child process; its headline numbers, or why not."""
    import subprocess

    cmd = [sys.executable, os.path.abspath(__file__), "--workload", "rollout", "--model", model, "--steps", "100", "--warmup", "5"]
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        line = next((ln for ln in reversed(proc.stdout.splitlines()) if ln.startswith("{")), None)
        if proc.returncode != 0 or line is None:
            return {"rollout_decode": {"error": f"child exited {proc.returncode}: {(proc.stderr or proc.stdout)[-300:]}"}}
        d = json.loads(line)
        return {"rollout_decode": {"metric": d["metric"], "model": model, "tokens_per_s": d["value"], "ms_per_step": d["ms_per_step"],
                                   "e2e_tokens_per_s": d["e2e"]["value"], "batch": d["config"].get("global_batch"),
                                   "note": "measured after the timed region by `bench.py --workload rollout` in a child process"}}
    except Exception as e:   # noqa: BLE001 - an extra must never cost the headline
        return {"rollout_decode": {"error": f"{type(e).__name__}: {e}"[:300]}}


def _hf_llama(args, dev):
    """Random-init HF Llama of the benchmark shape in bf16 on ``dev`` (no checkpoint is read or written)."""
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM

    from research_b200.models import get_preset

    cfg = get_preset(args.model)
    hf = LlamaConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                     num_hidden_layers=cfg.num_layers, num_attention_heads=cfg.num_heads, num_key_value_heads=cfg.num_kv_heads,
                     head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta,
                     max_position_embeddings=cfg.max_position_embeddings, tie_word_embeddings=cfg.tie_word_embeddings,
                     attention_bias=cfg.attention_bias, attn_implementation="sdpa")
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaForCausalLM(hf).to(torch.bfloat16)
    return cfg, model


def _ce_full_logits(logits, batch):
    """Next-token cross-entropy over the full ``[B, T, V]`` logits (the reference's loss shape)."""
    import torch.nn.functional as F

    labels = batch["labels"][:, 1:]
    mask = batch["loss_mask"][:, 1:].to(logits.dtype)
    lp = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), labels.reshape(-1), reduction="none")
    return (lp * mask.reshape(-1).float()).sum() / mask.sum().clamp(min=1).float()


def _time_train_arm(args, step_fn, world, rank, local, impl, extra):
    """Warm-up, K timed steps between barriers (CUDA events, max over ranks), one JSON line."""
    import torch

    from research_b200.models import get_preset
    from research_b200.utils.timing import ClockSampler

    cfg = get_preset(args.model)
    K, W = args.steps, max(args.warmup, 3)
    batches = host_batches(cfg, rank, W + K, args.batch, args.seq)
    pinned = [{k: v.pin_memory() for k, v in b.items()} for b in batches]
    for i in range(W):
        last = step_fn(pinned[i])
    sampler = ClockSampler(local).start()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        last = step_fn(pinned[W + i])
    e1.record()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    clocks = sampler.stop()
    tokens = args.batch * args.seq * world
    value = tokens * K / (ms * 1e-3)
    h2d = sum(v.numel() * v.element_size() for v in batches[0].values())
    out = {"metric": "fsdp_train_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": K,
           "warmup": W, "ms_per_step": round(ms / K, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "bf16", "data": "synthetic (uniform-random token ids, random-init weights)", "impl": impl,
           "config": train_config(args.model, world, args.seq, args.batch),
           "e2e": {"value": round(value, 1), "unit": "tokens/s", "ms_per_step": round(ms / K, 3), "h2d_bytes_per_step": h2d,
                   "d2h_bytes_per_step": 8,
                   "note": "this arm's step is end to end already: the host batch is copied to the device and the loss read back every step"},
           "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
           "mfu_of_sustained_cublas": round(value / world * train_flops_per_token(cfg, args.seq) / (args.peak_tflops * 1e12), 3),
           "loss": round(float(last), 4), "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1)}
    out.update(extra)
    return out if rank == 0 else {}


def run_library_train(args) -> dict:
    """Same-box library baseline (not the reference package): HF Llama + FSDP2 ``fully_shard`` per decoder layer and
    at the root + ``torch.optim.AdamW`` + ``clip_grad_norm_`` + full-logits cross-entropy, in bf16 as the reference
    loads its model (rollouts/training/backends/fsdp.py:253-325, 327-479; dev/integration_training/train.py:134-276)."""
    import torch

    rank, world, local = dist_setup(args.gpus)
    dev = torch.device(f"cuda:{local}")
    cfg, model = _hf_llama(args, dev)
    if world > 1:
        from torch.distributed.fsdp import fully_shard

        for layer in model.model.layers:
            fully_shard(layer)
        fully_shard(model)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-5, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    model.train()

    def step(b):
        b = {k: v.to(dev, non_blocking=True) for k, v in b.items()}
        logits = model(input_ids=b["input_ids"]).logits
        loss = _ce_full_logits(logits, b)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
        return loss.item()

    return _time_train_arm(args, step, world, rank, local, "library",
                           {"library": "HF LlamaForCausalLM (sdpa) + torch.distributed.fsdp.fully_shard + torch.optim.AdamW, bf16 "
                                       "parameters, gradients and moments (no fp32 master copy)"})


def _install_trio_standin() -> bool:
    """The reference's training package imports ``trio`` at module level (``training/types.py``: a ``trio.Event`` inside
    its futures; type annotations elsewhere). The image has no trio. This registers a stand-in module with a working
    ``Event`` and placeholder classes for every other name, so that the UNMODIFIED package imports; the backend calls
    this arm times return already-completed futures and never touch it. Returns True if the stand-in was installed."""
    import asyncio
    import threading
    import types

    try:
        import trio  # noqa: F401

        return False
    except ImportError:
        pass

    class Event:
        def __init__(self):
            self._e = threading.Event()

        def set(self):
            self._e.set()

        def is_set(self):
            return self._e.is_set()

        async def wait(self):
            while not self._e.is_set():
                await asyncio.sleep(0)

    class _Missing:
        def __init__(self, *a, **k):
            raise RuntimeError("trio is not installed; this is an import-time stand-in")

    mod = types.ModuleType("trio")
    mod.Event = Event

    def _getattr(name):
        if name.startswith("__"):
            raise AttributeError(name)
        return type(name, (_Missing,), {})

    mod.__getattr__ = _getattr
    sys.modules["trio"] = mod
    return True


def run_reference_train(args) -> dict:
    """The reference's own ``FSDPTrainingBackend`` (unmodified, from ``baseline/_ref``) on a random-init HF Llama of
    the benchmark shape, driven through ``forward_backward`` / ``optim_step``."""
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "rollouts")):
        return {"impl": "reference", "unavailable": "baseline/_ref/rollouts is absent (reference not installed on this box)"}
    sys.path.insert(0, ref_dir)
    # --impl reference imports the reference as the image allows it: its training package imports trio at module level
    # and trio is not installed, so that arm reports itself unavailable. --impl reference-standin is a separate,
    # labelled context measurement: the same unmodified package imported with a stand-in for trio.Event.
    standin = _install_trio_standin() if args.impl == "reference-standin" else False
    try:
        from rollouts.training.backends.fsdp import FSDPConfig as RefFSDPConfig
        from rollouts.training.backends.fsdp import FSDPTrainingBackend as RefBackend
        from rollouts.training.losses import sft_loss as ref_sft_loss
    except Exception as e:
        return {"impl": args.impl, "unavailable":
                (f"reference training backend cannot be imported: {type(e).__name__}: {e} (rollouts/training/types.py imports trio, "
                 "which is neither in this image nor in its wheelhouse; same-box context: --impl library, --impl reference-standin)")[:400]}
    import tempfile

    import torch

    rank, world, local = dist_setup(args.gpus)
    dev = torch.device(f"cuda:{local}")
    if world == 1 and not torch.distributed.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        torch.distributed.init_process_group("nccl", rank=0, world_size=1)
    cfg, model = _hf_llama(args, dev)

    def loss_fn(logits, batch):
        # the reference's own SFT loss (it returns (loss, metrics); its FSDP backend wants the tensor)
        return ref_sft_loss(logits, batch)[0]

    backend = RefBackend(model=model, optimizer_fn=lambda m: torch.optim.AdamW(m.parameters(), lr=1e-5, betas=(0.9, 0.95)),
                         loss_fn=loss_fn, checkpoint_dir=__import__("pathlib").Path(tempfile.mkdtemp(prefix="ref_ckpt_")),
                         config=RefFSDPConfig(clip_grad=1.0))

    def resolve(fut):
        for name in ("wait", "result_sync"):
            if hasattr(fut, name):
                return getattr(fut, name)()
        return getattr(fut, "_result", None)

    def step(b):
        # the reference's losses take labels already shifted to the next token (-100 = ignore)
        ids = b["input_ids"]
        labels = torch.full_like(ids, -100)
        labels[:, :-1] = ids[:, 1:]
        mask = torch.zeros_like(b["loss_mask"])
        mask[:, :-1] = b["loss_mask"][:, 1:]
        m = resolve(backend.forward_backward({"input_ids": ids, "labels": labels, "loss_mask": mask}))
        resolve(backend.optim_step())
        return (m or {}).get("loss", 0.0)

    extra = {"engine": "rollouts.training.backends.fsdp.FSDPTrainingBackend (unmodified) on a random-init HF LlamaForCausalLM, "
                       "the reference's sft_loss, torch AdamW"}
    if standin:
        extra["import_note"] = ("trio is not in this image: a stand-in module provides trio.Event (used by the reference's futures) so that "
                                "the unmodified training package imports; the timed path never awaits it")
    return _time_train_arm(args, step, world, rank, local, args.impl, extra)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=["native", "reference", "library", "reference-standin"], default="native",
                    help="reference = the unmodified reference through its own API (unavailable for training where its imports "
                         "cannot be met); library = HF Llama + FSDP2 + torch AdamW driven by this script; reference-standin = the "
                         "reference's FSDP backend class imported with a stand-in for the missing trio module (context only)")
    ap.add_argument("--workload", choices=["train", "rollout", "serving"], default="train",
                    help="train = sharded training step on the Llama-3-8B shape, seq 4096, one sequence per GPU (the flagship); "
                         "rollout = engine decode, 1024 requests, prompts U[128,1024], 512 new tokens, batch 256; "
                         "serving = batch 64, prompts of 2048 tokens, 256 new tokens (the tensor-parallel serving case)")
    ap.add_argument("--model", default=None, help="model preset (default: llama-3-8b for train / serving, qwen2.5-0.5b for rollout)")
    ap.add_argument("--seq", type=int, default=TRAIN_SEQ, help="train: tokens per sequence")
    ap.add_argument("--batch", type=int, default=TRAIN_BATCH_PER_GPU, help="train: sequences per GPU per step")
    ap.add_argument("--micro-batch", type=int, default=0, help="train: sequences per forward/backward pass (0 = the whole batch)")
    ap.add_argument("--sharding", default="shard_optimizer_and_grads",
                    choices=["shard_optimizer_and_grads", "full_shard"],
                    help="train, N > 1: replicated bf16 parameters with sharded gradients / optimizer state, or parameters "
                         "sharded too (layer weights gathered from the peers inside the consuming GEMM launch)")
    ap.add_argument("--no-extras", dest="extras", action="store_false",
                    help="train, 1 GPU: skip the rollout-decode measurement of the same model that follows the timed region")
    ap.add_argument("--peak-tflops", type=float, default=1426.3, help="sustained cuBLAS bf16 TFLOP/s per GPU for the MFU figure")
    ap.add_argument("--ep", action="store_true", help="engine workloads, MoE models: data-parallel engines with the experts split over all GPUs")
    ap.add_argument("--tp", action="store_true", help="engine workloads: one tensor-parallel engine over all GPUs instead of replicas")
    args = ap.parse_args()
    if args.model is None:
        args.model = "qwen2.5-0.5b" if args.workload == "rollout" else "llama-3-8b"
    if args.workload == "train":
        args.steps = 10 if args.steps is None else args.steps
        args.warmup = 3 if args.warmup is None else args.warmup
        out = {"native": run_train, "reference": run_reference_train, "library": run_library_train,
               "reference-standin": run_reference_train}[args.impl](args)
    else:
        if args.impl in ("library", "reference-standin"):
            out = {"impl": args.impl, "unavailable": "this arm exists for the train workload only"}
        else:
            if args.impl == "native":
                set_workload(args.workload)
            if args.steps is None:
                args.steps = 200 if args.impl == "native" else 3
            if args.warmup is None:
                args.warmup = 10 if args.impl == "native" else 3
            out = run_engine(args) if args.impl == "native" else run_reference_engine(args)
    if out and ("unavailable" not in out or int(os.environ.get("RANK", "0")) == 0):    # ONE line per job, also when an arm bows out on every rank
        print(json.dumps(out), flush=True)
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


if __name__ == "__main__":
    main()
