"""Headline benchmark: rollout decode throughput (tokens/s) of the inference engine.

Config (BASELINE.json, "Qwen2.5-0.5B-shaped inference engine throughput, bf16, data-parallel
replicas at 1/2/4/8 GPUs"): 24 layers, d 896, 14 query / 2 KV heads (head_dim 64), ffn 4864,
vocab 151936, random init; 1024 requests per replica with prompt lengths uniform in [128,1024]
of random token ids, 50% sharing one 512-token prefix; 512 output tokens each; temperature 1.0
from seed 0; CUDA-graph decode.

A "step" is one ``InferenceEngine.step()`` in steady state (the continuous batch is full: 256
running sequences per replica, each step produces one token per running sequence). The engine
is first ramped (untimed) until the running batch is full, then W warm-up steps, then exactly K
timed steps between barrier + synchronize, device-timed with CUDA events, MAX over ranks.

  value      : device time of the K decode steps replayed back to back (kernel-only)
  e2e.value  : the same K steps through the public ``engine.step()`` call, including every
               step's host->device copy of its inputs (token ids, positions, slots, sequence
               lengths, temperatures, seeds, block tables) from pinned memory and the
               device->host read of the sampled tokens and log-probabilities

``--impl reference`` runs the unmodified reference engine (rollouts.inference.InferenceEngine,
HF transformers model, no KV cache) on the same model shape and workload through its own
``add_request`` / ``step`` API.
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


# ------------------------------------------------------------------------------------ native arm
def run_native(args) -> dict:
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
        "config": {"model": (f"{args.model}-shaped ({cfg.num_layers}L d{cfg.hidden_size} {cfg.num_heads}q/{cfg.num_kv_heads}kv "
                             f"hd{cfg.head_dim} ffn{cfg.intermediate_size} vocab{cfg.vocab_size})"),
                   "global_batch": MAX_BATCH * replicas, "seq_len": SEQ_DESC, "workload": args.workload,
                   "parallelism": f"dp{world}+ep{world}" if ep is not None else f"dp{world}" if tp is None else f"tp{world}",
                   "requests_per_replica": N_REQUESTS, "temperature": 1.0,
                   "cuda_graph_decode": True, "kv_cache": "paged, radix prefix reuse",
                   "l2": "inputs larger than L2 (weights + KV read per step exceed 126 MB)"},
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


def run_reference(args) -> dict:
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
        "config": {"model": "qwen2.5-0.5b-shaped via HF transformers", "global_batch": MAX_BATCH * world,
                   "parallelism": f"dp{world}", "requests_per_replica": N_REQUESTS,
                   "engine": "rollouts.inference.InferenceEngine (unmodified; no KV cache, one sequence per forward)"},
        "e2e": {"value": round(value, 2), "unit": "tokens/s",
                "note": "the reference's step() is already end to end: it builds inputs on the host and reads .item() per token"},
    }
    return out if rank == 0 else {}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--model", default="qwen2.5-0.5b", help="model preset of the native arm (the flagship is the default)")
    ap.add_argument("--ep", action="store_true", help="native arm, MoE models: data-parallel engines with the experts split over all GPUs")
    ap.add_argument("--workload", choices=["rollout", "serving"], default="rollout",
                    help="native arm: rollout = 1024 requests, prompts U[128,1024], 512 new tokens, batch 256 (the flagship); "
                         "serving = batch 64, prompts of 2048 tokens, 256 new tokens (the tensor-parallel serving case)")
    ap.add_argument("--tp", action="store_true", help="native arm: one tensor-parallel engine over all GPUs instead of replicas")
    args = ap.parse_args()
    if args.impl == "native":
        set_workload(args.workload)
    if args.steps is None:
        args.steps = 200 if args.impl == "native" else 3
    if args.warmup is None:
        args.warmup = 10 if args.impl == "native" else 3
    out = run_native(args) if args.impl == "native" else run_reference(args)
    if out:
        print(json.dumps(out), flush=True)
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


if __name__ == "__main__":
    main()
