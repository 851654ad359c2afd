"""Two gloo ranks share one tensor-parallel engine; rank 0 submits requests, rank 1 follows."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from research_b200.inference import EngineConfig, InferenceEngine  # noqa: E402
from research_b200.inference.server import LockstepEngineService  # noqa: E402
from research_b200.inference.types import SamplingParams  # noqa: E402
from research_b200.models import get_preset, init_random_weights  # noqa: E402
from research_b200.parallel.symm import PeerComm  # noqa: E402
from research_b200.parallel.tp import TensorParallel  # noqa: E402

dist.init_process_group("gloo")
rank = dist.get_rank()
dev = torch.device("cpu")
cfg = get_preset("tiny-qwen2", num_layers=2)
w = init_random_weights(cfg, seed=0)
tp = TensorParallel(PeerComm(device=dev), max_rows=512, max_cols=1024)
ecfg = EngineConfig(max_batch_size=16, max_model_len=128, num_kv_blocks=64, use_cuda_graphs=False, ignore_eos=True)
eng = InferenceEngine(ecfg, cfg, w, device=dev, tp=tp)
svc = LockstepEngineService(eng)
if rank == 0:
    futs = [svc.submit([3 + i, 4, 5, 6], SamplingParams(temperature=0.0, max_tokens=5)) for i in range(3)]
    outs = [f.result(timeout=180) for f in futs]
    late = svc.submit([9, 9, 9], SamplingParams(temperature=0.0, max_tokens=3)).result(timeout=180)
    solo = InferenceEngine(EngineConfig(max_batch_size=16, max_model_len=128, num_kv_blocks=64, use_cuda_graphs=False, ignore_eos=True),
                           cfg, w, device=dev)
    ref = solo.generate([[3, 4, 5, 6]], SamplingParams(temperature=0.0, max_tokens=5))[0]
    assert outs[0].completion_tokens == ref.completion_tokens, (outs[0].completion_tokens, ref.completion_tokens)
    assert len(late.completion_tokens) == 3 and svc.steps > 0
    # a weight update and a cache flush go through the same broadcast: every rank swaps its shards at the same step
    import tempfile

    from research_b200.models.weights import save_safetensors_dir

    w2 = init_random_weights(cfg, seed=1)
    with tempfile.TemporaryDirectory() as d:
        save_safetensors_dir(w2, cfg, d)
        assert svc.update_weights_from_path(d) == 1
    svc.flush_cache()
    after = svc.submit([3, 4, 5, 6], SamplingParams(temperature=0.0, max_tokens=5)).result(timeout=180)
    solo.update_weights(w2)
    solo.flush_cache()
    ref2 = solo.generate([[3, 4, 5, 6]], SamplingParams(temperature=0.0, max_tokens=5))[0]
    assert after.completion_tokens == ref2.completion_tokens, (after.completion_tokens, ref2.completion_tokens)
    assert after.weight_version == 1
    svc.shutdown()
    print("LOCKSTEP_OK", flush=True)
else:
    svc.follow()
    assert svc.steps > 0
dist.barrier()
dist.destroy_process_group()
