"""HTTP front end of the engine on CPU: concurrent requests share batches; weight updates drain first."""

import torch
from fastapi.testclient import TestClient

from research_b200.inference import EngineConfig, InferenceEngine
from research_b200.inference.server import EngineService, create_app
from research_b200.inference.types import SamplingParams
from research_b200.models import get_preset, init_random_weights


def _engine():
    cfg = get_preset("tiny-qwen2")
    w = init_random_weights(cfg, seed=0)
    return cfg, w, InferenceEngine(EngineConfig(max_batch_size=8, max_model_len=128, num_kv_blocks=64, use_cuda_graphs=False),
                                   cfg, w, device="cpu")


def test_service_batches_concurrent_requests():
    cfg, w, eng = _engine()
    svc = EngineService(eng)
    try:
        futs = [svc.submit([1 + i, 2, 3, 4], SamplingParams(temperature=0.0, max_tokens=6)) for i in range(5)]
        samples = [f.result(timeout=120) for f in futs]
        assert all(len(s.completion_tokens) == 6 for s in samples)
        assert svc.steps < 5 * 7, "requests must share engine steps"
        # the service thread owns the engine: a later request alone gives the same greedy tokens
        ref = svc.submit([1, 2, 3, 4], SamplingParams(temperature=0.0, max_tokens=6)).result(timeout=120)
        assert samples[0].completion_tokens == ref.completion_tokens
    finally:
        svc.shutdown()


def test_http_endpoints(tmp_path):
    cfg, w, eng = _engine()
    svc = EngineService(eng)
    try:
        client = TestClient(create_app(svc, "tiny"))
        assert client.get("/health").json() == {"status": "ok"}
        r = client.post("/generate", json={"input_ids": [5, 6, 7], "sampling_params": {"temperature": 0.0, "max_new_tokens": 4},
                                           "return_logprob": True}).json()
        assert len(r["output_ids"]) == 4 and len(r["meta_info"]["output_token_logprobs"]) == 4
        assert r["meta_info"]["finish_reason"]["type"] == "length"
        rb = client.post("/generate", json={"input_ids": [[5, 6, 7], [8, 9]], "sampling_params": {"max_new_tokens": 3}}).json()
        assert isinstance(rb, list) and len(rb) == 2
        c = client.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 4, "temperature": 0.0, "logprobs": 1}).json()
        assert c["choices"][0]["token_ids"] == r["output_ids"] and len(c["choices"][0]["logprobs"]["token_logprobs"]) == 4
        assert client.post("/v1/completions", json={"prompt": "text without tokenizer"}).status_code == 400
        # weight update from a checkpoint on disk changes the output and bumps the version
        w2 = init_random_weights(cfg, seed=1)
        torch.save(w2, tmp_path / "pytorch_model.bin")
        u = client.post("/update_weights_from_disk", json={"model_path": str(tmp_path)}).json()
        assert u["success"] and u["weight_version"] == 1
        r2 = client.post("/generate", json={"input_ids": [5, 6, 7], "sampling_params": {"temperature": 0.0, "max_new_tokens": 4}}).json()
        assert r2["meta_info"]["weight_version"] == 1 and r2["output_ids"] != r["output_ids"]
        assert client.post("/update_weights_from_disk", json={"model_path": str(tmp_path / "nope")}).status_code == 404
        # the layout the training backend writes: a safetensors directory with config.json
        from research_b200.models.weights import save_safetensors_dir

        st_dir = tmp_path / "st_ckpt"
        save_safetensors_dir(init_random_weights(cfg, seed=2), cfg, st_dir)
        u3 = client.post("/update_weights_from_disk", json={"model_path": str(st_dir)})
        assert u3.status_code == 200 and u3.json()["weight_version"] == 2, u3.text
        r3 = client.post("/generate", json={"input_ids": [5, 6, 7], "sampling_params": {"temperature": 0.0, "max_new_tokens": 4}}).json()
        assert r3["meta_info"]["weight_version"] == 2 and r3["output_ids"] != r2["output_ids"]
        assert client.post("/flush_cache").json()["success"]
        info = client.get("/get_server_info").json()
        assert info["weight_version"] == 2 and info["running"] == 0
    finally:
        svc.shutdown()
