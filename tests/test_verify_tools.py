"""The functional-vs-module verification tools, run against tiny random-init Hugging Face models on CPU: this is
also the parity check of this package's oracle (``models.functional``) with the Hugging Face implementations."""

import pytest
import torch

transformers = pytest.importorskip("transformers")

from research_b200.models.config import ModelConfig  # noqa: E402
from research_b200.models.functional import decoder_layer_forward, rope_cos_sin  # noqa: E402
from research_b200.models.verify_tools import (DebugSession, FunctionalModelTestSuite, build_verification_script,  # noqa: E402
                                               capture_internals, compare_tensors, format_comparison, format_layer_report,
                                               native_functional_forward, per_position_diff, quick_debug, verify_functional)


def _tiny(kind: str):
    torch.manual_seed(0)
    common = dict(vocab_size=320, hidden_size=64, intermediate_size=112, num_hidden_layers=3, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=1e4, attn_implementation="eager")
    if kind == "llama":
        cfg = transformers.LlamaConfig(tie_word_embeddings=False, **common)
        model = transformers.LlamaForCausalLM(cfg)
    else:
        cfg = transformers.Qwen2Config(tie_word_embeddings=True, **common)
        model = transformers.Qwen2ForCausalLM(cfg)
    model = model.float().eval()
    weights = {k: v.detach() for k, v in model.state_dict().items()}
    mc = ModelConfig.from_hf_dict(cfg.to_dict())
    return model, weights, mc


def test_compare_helpers():
    a = torch.zeros(2, 3, 4)
    b = a.clone()
    b[1, 2, 3] = 0.5
    c = compare_tensors(a, b, "x", 0.0, 1e-3)
    assert not c["matches"] and c["max_diff"] == 0.5 and c["max_diff_pos"] == (1, 2, 3) and "DIFFERS" in format_comparison(c)
    assert compare_tensors(a, torch.zeros(2, 3), "y")["max_diff"] == float("inf")
    pp = per_position_diff(a, b, torch.tensor([[1, 1, 1], [1, 1, 0]]))
    assert pp[2]["max_diff"] == 0.5 and pp[2]["is_padding"] and not pp[0]["is_padding"]


@pytest.mark.parametrize("kind", ["llama", "qwen2"])
def test_battery_passes_for_the_oracle_against_hf(kind):
    model, weights, mc = _tiny(kind)
    res = verify_functional(f"tiny-{kind}", reference_model=model, tolerance=2e-4)
    assert res.passed, "\n".join(f"{r['name']}: {r['max_diff']} {r['details']}" for r in res.suite["results"] if not r["passed"])
    names = [r["name"] for r in res.suite["results"]]
    assert "mask: left padding" in names and "seq_len=128" in names and "dtype=bfloat16" in names and len(names) >= 18


def test_debug_session_finds_the_broken_layer():
    model, weights, mc = _tiny("llama")
    fwd = native_functional_forward(mc)
    ids = torch.randint(0, 320, (2, 10))
    s = DebugSession(model, fwd, weights)
    assert s.test_embeddings(ids)["matches"]
    rope = s.test_position_embeddings(ids, lambda pos: rope_cos_sin(pos, mc.head_dim, mc.rope_theta, torch.float32))
    assert rope["matches"] and rope["position_ids"] == list(range(10))
    assert s.compare_full_forward(ids, rtol=1e-4, atol=2e-4)["matches"]
    cap = capture_internals(model, ids)
    assert sorted(cap.layer_outputs) == [0, 1, 2] and cap.embeddings.shape == (2, 10, 64) and cap.logits.shape == (2, 10, 320)

    def layer_fn(hidden, w, idx, cos, sin, mask):
        pos = torch.arange(hidden.shape[1])[None].expand(hidden.shape[0], -1)
        return decoder_layer_forward(hidden, w, idx, mc, pos)

    clean = s.find_divergence_layer(ids, layer_forward_fn=layer_fn, threshold=2e-4)
    assert clean["divergence_layer"] is None and clean["num_layers"] == 3
    broken = dict(weights)
    broken["model.layers.1.mlp.down_proj.weight"] = weights["model.layers.1.mlp.down_proj.weight"] * 1.5
    bad = DebugSession(model, fwd, broken).find_divergence_layer(ids, layer_forward_fn=layer_fn, threshold=2e-4)
    assert bad["divergence_layer"] == 1 and bad["per_layer_diff"][0]["matches"] and bad["per_layer_diff"][2]["matches"]
    assert "first divergence: 1" in format_layer_report(bad)
    qd = quick_debug(model, fwd, broken, ids, layer_forward_fn=layer_fn)
    assert not qd["full"]["matches"] and qd["layers"]["divergence_layer"] == 1
    mask = torch.ones(2, 10, dtype=torch.long)
    mask[1, :3] = 0
    padded = s.compare_full_forward(ids, mask, rtol=1e-4, atol=2e-4)
    assert padded["max_diff_unpadded"] < 2e-4


def test_suite_reports_failures_and_remote_path():
    model, weights, mc = _tiny("qwen2")
    wrong = lambda ids, w, attention_mask=None: native_functional_forward(mc)(ids, w, attention_mask) + 0.01  # noqa: E731
    suite = FunctionalModelTestSuite("off-by-a-bit", model, wrong, weights, 320, tolerance=1e-4)
    suite.test_sequence_lengths((4, 8))
    suite.run_case("crashes", torch.zeros(1, 4, dtype=torch.long), weights={})
    assert [r.passed for r in suite.results] == [False, False, False] and "KeyError" in suite.results[2].details

    class FakeRemote:
        def __init__(self):
            self.pushed, self.cmds = [], []

        def push(self, d):
            self.pushed.append(d)

        def exec(self, cmd):
            self.cmds.append(cmd)
            return 0, 'noise\n{"model": "m", "all_passed": true, "seconds": 1.0, "results": []}\n'

    r = FakeRemote()
    res = verify_functional("org/model", remote=r, workdir="/src")
    assert res.passed and res.where == "remote" and r.pushed == ["/src"] and "verify_functional" in r.cmds[0]
    assert "org/model" in build_verification_script("org/model")
    r.exec = lambda cmd: (1, "Traceback ...")
    assert not verify_functional("org/model", remote=r).passed
