"""CPU tests of the training stack: losses (with the next-token shift), data buffer, filters,
rollout manager, backends, checkpoints and the full GRPO loop on the tiny Qwen2-style model."""

import asyncio
import json

import pytest
import torch

from research_b200.models import causal_lm_forward, get_preset, init_random_weights
from research_b200.training import losses as L
from research_b200.training.backends import PyTorchTrainingBackend, create_pytorch_backend, parse_dtype, warmup_cosine
from research_b200.training.datasets import BufferState, DataBuffer, get_samples, load_samples_from_jsonl, load_samples_from_list
from research_b200.training.filters import (check_any_success, check_quality_and_diversity, check_reward_nonzero_std,
                                            make_length_filter, make_threshold_filter)
from research_b200.training.grpo import GRPOConfig, grpo_train
from research_b200.training.loops import collate_batch, prepare_grpo_batch, prepare_sft_batch, run_sft_training
from research_b200.training.metrics import CompositeLogger, JSONLLogger, compute_stats_from_jsonl
from research_b200.training.rollout_gen import AsyncRolloutManager, convert_to_batch
from research_b200.training.types import (ImmediateTrainFuture, RolloutConfig, Sample, SFTTrainingConfig, Status,
                                          TrainerConfig, TrainFuture)


def test_group_advantages():
    adv = L.compute_group_advantages([1.0, 0.0, 1.0, 1.0], [0, 0, 1, 1])
    assert torch.allclose(adv, torch.tensor([0.5, -0.5, 0.0, 0.0]))
    adv = L.compute_group_advantages([2.0, 0.0], [0, 0], normalize_std=True)
    assert torch.allclose(adv, torch.tensor([0.7071, -0.7071]), atol=1e-3)


def test_losses_use_next_token_targets():
    torch.manual_seed(0)
    V = 7
    labels = torch.tensor([[1, 2, 3, 4]])
    mask = torch.tensor([[0.0, 1.0, 1.0, 1.0]])
    logits = torch.randn(1, 4, V)
    loss, m = L.sft_loss(logits, {"labels": labels, "loss_mask": mask})
    lp = torch.log_softmax(logits, -1)
    want = -(lp[0, 0, 2] + lp[0, 1, 3] + lp[0, 2, 4]) / 3  # position t is scored against token t+1
    assert torch.allclose(loss, want, atol=1e-6)
    assert m["num_tokens"] == 3
    seq = L.get_seq_logprobs(logits, labels, mask)
    assert torch.allclose(seq, -want.unsqueeze(0), atol=1e-6)


def test_grpo_variants_and_from_logprobs_agree():
    torch.manual_seed(1)
    logits = torch.randn(4, 6, 11, requires_grad=True)
    batch = {"labels": torch.randint(0, 11, (4, 6)), "loss_mask": (torch.rand(4, 6) > 0.3).float(),
             "advantages": torch.tensor([0.5, -0.5, 1.0, -1.0]), "old_logprobs": torch.full((4,), -2.4)}
    for fn in (L.grpo_loss, L.grpo_loss_clipped, L.grpo_loss_masked):
        loss, metrics = fn(logits, batch)
        assert torch.isfinite(loss) and "pg_loss" in metrics and "entropy" in metrics
        loss.backward()
    # on-policy: clipped loss gradient equals vanilla when ratio == 1
    b = L._with_shift(batch)
    lp = L.get_per_token_logprobs(logits, b["targets"])
    seq = L.seq_mean(lp, b["shift_mask"]).detach()
    l1, _ = L.grpo_from_logprobs(lp, None, b)
    l2, m2 = L.grpo_clipped_from_logprobs(lp, None, {**b, "old_logprobs": seq})
    g1 = torch.autograd.grad(l1, lp, retain_graph=True)[0]
    g2 = torch.autograd.grad(l2, lp, retain_graph=True)[0]
    assert torch.allclose(g1, g2, atol=1e-6) and m2["clipfrac"] == 0.0
    assert abs(float(L.compute_entropy(torch.zeros(1, 2, 8))) - torch.log(torch.tensor(8.0)).item()) < 1e-5


def test_data_buffer_deterministic_epochs_and_groups(tmp_path):
    samples = load_samples_from_list(["a", "b", "c"])
    g1, s1 = get_samples(samples, BufferState(seed=3), 2, 4)
    g2, _ = get_samples(samples, BufferState(seed=3), 2, 4)
    assert [g[0].prompt for g in g1] == [g[0].prompt for g in g2] and len(g1[0]) == 4
    assert all(s.group_index == 1 for s in g1[1]) and s1.sample_offset == 2
    _, s2 = get_samples(samples, s1, 2, 1)
    assert s2.epoch_id == 1 and s2.sample_offset == 1
    buf = DataBuffer(["p0", "p1", "p2"], seed=1)
    first = buf.get_prompts(2)
    st = buf.save_state()
    nxt = buf.get_prompts(2)
    buf.load_state(st)
    assert buf.get_prompts(2) == nxt and sorted(first + nxt[:1]) == ["p0", "p1", "p2"]
    p = tmp_path / "d.jsonl"
    p.write_text('{"prompt": "x", "answer": "1"}\n{"prompt": "y", "answer": "2"}\n')
    js = load_samples_from_jsonl(p)
    assert js[1].prompt == "y" and js[1].ground_truth == "2"


def test_filters():
    g = [Sample(reward=1.0, tokens=[1, 2, 3], response_length=2), Sample(reward=0.0, tokens=[1, 5, 6], response_length=2)]
    assert check_reward_nonzero_std(g) and check_any_success(g) and check_quality_and_diversity(g)
    assert not check_reward_nonzero_std([g[0], g[0]])
    assert make_threshold_filter(0.5)(g) and not make_threshold_filter(2.0)(g)
    assert make_length_filter(1, 4)(g) and not make_length_filter(3, 4)(g)


def test_sample_roundtrip_and_futures():
    s = Sample(id="1", prompt="p", tokens=[1, 2], loss_mask=[0, 1], reward=0.5, status=Status.COMPLETED, rollout_log_probs=[-0.1])
    s2 = Sample.from_dict(json.loads(json.dumps(s.to_dict())))
    assert s2.tokens == [1, 2] and s2.status == Status.COMPLETED and s2.reward == 0.5
    f = TrainFuture("x")
    assert not f.done()
    f.set_result(3)
    assert f.done() and f.wait() == 3 and asyncio.run(f.result()) == 3
    assert asyncio.run(ImmediateTrainFuture(4).result()) == 4
    with pytest.raises(AssertionError):
        TrainerConfig(micro_batch_size=2, num_minibatches=2)
    assert TrainerConfig(micro_batch_size=2).get_num_minibatches(8) == 4


def test_async_rollout_manager_oversampling_filter_and_state():
    calls = []

    def gen(prompts, **kw):
        calls.append(len(prompts))
        return [Sample(prompt=p, tokens=[1, 2, 3 + i], loss_mask=[0, 1, 1], response_length=2, rollout_log_probs=[-1.0, -1.0])
                for i, p in enumerate(prompts)]

    def score(s):
        return float(s.tokens[-1] % 2)

    cfg = RolloutConfig(batch_size=2, n_samples_per_prompt=2, over_sampling_factor=1.5, generate_fn=gen, score_fn=score,
                        filter_fn=check_reward_nonzero_std)
    mgr = AsyncRolloutManager(DataBuffer(["a", "b", "c", "d"], seed=0), cfg)
    batch = asyncio.run(mgr.generate_batch())
    assert len(batch) == 4 and batch.group_indices == [0, 0, 1, 1] and batch.rollout_log_probs is not None
    assert batch.response_lengths == [2, 2, 2, 2]
    st = mgr.state_dict()
    mgr2 = AsyncRolloutManager(DataBuffer(["a", "b", "c", "d"], seed=0), cfg)
    mgr2.load_state_dict(json.loads(json.dumps(st)))
    assert len(mgr2.partial_samples) == len(mgr.partial_samples)
    assert len(convert_to_batch(batch.samples)) == 4


def test_batch_preparation():
    samples = [Sample(tokens=[1, 2, 3, 4], loss_mask=[0, 0, 1, 1]), Sample(tokens=[5, 6], loss_mask=[0, 1])]
    b = collate_batch(samples)
    assert b["input_ids"].shape == (2, 4) and b["loss_mask"][1].tolist() == [0, 1, 0, 0] and b["attention_mask"][1].tolist() == [1, 1, 0, 0]
    p = prepare_sft_batch(samples)
    assert p["input_ids"].shape == (1, 6) and p["cu_seqlens"].tolist() == [0, 4, 6] and p["position_ids"][0].tolist() == [0, 1, 2, 3, 0, 1]
    rb = convert_to_batch([Sample(tokens=[1, 2, 3], loss_mask=[0, 1, 1], rollout_log_probs=[-1.0, -3.0], reward=1.0, group_index=0)])
    g = prepare_grpo_batch(rb, torch.tensor([0.5]), max_seq_len=8)
    assert g["old_logprobs"].tolist() == [-2.0] and g["advantages"].tolist() == [0.5]


def test_metrics_loggers(tmp_path):
    lg = CompositeLogger([JSONLLogger(tmp_path), JSONLLogger(tmp_path, filename="b.jsonl", max_lines=1)])
    lg.log({"loss": 1.0, "bad": float("nan")}, 0)
    lg.log({"loss": 0.5}, 1)
    lg.finish()
    st = compute_stats_from_jsonl(tmp_path / "metrics.jsonl")
    assert st["loss"]["last"] == 0.5 and st["loss"]["count"] == 2
    assert len((tmp_path / "b.jsonl").read_text().splitlines()) == 1


def test_backend_gradients_match_autograd_oracle():
    cfg = get_preset("tiny-qwen2", num_layers=2)
    w = init_random_weights(cfg, seed=0)
    be = PyTorchTrainingBackend(cfg, w, device="cpu", loss_fn="ce", lr=1e-3, trainer_config=TrainerConfig(micro_batch_size=1))
    ids = torch.randint(0, cfg.vocab_size, (2, 12))
    m = be.forward_backward({"input_ids": ids, "labels": ids}).wait()
    leaves = {k: v.clone().requires_grad_(True) for k, v in w.items()}
    logits = causal_lm_forward(ids, leaves, cfg)
    ref, _ = L.sft_loss(logits, {"labels": ids})
    # micro-batches of 1: mean of per-sequence means == ref here because both rows have equal token counts
    ref.backward()
    assert abs(m["loss"] - float(ref)) < 1e-4
    for n in ("model.layers.1.mlp.down_proj.weight", "model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.bias"):
        assert torch.allclose(be.buckets.grad_view(n), leaves[n].grad, atol=1e-5), n
    o = be.optim_step().wait()
    assert o["step"] == 1 and o["grad_norm"] > 0 and float(be.buckets.grads.abs().sum()) == 0.0


def test_backend_sft_loop_checkpoint_resume(tmp_path):
    cfg = get_preset("tiny-qwen2", num_layers=1)
    be = PyTorchTrainingBackend(cfg, device="cpu", loss_fn="sft", lr=1e-2, checkpoint_dir=tmp_path, lr_schedule=warmup_cosine(2, 10))
    g = torch.Generator().manual_seed(0)
    samples = [Sample(tokens=torch.randint(0, cfg.vocab_size, (16,), generator=g).tolist(), loss_mask=[0.0] * 4 + [1.0] * 12) for _ in range(4)]
    hist = asyncio.run(run_sft_training(be, samples, SFTTrainingConfig(num_steps=6, batch_size=4, log_every=1, checkpoint_every=3),
                                        JSONLLogger(tmp_path)))
    assert hist[-1]["loss"] < hist[0]["loss"]
    ck = tmp_path / "step_0006"
    assert (ck / "model.safetensors").exists() and (ck / "config.json").exists() and (ck / "metadata.json").exists()
    be2 = PyTorchTrainingBackend(cfg, device="cpu", loss_fn="sft", lr=1e-2, seed=5)
    meta = be2.load_checkpoint(ck)
    assert meta["step"] == 6 and be2.current_step == 6 and be2.weight_version == be.weight_version
    assert torch.equal(be2.buckets.params, be.buckets.params)
    assert torch.equal(be2.optimizer.exp_avg[0], be.optimizer.exp_avg[0]) and be2.optimizer.step_count == 6
    snap = be2.get_state_snapshot()
    assert snap["step"] == 6 and not snap["poisoned"]
    with pytest.raises(Exception):
        be2.forward_backward({"input_ids": torch.full((1, 4), cfg.vocab_size + 5)})
    with pytest.raises(AssertionError):
        be2.forward_backward({"input_ids": torch.zeros(1, 4, dtype=torch.long)})  # poisoned after a failure
    assert parse_dtype("bf16") == torch.bfloat16
    be3 = create_pytorch_backend("tiny-llama", device="cpu", loss_fn="ce", lr=1e-3)
    assert be3.model_config.family == "llama"


def test_grpo_train_end_to_end(tmp_path):
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, 4096, (24,), generator=g).tolist()
    prompts = []
    for i in range(8):
        n = int(torch.randint(30, 64, (1,), generator=g))
        p = torch.randint(0, 4096, (n,), generator=g).tolist()
        prompts.append(shared + p[24:] if i < 4 else p)

    def score(s):
        return float(sum(s.tokens[-s.response_length:]) % 2)

    cfg = GRPOConfig(model_name="tiny-qwen2", lr=1e-5, batch_size=2, n_samples_per_prompt=4, num_minibatches=2, max_tokens=6,
                     max_seq_len=128, temperature=1.0, num_steps=2, output_dir=str(tmp_path), checkpoint_every=2,
                     max_batch_size=8, kv_blocks=128, experiment_name="t")
    hist = grpo_train(cfg, prompts, score, device="cpu")
    assert len(hist) == 2 and hist[1]["weight_version"] == 2.0 and all("pg_loss" in h for h in hist)
    run = next(tmp_path.iterdir())
    assert {"config.json", "metrics.jsonl", "rollouts.jsonl", "checkpoints", "rollout_state.json"} <= {p.name for p in run.iterdir()}
    assert len((run / "rollouts.jsonl").read_text().splitlines()) == 16


def test_polar_express_and_muon_cpu():
    from research_b200.training.muon import Muon, polar_express, polar_express_reference

    g = torch.Generator().manual_seed(0)
    G = torch.randn(24, 40, generator=g)
    X = polar_express(G).float()
    ref = polar_express_reference(G)
    assert (X - ref).abs().max() < 0.08                                   # bf16 iteration vs fp32
    s = torch.linalg.svdvals(ref)
    assert s.min() > 0.6 and s.max() < 1.25                               # singular values pushed towards 1
    tall = polar_express(torch.randn(40, 24, generator=g))
    assert tall.shape == (40, 24)
    w = torch.nn.Parameter(torch.randn(16, 32, generator=g))
    opt = Muon([w], lr=0.1, momentum=0.9, weight_decay=0.01)
    target = torch.randn(16, 32, generator=g)
    losses = []
    for _ in range(30):
        opt.zero_grad()
        loss = ((w - target) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.5 * losses[0]


class _ToyChatTokenizer:
    """Character-level tokenizer with a prefix-stable chat template: <role>text\\n per message."""

    def encode(self, text, add_special_tokens=False):
        return [ord(c) for c in text]

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=False):
        text = "".join(f"<{m['role']}>{m['content']}\n" for m in messages) + ("<assistant>" if add_generation_prompt else "")
        return self.encode(text) if tokenize else text


def test_sft_dataset_preparation(tmp_path):
    import json

    from research_b200.training.datasets.sft import (export_samples_to_jsonl, load_rl_prompts, load_samples_from_export,
                                                     load_sft_dataset, tokenize_conversation)

    tok = _ToyChatTokenizer()
    conv = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"},
            {"role": "user", "content": "bye"}, {"role": "assistant", "content": "ciao"}]
    ids, spans = tokenize_conversation(tok, conv)
    assert [r for _, _, r in spans] == ["system", "user", "assistant", "user", "assistant"] and spans[-1][1] == len(ids)
    rows = [{"messages": conv}, {"conversations": [{"from": "human", "value": "q"}, {"from": "gpt", "value": "a"}]},
            {"prompt": "2+2?", "response": "4"}, {"messages": [{"role": "user", "content": "no answer"}]}]
    p = tmp_path / "sft.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in rows))
    samples = load_sft_dataset(p, tok, max_length=200)
    assert len(samples) == 3
    s = samples[0]
    text = "".join(chr(t) for t, m in zip(s.tokens, s.loss_mask) if m)
    assert text == "<assistant>hello\n<assistant>ciao\n" and s.response_length == len(text)
    assert len(load_sft_dataset(rows, tok, max_length=30, skip_too_long=True)) == 2
    export_samples_to_jsonl(samples, tmp_path / "out.jsonl")
    back = load_samples_from_export(tmp_path / "out.jsonl")
    assert back[0].tokens == s.tokens and back[0].loss_mask == s.loss_mask
    prompts = load_rl_prompts([{"question": "1+1?", "answer": 2}, {"messages": conv}, {"nothing": 1}])
    assert [x.prompt for x in prompts] == ["1+1?", "hi"] and prompts[0].ground_truth == "2"


def test_hybrid_oracle_blocks():
    import math

    from research_b200.models.hybrid import (causal_conv1d, gated_attention, gated_delta_net, gated_delta_rule_chunked,
                                             gated_delta_rule_recurrent, partial_rope, qwen3_next_moe)

    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    T, H, dk, dv, hidden = 37, 3, 8, 12, 32
    q, k = torch.nn.functional.normalize(r(T, H, dk), dim=-1), torch.nn.functional.normalize(r(T, H, dk), dim=-1)
    v, a, b = r(T, H, dv), torch.sigmoid(r(T, H) + 2), torch.sigmoid(r(T, H))
    o1, s1 = gated_delta_rule_recurrent(q, k, v, a, b)
    o2, s2 = gated_delta_rule_chunked(q, k, v, a, b, chunk=8)
    assert torch.allclose(o1, o2, atol=2e-4) and torch.allclose(s1, s2, atol=2e-4)
    # decode: carrying the state over a split gives the same result as one pass
    oa, sa = gated_delta_rule_recurrent(q[:20], k[:20], v[:20], a[:20], b[:20])
    ob, sb = gated_delta_rule_chunked(q[20:], k[20:], v[20:], a[20:], b[20:], chunk=8, state=sa)
    assert torch.allclose(torch.cat([oa, ob]), o1, atol=2e-4) and torch.allclose(sb, s1, atol=2e-4)
    # conv state carry
    x, cw = r(T, 10), r(10, 4)
    y, _ = causal_conv1d(x, cw)
    y1, st = causal_conv1d(x[:15], cw)
    y2, _ = causal_conv1d(x[15:], cw, st)
    assert torch.allclose(torch.cat([y1, y2]), y, atol=1e-5)
    # partial rope leaves the tail channels alone and preserves norms of the rotated part
    xr = r(T, H, 16)
    pr = partial_rope(xr, torch.arange(T), 8, 10000.0)
    assert torch.equal(pr[..., 8:], xr[..., 8:]) and torch.allclose(pr[..., :8].norm(dim=-1), xr[..., :8].norm(dim=-1), atol=1e-4)
    # full blocks run, are causal, and the chunked/recurrent block outputs agree
    p = "l"
    w = {f"{p}.in_proj_qkvz.weight": r(2 * H * dk + 2 * H * dv, hidden) * 0.2, f"{p}.in_proj_ba.weight": r(2 * H, hidden) * 0.2,
         f"{p}.conv1d.weight": r(2 * H * dk + H * dv, 4) * 0.3, f"{p}.A_log": r(H) * 0.1, f"{p}.dt_bias": r(H) * 0.1,
         f"{p}.norm.weight": torch.ones(dv), f"{p}.out_proj.weight": r(hidden, H * dv) * 0.2}
    xh = r(T, hidden)
    y_c, _ = gated_delta_net(xh, w, p, H, dk, dv, 1e-6, chunk=8)
    y_r, _ = gated_delta_net(xh, w, p, H, dk, dv, 1e-6, chunk=None)
    assert torch.allclose(y_c, y_r, atol=5e-4)
    y_prefix, _ = gated_delta_net(xh[:10], w, p, H, dk, dv, 1e-6, chunk=8)
    assert torch.allclose(y_prefix, y_c[:10], atol=5e-4), "block must be causal"
    hd = 16
    wa = {"a.q_proj.weight": r(4 * 2 * hd, hidden) * 0.2, "a.k_proj.weight": r(2 * hd, hidden) * 0.2, "a.v_proj.weight": r(2 * hd, hidden) * 0.2,
          "a.q_norm.weight": torch.ones(hd), "a.k_norm.weight": torch.ones(hd), "a.o_proj.weight": r(hidden, 4 * hd) * 0.2}
    ya = gated_attention(xh, wa, "a", 4, 2, hd, torch.arange(T), 8, 10000.0, 1e-6)
    assert ya.shape == (T, hidden) and torch.allclose(gated_attention(xh[:9], wa, "a", 4, 2, hd, torch.arange(9), 8, 10000.0, 1e-6), ya[:9], atol=1e-4)
    E, F_ = 4, 24
    wm = {"m.gate.weight": r(E, hidden), "m.shared_expert_gate.weight": r(1, hidden)}
    for e in list(range(E)) + ["s"]:
        pe = "m.shared_expert" if e == "s" else f"m.experts.{e}"
        wm.update({f"{pe}.gate_proj.weight": r(F_, hidden) * 0.2, f"{pe}.up_proj.weight": r(F_, hidden) * 0.2, f"{pe}.down_proj.weight": r(hidden, F_) * 0.2})
    ym = qwen3_next_moe(xh, wm, "m", top_k=2)
    assert ym.shape == xh.shape and torch.isfinite(ym).all() and not math.isnan(float(ym.sum()))


def test_layerwise_debug_report():
    from research_b200.models import get_preset, init_random_weights
    from research_b200.models.debug import compare_traces, oracle_trace

    cfg = get_preset("tiny-qwen2", num_layers=3)
    w = init_random_weights(cfg, seed=0)
    ids = torch.randint(0, cfg.vocab_size, (2, 9), generator=torch.Generator().manual_seed(0))
    ref = oracle_trace(ids, w, cfg)
    assert list(ref)[:2] == ["embed", "layer.0"] and "logits" in ref
    rep = compare_traces(oracle_trace(ids, w, cfg, torch.bfloat16), ref, rel_tol=5e-2)
    assert rep.ok and "within tolerance" in rep.format()
    broken = dict(w)
    broken["model.layers.1.mlp.down_proj.weight"] = w["model.layers.1.mlp.down_proj.weight"] * 1.5
    rep = compare_traces(oracle_trace(ids, broken, cfg), ref, rel_tol=1e-3)
    assert rep.first_divergence.name == "layer.1" and "first divergence at layer.1" in rep.format()


def test_moe_training_backend_cpu():
    from research_b200.models import get_preset
    from research_b200.training.backends import PyTorchTrainingBackend

    cfg = get_preset("tiny-moe", num_layers=2)
    be = PyTorchTrainingBackend(cfg, device="cpu", loss_fn="ce", lr=3e-3)
    ids = torch.randint(0, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(0))
    losses = []
    for _ in range(4):
        losses.append(be.forward_backward({"input_ids": ids, "labels": ids}).wait()["loss"])
        be.optim_step().wait()
    assert losses[-1] < losses[0]


def test_packed_shards_bos_aligned_batches(tmp_path):
    import numpy as np
    import pytest

    from research_b200.training.datasets.packed_shards import (document_starts, load_shard, pack_documents, packed_batches,
                                                               write_shard)

    BOS = 1
    rng = np.random.default_rng(0)
    docs = [[BOS] + list(rng.integers(2, 500, size=int(n))) for n in rng.integers(5, 40, size=60)]
    flat = [t for d in docs for t in d]
    write_shard(tmp_path / "a.bin", flat)
    toks = load_shard(tmp_path / "a.bin")
    assert toks.tolist() == flat and len(document_starts(toks, BOS)) == 60
    (tmp_path / "bad.bin").write_bytes(b"\0" * 2048)
    with pytest.raises(ValueError):
        load_shard(tmp_path / "bad.bin")
    x, y, cu, nxt = pack_documents(toks, document_starts(toks, BOS), 0, 64, 16)
    assert x.numel() == y.numel() == 64 and int(cu[-1]) == 64 and nxt > 0
    lens = (cu[1:] - cu[:-1]).tolist()
    assert max(lens) <= 16 and all(int(x[int(s)]) == BOS for s in cu[:-1])          # every sequence starts a document
    assert torch.equal(y[:lens[0] - 1], x[1:lens[0]])                                # targets are the inputs shifted by one
    b0 = list(packed_batches([tmp_path / "a.bin"], 64, 16, BOS, rank=0, world=2))
    b1 = list(packed_batches([tmp_path / "a.bin"], 64, 16, BOS, rank=1, world=2))
    assert len(b0) == len(b1) >= 2 and not torch.equal(b0[0][0], b1[0][0])
    single = list(packed_batches([tmp_path / "a.bin"], 64, 16, BOS))
    assert torch.equal(single[0][0], b0[0][0]) and torch.equal(single[1][0], b1[0][0])    # ranks split the same stream


def test_grouped_experts_layout_and_reference():
    """The experts of a layer lie back to back in the flat bucket (gate|up of every expert, then every down projection),
    and the grouped-experts oracle equals the functional MoE layer."""
    from research_b200.models.functional import moe_mlp
    from research_b200.ops.moe_train import grouped_experts_reference
    from research_b200.parallel.symm import LocalComm
    from research_b200.training.backends.native import build_buckets

    cfg = get_preset("tiny-moe", num_layers=2, init_std=0.05)
    b = build_buckets(cfg, LocalComm(torch.device("cpu")), torch.float32)
    E, F, d = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
    m = "model.layers.1.mlp."
    names = [f"{m}experts.{e}.{p}.weight" for e in range(E) for p in ("gate_proj", "up_proj")] + [f"{m}experts.{e}.down_proj.weight" for e in range(E)]
    specs = [b.specs[n] for n in names]
    assert all(x.offset + x.numel == y.offset for x, y in zip(specs, specs[1:]))
    w = init_random_weights(cfg, seed=0)
    wgu = torch.cat([w[n] for n in names[:2 * E]])
    wd = torch.cat([w[n] for n in names[2 * E:]])
    assert wgu.shape == (E * 2 * F, d) and wd.shape == (E * d, F)
    h = torch.randn(37, d) * 0.5
    logits = h @ w[m + "gate.weight"].t()
    wt, idx = logits.softmax(-1).topk(cfg.num_experts_per_tok, dim=-1)
    if cfg.norm_topk_prob:
        wt = wt / wt.sum(-1, keepdim=True)
    got = grouped_experts_reference(h, idx, wt, wgu, wd)
    want = moe_mlp(h[None], w, m, cfg)[0]
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-4)


def test_lazy_weights_and_lazy_state_dict():
    """Presets above 12 B parameters come back as a lazy mapping (one tensor at a time); a model's lazy state dict
    resolves names against its buckets when asked."""
    from research_b200.models.weights import LazyRandomWeights, param_shapes
    from research_b200.training.backends import load_model_weights
    from research_b200.training.backends.native import NativeTrainingBackend
    from research_b200.training.native_model import LazyStateDict

    w, cfg = load_model_weights("qwen3-30b-a3b")
    assert isinstance(w, LazyRandomWeights) and len(w) == len(param_shapes(cfg))
    t = w["model.layers.3.mlp.experts.17.down_proj.weight"]
    assert t.shape == (cfg.hidden_size, cfg.moe_intermediate_size) and torch.equal(t, w["model.layers.3.mlp.experts.17.down_proj.weight"])
    small, _ = load_model_weights("tiny-moe")
    assert isinstance(small, dict)
    tiny = get_preset("tiny-moe", num_layers=2)
    be = NativeTrainingBackend(tiny, init_random_weights(tiny, seed=0), device="cpu", loss_fn="ce")
    lazy = LazyStateDict(be.model)
    assert set(lazy) == set(param_shapes(tiny)) and len(lazy) == len(param_shapes(tiny))
    n = "model.layers.1.mlp.experts.3.up_proj.weight"
    assert torch.equal(lazy[n], be.buckets.full_param(n))


def test_vocab_parallel_logprob_matches_log_softmax_and_tp_backend_runs_alone():
    """The split log-softmax on one shard (no group) is the ordinary one, values and gradients, entropy included; the
    tensor-parallel backend with a single rank is an ordinary trainer."""
    from research_b200.training.backends.tensor_parallel import TensorParallelTrainingBackend, split_dim, vocab_parallel_logprob

    g = torch.Generator().manual_seed(0)
    logits = torch.randn(3, 5, 17, generator=g, requires_grad=True)
    targets = torch.randint(0, 17, (3, 5), generator=g)
    targets[0, 0] = -1
    lp, ent = vocab_parallel_logprob(logits, targets, 0, None, True)
    w_lp, w_ent = torch.randn(3, 5, generator=g), torch.randn(3, 5, generator=g)
    ((lp * w_lp).sum() + (ent * w_ent).sum()).backward()
    ref = logits.detach().clone().requires_grad_(True)
    lsm = torch.log_softmax(ref, -1)
    r_lp = torch.where(targets >= 0, lsm.gather(-1, targets.clamp(min=0)[..., None])[..., 0], torch.zeros(3, 5))
    r_ent = -(lsm.exp() * lsm).sum(-1)
    ((r_lp * w_lp).sum() + (r_ent * w_ent).sum()).backward()
    assert torch.allclose(lp, r_lp, atol=1e-6) and torch.allclose(ent, r_ent, atol=1e-5) and torch.allclose(logits.grad, ref.grad, atol=1e-5)
    assert lp[0, 0] == 0 and split_dim("model.layers.3.mlp.down_proj.weight") == 1 and split_dim("model.norm.weight") is None
    cfg = get_preset("tiny-qwen2", num_layers=1)
    be = TensorParallelTrainingBackend(cfg, init_random_weights(cfg, seed=0), lr=1e-2)
    ids = torch.randint(0, cfg.vocab_size, (2, 10), generator=g)
    first = be.forward_backward({"input_ids": ids, "labels": ids}).wait()["loss"]
    be.optim_step()
    for _ in range(5):
        be.forward_backward({"input_ids": ids, "labels": ids})
        be.optim_step()
    assert be.forward_backward({"input_ids": ids, "labels": ids}).wait()["loss"] < first and be.tp_size == 1 and be.current_step == 6
    with pytest.raises(AssertionError, match="expert parallelism"):
        TensorParallelTrainingBackend(get_preset("tiny-moe"))
