"""TOML-driven pretraining loop on CPU: config parsing, the derived model, synthetic and shard data."""

from pathlib import Path

import numpy as np
import pytest
import torch

from research_b200.training.datasets.packed_shards import write_shard
from research_b200.training.pretrain import (PretrainConfig, PretrainData, PretrainModel, PretrainTraining, main, pretrain,
                                              shard_batches, synthetic_batches)

ROOT = Path(__file__).resolve().parents[1]


def test_shipped_config_gives_a_moe_model():
    cfg = PretrainConfig.from_toml(ROOT / "configs" / "dsv3_tiny.toml")
    assert cfg.training.batch_size == 4 and cfg.training.seq_len == 2048 and cfg.training.lr == pytest.approx(1e-4)
    mc = cfg.model_config()
    assert mc.is_moe and mc.num_experts == 8 and mc.num_experts_per_tok == 2 and mc.hidden_size == 1024 and mc.head_dim == 128
    assert mc.router_type == "sigmoid" and mc.n_shared_experts == 1 and mc.first_k_dense_replace == 1
    assert mc.intermediate_size % 128 == 0 and mc.moe_intermediate_size % 128 == 0


def test_config_errors(tmp_path):
    p = tmp_path / "c.toml"
    p.write_text("[model]\nhidden_sizee = 3\n")
    with pytest.raises(ValueError, match="unknown keys"):
        PretrainConfig.from_toml(p)
    p.write_text("[optimizer]\nlr = 1\n")
    with pytest.raises(ValueError, match="unknown sections"):
        PretrainConfig.from_toml(p)
    with pytest.raises(ValueError):
        PretrainConfig(PretrainModel(hidden_size=100, num_attention_heads=8)).model_config()
    with pytest.raises(ValueError):
        PretrainConfig(PretrainModel(num_experts=4, num_active_experts=5)).model_config()
    assert not PretrainConfig(PretrainModel(num_experts=0)).model_config().is_moe


def _small(**data) -> PretrainConfig:
    return PretrainConfig(PretrainModel(hidden_size=64, num_layers=2, num_attention_heads=2, num_experts=4, num_active_experts=2,
                                        vocab_size=64, intermediate_size=128, moe_intermediate_size=128),
                          PretrainTraining(batch_size=4, seq_len=32, lr=3e-3, warmup_steps=2), PretrainData(**data))


def test_synthetic_stream_is_learnable_and_loss_falls():
    b = next(synthetic_batches(64, 3, 16, seed=1))
    ids = b["input_ids"]
    assert ids.shape == (3, 16) and int(ids.max()) < 64
    step = {(int((a * ids[r, 0] + c) % 64)) for r in range(3) for a, c in [(3, 1), (5, 7), (7, 3), (11, 5)]}
    assert all(int(ids[r, 1]) in step for r in range(3))
    lines = []
    hist = pretrain(_small(synthetic=True), steps=12, device="cpu", log=lines.append)
    assert len(hist) == 12 and hist[-1]["loss"] < hist[0]["loss"] - 0.2 and hist[0]["tokens_per_s"] > 0
    assert hist[1]["lr"] == pytest.approx(3e-3) and hist[-1]["lr"] < 1e-3 and "experts top-2" in lines[0]


def test_shards_feed_the_loop(tmp_path):
    rng = np.random.default_rng(0)
    docs = []
    for _ in range(40):
        docs += [1] + list(rng.integers(2, 64, size=int(rng.integers(10, 60))))
    write_shard(tmp_path / "train_000.bin", np.array(docs, dtype=np.uint16))
    files = [tmp_path / "train_000.bin"]
    b = next(shard_batches(files, 2, 32, bos_id=1))
    assert b["input_ids"].shape == (2, 32) and torch.equal(b["labels"][:, 0], b["input_ids"][:, 0])
    hist = pretrain(_small(path=str(tmp_path)), steps=3, device="cpu", log=None)
    assert len(hist) == 3 and all(np.isfinite(h["loss"]) for h in hist)
    with pytest.raises(FileNotFoundError):
        pretrain(_small(path=str(tmp_path / "none")), steps=1, device="cpu", synthetic=False, log=None)


def test_cli_runs_a_tiny_config(tmp_path):
    p = tmp_path / "t.toml"
    p.write_text("[model]\nhidden_size = 64\nnum_layers = 1\nnum_attention_heads = 2\nnum_experts = 0\nvocab_size = 64\n"
                 "intermediate_size = 128\n[training]\nbatch_size = 2\nseq_len = 16\nlr = 1e-3\n[data]\nsynthetic = true\n")
    out = tmp_path / "h.json"
    assert main([str(p), "--steps", "2", "--device", "cpu", "--json", str(out)]) == 0
    import json
    assert len(json.loads(out.read_text())) == 2
