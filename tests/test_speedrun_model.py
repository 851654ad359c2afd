"""The speedrun GPT oracle: shapes, causality, sliding windows, document boundaries, gradients."""

import torch

from research_b200.models.speedrun import SpeedrunConfig, forward, init_weights, loss, rotary, rotary_tables

CFG = SpeedrunConfig(vocab_size=97, num_heads=2, head_dim=16, max_seq_len=64, block_size=4)


def test_shapes_softcap_and_zero_init():
    w0 = init_weights(CFG, seed=0)
    toks = torch.randint(0, CFG.vocab_size, (32,), generator=torch.Generator().manual_seed(1))
    out0 = forward(w0, toks, CFG)
    assert out0.shape == (32, CFG.vocab_size) and torch.allclose(out0, torch.full_like(out0, 15.0))   # zero head: sigmoid(0) * 30
    w = init_weights(CFG, seed=0, zero_init_projections=False)
    out = forward(w, toks, CFG)
    assert float(out.min()) > 0 and float(out.max()) < 30 and out.std() > 1e-3
    cos, sin = rotary_tables(CFG)
    assert cos.shape == (64, 8) and torch.all(cos[:, 4:] == 1) and torch.all(sin[:, 4:] == 0)    # half of the pairs carry no position
    x = torch.randn(5, 2, 16)
    assert torch.allclose(rotary(x, cos, sin).norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_causality_windows_and_documents():
    w = init_weights(CFG, seed=2, zero_init_projections=False)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, CFG.vocab_size, (48,), generator=g)
    base = forward(w, toks, CFG, ws_short=2, ws_long=3)
    fut = toks.clone()
    fut[30] = (fut[30] + 1) % CFG.vocab_size
    changed = forward(w, fut, CFG, ws_short=2, ws_long=3)
    assert torch.allclose(base[:30], changed[:30], atol=1e-6) and not torch.allclose(base[30:], changed[30:])
    # a packed second document does not see the first one
    cu = torch.tensor([0, 20, 48])
    two = forward(w, toks, CFG, cu_seqlens=cu, ws_short=2, ws_long=3)
    alone = forward(w, toks[20:], CFG, ws_short=2, ws_long=3)
    # the smear gate starts at zero, so the packed document equals the same document run on its own
    assert torch.allclose(two[20:], alone, atol=1e-4)
    first_changed = toks.clone()
    first_changed[5] = (first_changed[5] + 1) % CFG.vocab_size
    two_b = forward(w, first_changed, CFG, cu_seqlens=cu, ws_short=2, ws_long=3)
    assert torch.allclose(two[21:], two_b[21:], atol=1e-6)            # document 2 is blind to document 1
    one_b = forward(w, first_changed, CFG, ws_short=2, ws_long=3)
    assert not torch.allclose(base[6:12], one_b[6:12])                 # inside one document the change is seen nearby


def test_loss_and_gradients_reach_every_parameter():
    raw = init_weights(CFG, seed=4, zero_init_projections=False)
    raw["scalars"][-2] = 0.3            # the smear scalar starts at zero, which would hide its gate from the gradient
    w = {k: v.clone().requires_grad_(True) for k, v in raw.items()}
    toks = torch.randint(0, CFG.vocab_size, (24,), generator=torch.Generator().manual_seed(5))
    val = loss(w, toks[:-1], toks[1:], CFG, ws_short=1, ws_long=2)
    assert torch.isfinite(val) and abs(float(val.detach()) - torch.log(torch.tensor(float(CFG.vocab_size)))) < 1.5
    val.backward()
    silent = [k for k, v in w.items() if v.grad is None or float(v.grad.abs().sum()) == 0.0]
    assert silent == [], silent


import pytest  # noqa: E402


@pytest.mark.gpu
def test_flash_attention_path_matches_the_masked_oracle(cuda_device):
    """Sliding windows over packed documents through the tcgen05 flash kernel against the explicit-mask oracle."""
    cfg = SpeedrunConfig(vocab_size=211, num_heads=2, head_dim=64, max_seq_len=512, block_size=16)
    w = {k: v.to(cuda_device) for k, v in init_weights(cfg, seed=6, zero_init_projections=False).items()}
    toks = torch.randint(0, cfg.vocab_size, (384,), generator=torch.Generator().manual_seed(7)).to(cuda_device)
    cu = torch.tensor([0, 100, 257, 384], device=cuda_device)
    want = forward(w, toks, cfg, cu_seqlens=cu, ws_short=2, ws_long=5)
    got = forward(w, toks, cfg, cu_seqlens=cu, ws_short=2, ws_long=5, use_flash=True)
    assert (got - want).abs().max() < 0.15 and (got - want).abs().mean() < 0.01, ((got - want).abs().max(), (got - want).abs().mean())
    # gradients through the flash backward kernels against autograd through the masked oracle
    grads = {}
    for flash in (False, True):
        leaves = {k: v.clone().requires_grad_(True) for k, v in w.items()}
        loss(leaves, toks[:-1], toks[1:], cfg, cu_seqlens=torch.tensor([0, 100, 257, 383], device=cuda_device), ws_short=2, ws_long=5,
             use_flash=flash).backward()
        grads[flash] = leaves
    for name in ("blocks.3.qkv", "blocks.10.qkv", "embed", "value_embed.1"):
        a, b = grads[True][name].grad.float(), grads[False][name].grad.float()
        assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.98, name


def test_speedrun_training_driver_learns_a_repeating_stream(tmp_path):
    from research_b200.training.datasets.packed_shards import packed_batches, write_shard
    from research_b200.training.speedrun import SpeedrunHyper, get_lr, get_muon_momentum, get_windows, train

    h = SpeedrunHyper(num_iterations=40, adam_lr=0.02, muon_lr=0.02, ws_short_final=2, ws_long_final=4, muon_momentum_warmup=10)
    assert get_lr(0, h) == 1.0 and abs(get_lr(40, h) - 0.1) < 1e-9 and 0.1 < get_lr(35, h) < 1.0
    assert get_windows(0, h) == (1, 1) and get_windows(39, h) == (2, 4)
    assert get_muon_momentum(0, h) == 0.85 and get_muon_momentum(100, h) == 0.95
    BOS = 1
    doc = [BOS] + [2 + (i * 7) % 11 for i in range(15)]                    # every document is the same 16 tokens
    write_shard(tmp_path / "s.bin", doc * 400)
    cfg = SpeedrunConfig(vocab_size=32, num_heads=2, head_dim=16, max_seq_len=64, block_size=8)
    _, losses = train(cfg, packed_batches([tmp_path / "s.bin"], 64, 16, BOS, loop=True), h)
    assert len(losses) == 40 and losses[0] > 3.0 and losses[-1] < 0.6 * losses[0], (losses[0], losses[-1])


def test_yarn_follows_the_window():
    import math

    from research_b200.models.speedrun import SpeedrunConfig, Yarn, rotary_tables

    cfg = SpeedrunConfig(num_layers=4, num_heads=2, head_dim=16, max_seq_len=256, block_size=16, vocab_size=64)
    y = Yarn(cfg)
    cos0, sin0 = y.tables()
    ref_cos, ref_sin = rotary_tables(cfg)
    assert torch.allclose(cos0, ref_cos) and torch.allclose(sin0, ref_sin)              # before any growth: the plain tables
    assert not y.follow(3) and not y.follow(3) and y.attn_scale == 0.1
    before = y.angular_freq.clone()
    assert y.follow(6) and y.window == 6
    rot = cfg.block_size * 3 * before / (2 * math.pi)
    # the fastest frequency (7.6 rotations inside the old window) moves a little, slow ones are halved, zeros stay zero
    ratio = y.angular_freq[:4] / before[:4]
    assert rot[0] > 1 and 0.5 < float(ratio[0]) < 1.0 and torch.allclose(ratio[rot[:4] <= 1], torch.tensor(0.5)) and torch.equal(y.angular_freq[4:], torch.zeros(4))
    assert abs(y.attn_scale - 0.1 * (0.2 * math.log(2) + 1)) < 1e-12
    many = Yarn(SpeedrunConfig(num_layers=4, num_heads=2, head_dim=16, max_seq_len=256, block_size=128, vocab_size=64))
    f0 = many.angular_freq.clone()
    many.apply(8, 16)
    assert float(many.angular_freq[0] / f0[0]) == 1.0                                      # >= 32 rotations: left alone
