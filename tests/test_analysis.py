"""Outlier-feature statistics and corpus-proximity utilities (CPU)."""

import torch

from research_b200.analysis import (CorpusIndex, chunk_text, cluster_recursively, collect_residual_stream, contamination_report,
                                    find_outlier_features, hashed_ngram_embedding, perplexity)
from research_b200.models import get_preset, init_random_weights


def test_outlier_features_on_synthetic_and_model_activations():
    g = torch.Generator().manual_seed(0)
    layers = [torch.randn(2, 50, 64, generator=g) for _ in range(8)]
    for li in (1, 3, 4, 6):                      # dim 7 explodes in half of the layers, on 20 % of the positions
        layers[li][:, ::5, 7] = 9.0
    layers[2][0, 0, 11] = 50.0                   # a single spike does not qualify
    rep = find_outlier_features(layers)
    assert rep.dims == [7] and abs(rep.layer_frac[7] - 0.5) < 1e-6 and rep.token_frac[7] >= 0.06 and rep.max_abs[7] == 9.0
    assert rep.per_layer_counts[1] == 1 and rep.per_layer_counts[0] == 0 and "dim 7" in rep.summary()
    cfg = get_preset("tiny-qwen2", num_layers=2)
    w = init_random_weights(cfg, seed=0)
    ids = torch.randint(0, cfg.vocab_size, (2, 12), generator=g)
    stream = collect_residual_stream(ids, w, cfg)
    assert set(stream) == {"embed", "layer.0", "layer.1"} and stream["layer.1"].shape == (2, 12, cfg.hidden_size)
    assert find_outlier_features(stream).dims == []                 # N(0, 0.02) init: nothing near 6
    ppl = perplexity(ids, w, cfg)
    assert 0.5 * cfg.vocab_size < ppl < 2 * cfg.vocab_size         # a random model is about uniform


def test_corpus_proximity():
    docs = ["Natalia sold clips to 48 of her friends in April. Then she sold half as many clips in May. How many clips did she sell?",
            "The mitochondria is the powerhouse of the cell. It produces energy. Cells need energy to live.",
            "Gradient descent updates parameters against the gradient. The learning rate scales the step. Momentum smooths it."]
    assert chunk_text("A b c. D e. F g h. I.", "sentences", size=2, overlap=1) == ["A b c. D e.", "D e. F g h.", "F g h. I."]
    assert chunk_text("one two three four five", "words", size=2, overlap=0) == ["one two", "three four", "five"]
    assert chunk_text("p1 line\n\np2 line", "paragraphs") == ["p1 line", "p2 line"]
    idx = CorpusIndex.build(docs, names=["gsm8k", "bio", "ml"], size=2, overlap=1)
    hit = idx.search(["natalia sold clips to 48 of her friends in april"], k=2)[0]
    assert idx.sources[hit[0][1]] == "gsm8k" and hit[0][0] < 0.4 and hit[0][0] <= hit[1][0]
    for metric in ("euclidean", "manhattan"):
        assert idx.sources[idx.search(["the learning rate scales the step"], k=1, metric=metric)[0][0][1]] == "ml"
    rep = contamination_report(idx, ["Then she sold half as many clips in May.", "Quantum chromodynamics describes the strong force."])
    assert rep["items"][0]["distance"] < rep["items"][1]["distance"] and rep["contaminated_fraction"] == 0.5
    e = hashed_ngram_embedding(["abc", "abc", "xyz"])
    assert torch.allclose(e[0], e[1]) and float(e[0] @ e[2]) < 0.5
    g = torch.Generator().manual_seed(0)
    pts = torch.cat([torch.randn(30, 8, generator=g) + 10 * torch.eye(8)[i] for i in range(4)])
    tree = cluster_recursively(pts, max_depth=1, branching=4, min_size=8)
    sizes = sorted(len(c["ids"]) for c in tree["children"])
    assert sum(sizes) == 120 and len(tree["ids"]) == 120 and max(sizes) <= 60


def test_optimizer_paths():
    from research_b200.analysis.optimizer_paths import distance_to_minimum, render, trajectory

    adam = trajectory("quadratic", "adam", steps=400, lr=0.05)
    sgd = trajectory("quadratic", "sgd", steps=400, lr=0.05)
    mom = trajectory("quadratic", "momentum", steps=400, lr=0.01)
    assert adam.shape == (401, 2) and distance_to_minimum("quadratic", adam) < 0.05
    assert distance_to_minimum("quadratic", sgd) < 1e-3 and distance_to_minimum("quadratic", mom) < 1e-2
    ref = torch.tensor([2.0, 2.0], dtype=torch.float64, requires_grad=True)      # hand-written Adam against torch's
    opt = torch.optim.Adam([ref], lr=0.05)
    for _ in range(10):
        opt.zero_grad()
        (0.5 * (10 * ref[0] ** 2 + ref[1] ** 2)).backward()
        opt.step()
    assert torch.allclose(adam[10], ref.detach(), atol=1e-9)
    blew_up = trajectory("rosenbrock", "sgd", steps=50, lr=0.1)                     # diverges: the path stops early
    assert blew_up.shape[0] < 51
    rose = trajectory("rosenbrock", "adam", steps=3000, lr=0.02)
    assert distance_to_minimum("rosenbrock", rose) < 0.2
    pic = render("rosenbrock", {"adam": rose[::50]}, width=40, height=16)
    assert len(pic.split("\n")) == 16 and "*" in pic and "A" in pic
