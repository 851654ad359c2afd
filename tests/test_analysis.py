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


def test_outlier_pipeline_batches_comparison_and_memory_estimate(tmp_path, capsys):
    from research_b200.analysis import outlier_features as of

    # the two readings of "6 % of the sequence": dim 3 crosses in ONE layer per position, spread over many positions
    g = torch.Generator().manual_seed(1)
    layers = [torch.randn(1, 100, 16, generator=g) for _ in range(4)]
    for li in range(4):
        layers[li][0, li * 3:(li * 3) + 3, 3] = 8.0                   # 3 positions per layer, 12 distinct positions = 12 %
    assert of.find_outlier_features(layers, criterion="positions").dims == [3] and of.find_outlier_features(layers, criterion="cells").dims == []
    rec = of.find_outlier_features(layers, criterion="positions").to_records()[0]
    assert abs(rec["seq_percentage"] - 0.12) < 1e-6 and abs(rec["cell_percentage"] - 0.03) < 1e-6 and rec["layer_percentage"] == 1.0
    # text -> windows
    assert of.chunk_text_by_chars("aaa bbb ccc ddd", 8) == ["aaa bbb", "ccc ddd"] and of.chunk_ids(list(range(10)), 4) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert of.chunk_ids(list(range(10)), 4, stride=2)[-1] == [6, 7, 8, 9] and of.chunk_ids(list(range(10)), 4, drop_last=False)[-1] == [6, 7, 8, 9]
    from research_b200.utils.char_tokenizer import CharTokenizer

    tok = CharTokenizer()
    seqs = of.get_token_sequences(["hello world", "second document here"], tok, 3, 8)
    assert seqs.shape == (3, 8) and tok.eos_token_id in seqs[1].tolist()
    # a model with a planted outlier dimension: a large embedding column survives the residual stream in every layer
    cfg = get_preset("tiny-qwen2", num_layers=3)
    w = init_random_weights(cfg, seed=0)
    w["model.embed_tokens.weight"][:, 5] = 12.0
    ids = torch.randint(0, cfg.vocab_size, (4, 16), generator=g)
    res = of.run_analysis(w, cfg, ids, batch_size=2, model_name="tiny-planted", out_dir=tmp_path / "planted")
    assert res["num_batches"] == 2 and [o["feature_dim"] for o in res["systematic_outliers"]] == [5] and res["systematic_outliers"][0]["batch_percentage"] == 1.0
    assert res["layer_max"]["embed"] >= 12.0 and res["perplexity"] > 1.0
    clean = of.run_analysis(init_random_weights(cfg, seed=0), cfg, ids, 2, "tiny-clean", tmp_path / "clean")
    assert clean["num_systematic"] == 0
    agg = of.aggregate_batch_results([{"outliers": [{"feature_dim": 1, "max_magnitude": 7.0, "layer_percentage": 0.5, "seq_percentage": 0.1}], "layer_max": {}, "num_tokens": 10, "perplexity": 4.0},
                                      {"outliers": [], "layer_max": {}, "num_tokens": 30, "perplexity": 16.0},
                                      {"outliers": [], "layer_max": {}, "num_tokens": 0, "perplexity": 1.0}])
    assert agg["num_systematic"] == 0 and agg["candidate_dims"] == 1 and abs(agg["perplexity"] - 16 ** 0.75 * 4 ** 0.25) < 1e-6
    rows = of.collect_results(tmp_path)
    assert [r["model"] for r in rows] == ["tiny-planted", "tiny-clean"] or {r["model"] for r in rows} == {"tiny-planted", "tiny-clean"}
    planted = next(r for r in rows if r["model"] == "tiny-planted")
    assert planted["num_outliers"] == 1 and planted["mean_layer_pct"] == 100.0
    assert "tiny-planted" in of.format_table(rows) and of.to_csv(rows).splitlines()[0].startswith("model,num_params,num_outliers")
    assert "a=tiny" in of.terminal_plot(rows) and of.terminal_plot([]) == "(no results)"
    # memory: an 8B model in bf16 is ~16 GB of weights; training adds 12 bytes per parameter of optimizer state; sharding divides it
    big = get_preset("llama-3-8b")
    inf = of.estimate_vram(big, "bfloat16", batch_size=1, seq_len=4096)
    assert 15 < inf["weights_gb"] < 17 and abs(inf["kv_cache_gb"] - 2 * 32 * 4096 * 8 * 128 * 2 / 1e9) < 1e-6 and inf["fits"]
    tr1, tr8 = of.estimate_vram(big, mode="training", seq_len=4096, gpu_gb=80), of.estimate_vram(big, mode="training", seq_len=4096, num_gpus=8, gpu_gb=80)
    assert of.estimate_vram(big, mode="training", seq_len=4096)["fits"]                      # 180 GB holds an 8B training run on one GPU
    assert abs(tr1["optimizer_gb"] - 12 * big.num_params() / 1e9) < 1e-6 and not tr1["fits"] and tr8["fits"] and tr1["min_gpus"] >= 2
    assert abs(tr8["optimizer_gb"] * 8 - tr1["optimizer_gb"]) < 1e-6 and tr8["activations_gb"] == tr1["activations_gb"]
    assert of.estimate_vram(big, mode="analysis", seq_len=2048)["activations_gb"] > of.estimate_vram(big, seq_len=2048)["activations_gb"]
    n, how = of.params_from_hf_config(big.to_hf_dict())
    assert n == big.num_params() and "32 layers" in how and "dense" in how
    assert of.main(["vram", "--model", "llama-3-8b", "--mode", "training", "--num-gpus", "8"]) == 0 and "optimizer state" in capsys.readouterr().out
    assert of.main(["compare", str(tmp_path)]) == 0 and "tiny-clean" in capsys.readouterr().out


def test_cluster_tree_names_annotation_and_stage_similarity(tmp_path):
    import asyncio

    from research_b200.analysis import corpus_clusters as cc

    assert cc.split_into_sentences("Dr. Smith paid 3.50 dollars. He left! Did she? Yes.") == ["Dr. Smith paid 3.50 dollars.", "He left!", "Did she?", "Yes."]
    text = "alpha beta gamma delta epsilon zeta eta theta iota kappa lambda mu"
    fixed = cc.chunk_fixed_chars(text, 24, 0.25)
    assert all(len(c) <= 24 for c in fixed) and fixed[0].startswith("alpha") and fixed[-1].endswith("mu") and len(fixed) >= 3
    assert any(a.split()[-1] in b for a, b in zip(fixed, fixed[1:]))                      # neighbours overlap
    from research_b200.utils.char_tokenizer import CharTokenizer

    toks = cc.chunk("abcdefghij", "fixed_tokens", size=4, overlap_pct=0.5, tokenizer=CharTokenizer())
    assert toks == ["abcd", "cdef", "efgh", "ghij"] and cc.chunk("p1\n\np2", "paragraph") == ["p1", "p2"]
    # three well-separated families, one of them with two sub-families
    g = torch.Generator().manual_seed(0)
    centres = [torch.eye(12)[0] * 10, torch.eye(12)[1] * 10, torch.eye(12)[2] * 10 + torch.eye(12)[3] * 3, torch.eye(12)[2] * 10 - torch.eye(12)[3] * 3]
    vectors = torch.cat([c + 0.3 * torch.randn(25, 12, generator=g) for c in centres])
    texts = [f"{['math', 'cooking', 'law-contracts', 'law-criminal'][i // 25]} text {i}" for i in range(100)]
    tree = cc.recursive_cluster(vectors, max_depth=2, min_cluster_size=5, seed=0)
    top = sorted(n.size for n in tree.children)
    assert len(tree.children) in (3, 4) and sum(top) + len(tree.noise_indices) == 100 and tree.silhouette > 0.5
    stats = cc.compute_cluster_stats(tree)
    assert stats["max_depth"] >= 1 and stats["total_clusters"] == len(list(tree.walk())) and stats["clusters_per_depth"][0] == 1
    m = cc.build_chunk_to_cluster_map(tree)
    top_of = lambda i: ".".join(m[i].split(".")[:2])                                    # noqa: E731
    assert len({top_of(i) for i in range(25)} - {"0"}) == 1 and top_of(0) != top_of(30) and all(m[i].startswith(top_of(i)) for i in range(100))
    again = cc.tree_from_dict(json_round_trip(cc.tree_to_dict(tree)))
    assert [n.cluster_id for n in again.walk()] == [n.cluster_id for n in tree.walk()] and cc.find_node_by_id(again, "0.1").size == cc.find_node_by_id(tree, "0.1").size
    # naming: the prompt carries typical members, the parent's name and named siblings; failures leave a node unnamed
    prompts = []

    async def complete(prompt):
        prompts.append(prompt)
        if "cooking" in prompt.split("Excerpts:")[1]:
            raise RuntimeError("model unavailable")
        first = prompt.split("1. ")[1].split()[0]
        return f'Name: "{first} documents."\nextra line'

    n = asyncio.run(cc.name_cluster_tree(tree, vectors, texts, complete, samples_per_cluster=3))
    names = {c.cluster_id: c.name for c in tree.walk()}
    assert n == len([v for v in names.values() if v]) and "" in names.values() and any(v == "math documents" for v in names.values())
    assert any("Sibling groups already named" in p for p in prompts) and any('part of the larger group "' in p for p in prompts)
    assert "(unnamed)" in cc.format_cluster_tree(tree) and "most typical:" in cc.inspect_cluster(tree, "0.0", vectors, texts) and "no cluster" in cc.inspect_cluster(tree, "9", vectors, texts)
    # a staged text corpus, stored and loaded, annotates a generation sentence by sentence
    docs = ["Natalia sold 48 clips in April. She sold half as many in May. How many clips did she sell altogether? " * 2,
            "The defendant signed the contract. The court found the clause void. Damages were awarded to the buyer. " * 2,
            "Whisk the eggs with sugar. Fold in the flour gently. Bake for twenty minutes at 180 degrees. " * 2]
    corpus = cc.ClusteredCorpus.build(docs, stages=["sft", "pretrain", "pretrain"], strategy="sentence", max_depth=1, min_cluster_size=2)
    for node in corpus.tree.walk():
        node.name = f"cluster {node.cluster_id}"
    corpus.save(tmp_path / "corpus")
    loaded = cc.ClusteredCorpus.load(tmp_path / "corpus")
    assert loaded.index.chunks == corpus.index.chunks and loaded.metadata[0]["corpus_stage"] == "sft" and loaded.path.endswith("corpus")
    gen = "She sold half as many in May. The weather on Mars is cold."
    lps = [("She sold half", -0.1), (" as many in May.", -0.3), (" The weather", -2.0), (" on Mars is cold.", -4.0)]
    ann = cc.annotate_text(loaded, gen, k=2, prompt="How many clips?", token_logprobs=lps)
    first, far = [a for a in ann.annotations if a.rank == 1]
    assert len(ann.annotations) == 4 and first.corpus_stage == "sft" and first.distance < 0.1 < far.distance and first.cluster_name.startswith("cluster 0")
    assert abs(first.avg_logprob + 0.2) < 1e-9 and abs(far.avg_logprob + 3.0) < 1e-9
    shown = cc.format_annotations(ann, show_chunks=True)
    assert "Prompt: How many clips?" in shown and "mean logprob -0.20" in shown and "nearest: She sold half as many in May." in shown
    assert len(cc.format_annotations_compact(ann).splitlines()) == 2 and cc.AnnotatedOutput.from_dict(json_round_trip(ann.to_dict())).annotations[0] == ann.annotations[0]
    assert cc.annotate_text(loaded, "  ").annotations == []
    sim = cc.similarity_by_stage(loaded, ["How many clips did she sell altogether?", "She sold 48 clips."])
    assert set(sim) == {"pretrain", "sft"} and sim["sft"]["mean"] < sim["pretrain"]["mean"] and sim["sft"]["chunks"] == 6


def json_round_trip(obj):
    import json

    return json.loads(json.dumps(obj))


def test_optimizer_comparison_export_and_momentum_rank(tmp_path):
    import json

    from research_b200.analysis.optimizer_paths import compare, export_viz_data, landscape, momentum_rank_experiment

    res = compare("narrow_valley", steps=400)
    # plain SGD crawls along the valley floor; momentum and Adam get there
    assert res["momentum"]["final_distance"] < res["sgd"]["final_distance"] and res["adam"]["final_distance"] < 0.5 and not res["adam"]["diverged"]
    assert res["momentum"]["steps_to_1pct"] is not None and res["sgd"]["steps_to_1pct"] < 20 and res["sgd"]["final_value"] > 1e6 * res["momentum"]["final_value"]
    assert compare("quadratic", {"sgd": {"lr": 0.5}}, steps=50)["sgd"]["diverged"]                    # lr above 2 / L = 0.2
    land = landscape("quadratic", resolution=11)
    assert len(land["z"]) == 11 and land["z"][5][5] == 0.0 and land["minimum"] == [0.0, 0.0]
    data = export_viz_data("narrow_valley", {k: res[k] for k in ("sgd", "adam")}, tmp_path / "viz.json", resolution=8)
    on_disk = json.loads((tmp_path / "viz.json").read_text())
    assert set(on_disk["trajectories"]) == {"sgd", "adam"} and len(on_disk["trajectories"]["adam"]["points"]) == 401 and len(on_disk["landscape"]["x"]) == 8
    assert data["trajectories"]["adam"]["values"][-1] < data["trajectories"]["adam"]["values"][0]
    # a rank-4 problem: the moment matrix of Adam concentrates on four directions while the loss falls
    r = momentum_rank_experiment(input_dim=24, output_dim=24, true_rank=4, steps=300, lr=0.05, record_every=75)
    first, last = r["records"][0], r["records"][-1]
    assert [x["step"] for x in r["records"]] == [1, 75, 150, 225, 300] and last["loss"] < 1e-3 * first["loss"] and r["weight_error"] < 0.01
    assert first["top_energy"] > 0.99 and first["effective_rank"] < 4.5 and len(first["singular_values"]) == 24
    assert all(x["top_energy"] > 0.9 for x in r["records"]) and last["effective_rank"] < 2.0      # never far from rank 4, collapsing at the end
