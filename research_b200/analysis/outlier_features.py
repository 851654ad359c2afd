"""Outlier features of the residual stream, after Dettmers et al. 2022 as applied in dev/outlier-features/
analyze_activations.py: a hidden dimension is an outlier feature when its magnitude reaches ``magnitude`` (6.0) in at
least ``min_layer_frac`` (25 %) of the layers and ``min_token_frac`` (6 %) of the sequence positions."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class OutlierReport:
    dims: list[int]                                  # hidden dimensions that qualify
    layer_frac: dict[int, float]                     # dim -> fraction of layers in which it crosses the threshold
    token_frac: dict[int, float]                     # dim -> fraction of (layer, position) cells in which it does
    max_abs: dict[int, float]
    per_layer_counts: list[int] = field(default_factory=list)   # qualifying dims seen crossing in each layer
    seq_frac: dict[int, float] = field(default_factory=dict)    # dim -> fraction of positions hit in at least one layer
    layer_names: list[str] = field(default_factory=list)
    layer_max: list[float] = field(default_factory=list)        # largest magnitude seen in each layer (any dimension)

    def to_records(self) -> list[dict]:
        """One JSON-able record per outlier feature, largest magnitude first."""
        return sorted(({"feature_dim": d, "layer_percentage": self.layer_frac[d], "seq_percentage": self.seq_frac.get(d, self.token_frac[d]),
                        "cell_percentage": self.token_frac[d], "max_magnitude": self.max_abs[d]} for d in self.dims),
                      key=lambda r: r["max_magnitude"], reverse=True)

    def summary(self) -> str:
        head = f"{len(self.dims)} outlier feature(s)"
        rows = [f"  dim {d}: {self.layer_frac[d]:.0%} of layers, {self.token_frac[d]:.1%} of positions, max |x| {self.max_abs[d]:.1f}"
                for d in self.dims]
        return "\n".join([head, *rows])


def find_outlier_features(activations: dict[str, torch.Tensor] | list[torch.Tensor], magnitude: float = 6.0,
                          min_layer_frac: float = 0.25, min_token_frac: float = 0.06, criterion: str = "cells") -> OutlierReport:
    """``activations``: one ``[..., hidden]`` tensor per layer (leading dimensions are flattened into positions).

    ``criterion`` picks what the 6 % applies to: ``"cells"`` = the fraction of (layer, position) cells in which the
    dimension crosses the threshold (strict), ``"positions"`` = the fraction of positions in which it crosses it in at
    least one layer (the reading of dev/outlier-features/analyze_activations.py:143-219). Both fractions are reported."""
    assert criterion in ("cells", "positions")
    names = list(activations) if isinstance(activations, dict) else [f"layer.{i}" for i in range(len(activations))]
    layers = list(activations.values()) if isinstance(activations, dict) else list(activations)
    assert layers, "no activations"
    d = layers[0].shape[-1]
    layer_hits = torch.zeros(d)
    token_hits = torch.zeros(d)
    max_abs = torch.zeros(d)
    positions = 0
    crossing, layer_max = [], []
    pos_hit = None
    for x in layers:
        a = x.detach().float().reshape(-1, d).abs()
        over = a >= magnitude
        crossing.append(over.any(0))
        layer_hits += over.any(0).float()
        token_hits += over.float().sum(0)
        max_abs = torch.maximum(max_abs, a.max(0).values)
        layer_max.append(float(a.max()))
        positions += a.shape[0]
        pos_hit = over if pos_hit is None or pos_hit.shape != over.shape else pos_hit | over
    lf, tf = layer_hits / len(layers), token_hits / max(positions, 1)
    sf = pos_hit.float().mean(0)
    keep = (lf >= min_layer_frac) & ((tf if criterion == "cells" else sf) >= min_token_frac)
    dims = [int(i) for i in torch.nonzero(keep).flatten()]
    sel = torch.tensor(dims, dtype=torch.long)
    return OutlierReport(dims, {i: float(lf[i]) for i in dims}, {i: float(tf[i]) for i in dims}, {i: float(max_abs[i]) for i in dims},
                         [int(c[sel].sum()) if dims else 0 for c in crossing], {i: float(sf[i]) for i in dims}, names, layer_max)


def collect_residual_stream(input_ids: torch.Tensor, weights: dict[str, torch.Tensor], cfg) -> dict[str, torch.Tensor]:
    """Residual stream after the embedding and after every layer (``[B, T, hidden]`` each) from the functional model."""
    from ..models import causal_lm_forward

    trace: dict[str, torch.Tensor] = {}
    causal_lm_forward(input_ids, weights, cfg, trace=trace)
    return {k: v for k, v in trace.items() if k == "embed" or k.startswith("layer.")}


def perplexity(input_ids: torch.Tensor, weights: dict[str, torch.Tensor], cfg) -> float:
    """exp(mean next-token negative log-likelihood) of ``input_ids [B, T]`` under the functional model
    (dev/outlier-features/compute_perplexity.py)."""
    from ..models import causal_lm_forward

    logits = causal_lm_forward(input_ids, weights, cfg).float()
    lp = torch.log_softmax(logits[:, :-1], -1).gather(-1, input_ids[:, 1:, None].long()).squeeze(-1)
    return float(torch.exp(-lp.mean()))


# ------------------------------------------------------------------------------------------- text -> sequences
def chunk_text_by_chars(text: str, chunk_size: int) -> list[str]:
    """Pieces of at most ``chunk_size`` characters, cut at the last whitespace before the limit where there is one."""
    assert chunk_size > 0
    out, i, n = [], 0, len(text)
    while i < n:
        j = min(i + chunk_size, n)
        if j < n:
            k = text.rfind(" ", i + chunk_size // 2, j)
            j = k if k > i else j
        piece = text[i:j].strip()
        if piece:
            out.append(piece)
        i = j
    return out


def chunk_ids(ids: list[int], seq_len: int, stride: int | None = None, drop_last: bool = True) -> list[list[int]]:
    """Windows of ``seq_len`` tokens every ``stride`` tokens (default: no overlap); a short tail is dropped unless asked."""
    stride = stride or seq_len
    out = [ids[i:i + seq_len] for i in range(0, max(len(ids) - seq_len + 1, 1), stride)]
    if not drop_last and len(ids) > seq_len and (len(ids) - seq_len) % stride:
        out.append(ids[-seq_len:])
    return [w for w in out if len(w) == seq_len or not drop_last]


def get_token_sequences(texts, tokenizer, num_sequences: int, seq_len: int) -> torch.Tensor:
    """``[num_sequences, seq_len]`` token ids: documents are tokenised, joined with the end-of-text token between them, and
    cut into full windows, taking documents until there are enough (dev/outlier-features/dataset_utils.py:137-237)."""
    eos = getattr(tokenizer, "eos_token_id", None)
    buf: list[int] = []
    rows: list[list[int]] = []
    for t in texts:
        buf += list(tokenizer.encode(t)) + ([eos] if eos is not None else [])
        while len(buf) >= seq_len and len(rows) < num_sequences:
            rows.append(buf[:seq_len])
            buf = buf[seq_len:]
        if len(rows) >= num_sequences:
            break
    assert rows, f"the texts hold fewer than {seq_len} tokens"
    return torch.tensor(rows, dtype=torch.long)


# ------------------------------------------------------------------------------------------- batches -> a run
def analyze_batch(input_ids: torch.Tensor, weights, cfg, magnitude: float = 6.0, min_layer_frac: float = 0.25, min_token_frac: float = 0.06,
                  criterion: str = "positions") -> dict:
    """One batch through the model: its outlier records, per-layer maxima and perplexity."""
    stream = collect_residual_stream(input_ids, weights, cfg)
    rep = find_outlier_features(stream, magnitude, min_layer_frac, min_token_frac, criterion)
    return {"outliers": rep.to_records(), "layer_max": dict(zip(rep.layer_names, rep.layer_max)), "num_tokens": int(input_ids.numel()),
            "perplexity": perplexity(input_ids, weights, cfg)}


def aggregate_batch_results(batches: list[dict], min_batch_frac: float = 0.5) -> dict:
    """A dimension is a SYSTEMATIC outlier of the model when it qualifies in at least ``min_batch_frac`` of the batches
    (what depends on one text is noise). Magnitudes and fractions are averaged over the batches where it appears; the
    perplexity is the token-weighted geometric mean (dev/outlier-features/run_full_analysis.py:259-320)."""
    import math

    assert batches, "no batch results"
    seen: dict[int, list[dict]] = {}
    for b in batches:
        for r in b["outliers"]:
            seen.setdefault(int(r["feature_dim"]), []).append(r)
    systematic = []
    for dim, recs in seen.items():
        if len(recs) / len(batches) >= min_batch_frac:
            systematic.append({"feature_dim": dim, "batch_percentage": len(recs) / len(batches),
                               "max_magnitude": max(r["max_magnitude"] for r in recs),
                               "mean_magnitude": sum(r["max_magnitude"] for r in recs) / len(recs),
                               "layer_percentage": sum(r["layer_percentage"] for r in recs) / len(recs),
                               "seq_percentage": sum(r["seq_percentage"] for r in recs) / len(recs)})
    systematic.sort(key=lambda r: r["max_magnitude"], reverse=True)
    tokens = sum(b["num_tokens"] for b in batches)
    log_ppl = sum(math.log(b["perplexity"]) * b["num_tokens"] for b in batches) / max(tokens, 1)
    layer_max: dict[str, float] = {}
    for b in batches:
        for k, v in b["layer_max"].items():
            layer_max[k] = max(layer_max.get(k, 0.0), v)
    return {"num_batches": len(batches), "num_tokens": tokens, "systematic_outliers": systematic, "num_systematic": len(systematic),
            "candidate_dims": len(seen), "perplexity": math.exp(log_ppl), "layer_max": layer_max}


def run_analysis(weights, cfg, input_ids: torch.Tensor, batch_size: int = 2, model_name: str = "", out_dir=None, **criteria) -> dict:
    """All of it for one model: batches of ``input_ids`` -> per-batch results -> the aggregate, optionally written to
    ``<out_dir>/final_analysis_results.json`` (the file ``compare_results`` collects)."""
    import json
    from pathlib import Path

    batches = [analyze_batch(input_ids[i:i + batch_size], weights, cfg, **criteria) for i in range(0, input_ids.shape[0], batch_size)]
    result = {"model": model_name or getattr(cfg, "family", "model"), "num_params": cfg.num_params(), "hidden_size": cfg.hidden_size,
              "num_layers": cfg.num_layers, "sequence_length": int(input_ids.shape[1]), **aggregate_batch_results(batches),
              "batch_results": batches}
    if out_dir is not None:
        Path(out_dir).mkdir(parents=True, exist_ok=True)
        (Path(out_dir) / "final_analysis_results.json").write_text(json.dumps(result, indent=2))
    return result


# ------------------------------------------------------------------------------------------- comparing runs
def collect_results(results_dir) -> list[dict]:
    """One row per ``final_analysis_results.json`` found under ``results_dir``: model, size, number of systematic
    outliers, their mean magnitude and coverage, perplexity. Sorted by parameter count."""
    import json
    from pathlib import Path

    rows = []
    for f in sorted(Path(results_dir).rglob("final_analysis_results.json")):
        try:
            r = json.loads(f.read_text())
        except ValueError:
            continue
        so = r.get("systematic_outliers", [])
        mean = (lambda key: sum(o[key] for o in so) / len(so) if so else 0.0)
        rows.append({"model": r.get("model", f.parent.name), "num_params": r.get("num_params", 0), "num_outliers": len(so),
                     "mean_magnitude": mean("mean_magnitude"), "max_magnitude": max((o["max_magnitude"] for o in so), default=0.0),
                     "mean_layer_pct": 100 * mean("layer_percentage"), "mean_seq_pct": 100 * mean("seq_percentage"),
                     "perplexity": r.get("perplexity"), "path": str(f)})
    return sorted(rows, key=lambda r: r["num_params"])


def format_table(rows: list[dict]) -> str:
    head = f"{'model':<24}{'params':>10}{'outliers':>10}{'mean |x|':>10}{'max |x|':>10}{'layers %':>10}{'seq %':>8}{'ppl':>10}"
    def size(n: float) -> str:
        return f"{n / 1e9:.1f}B" if n >= 1e9 else f"{n / 1e6:.0f}M" if n >= 1e6 else f"{n / 1e3:.0f}K"
    body = [f"{r['model'][:23]:<24}{size(r['num_params']):>10}{r['num_outliers']:>10}{r['mean_magnitude']:>10.1f}{r['max_magnitude']:>10.1f}"
            f"{r['mean_layer_pct']:>10.0f}{r['mean_seq_pct']:>8.0f}{(r['perplexity'] or 0):>10.1f}" for r in rows]
    return "\n".join([head, "-" * len(head), *body])


def to_csv(rows: list[dict]) -> str:
    import csv
    import io

    buf = io.StringIO()
    cols = ["model", "num_params", "num_outliers", "mean_magnitude", "max_magnitude", "mean_layer_pct", "mean_seq_pct", "perplexity"]
    w = csv.DictWriter(buf, cols, extrasaction="ignore")
    w.writeheader()
    w.writerows(rows)
    return buf.getvalue()


def terminal_plot(rows: list[dict], y: str = "num_outliers", width: int = 60, height: int = 12) -> str:
    """Scatter of ``y`` against log10(parameters), one letter per model, for a look at the trend without a plotting stack."""
    import math

    pts = [(math.log10(max(r["num_params"], 1)), float(r[y] or 0.0), r["model"]) for r in rows]
    if not pts:
        return "(no results)"
    x0, x1 = min(p[0] for p in pts), max(p[0] for p in pts)
    y0, y1 = min(p[1] for p in pts), max(p[1] for p in pts)
    grid = [[" "] * width for _ in range(height)]
    legend = []
    for i, (x, v, name) in enumerate(pts):
        c = chr(ord("a") + i % 26)
        col = int((x - x0) / (x1 - x0) * (width - 1)) if x1 > x0 else width // 2
        row = height - 1 - (int((v - y0) / (y1 - y0) * (height - 1)) if y1 > y0 else height // 2)
        grid[row][col] = c
        legend.append(f"{c}={name}")
    lines = [f"{y} ({y0:g} .. {y1:g}) vs log10(params) ({x0:.1f} .. {x1:.1f})"] + ["|" + "".join(r) for r in grid] + ["+" + "-" * width, "  ".join(legend)]
    return "\n".join(lines)


# ------------------------------------------------------------------------------------------- memory estimate
DTYPE_BYTES = {"float32": 4, "fp32": 4, "bfloat16": 2, "bf16": 2, "float16": 2, "fp16": 2, "fp8": 1, "int8": 1, "nvfp4": 0.5625, "int4": 0.5}


def params_from_hf_config(config: dict) -> tuple[int, str]:
    """Parameter count from a ``config.json`` dict (dense and mixture-of-experts decoders) and a line that says how it
    was obtained (dev/outlier-features/estimate_vram.py:63-176)."""
    from ..models.config import ModelConfig

    cfg = ModelConfig.from_hf_dict(config)
    kind = f"{cfg.num_experts} experts x {cfg.moe_intermediate_size}" if cfg.is_moe else f"dense, intermediate {cfg.intermediate_size}"
    return cfg.num_params(), f"{cfg.num_layers} layers x hidden {cfg.hidden_size}, {kind}, vocab {cfg.vocab_size}"


def estimate_vram(cfg, dtype: str = "bfloat16", batch_size: int = 1, seq_len: int = 2048, mode: str = "inference", num_gpus: int = 1,
                  keep_activations_of_layers: int | None = None, gpu_gb: float = 180.0, overhead: float = 0.1) -> dict:
    """Memory a run needs, in GB, by component. ``mode``: ``inference`` (weights + KV cache + one layer's activations),
    ``analysis`` (the residual stream of every layer is kept, in fp32, as the outlier analysis does) or ``training``
    (weights, fp32 master copy, two AdamW moments, gradients, activations of every layer for the backward pass).
    Weights, optimizer state and KV cache divide over ``num_gpus``; activations of a data-parallel shard do not."""
    import math

    assert mode in ("inference", "analysis", "training")
    b = DTYPE_BYTES[dtype]
    n = cfg.num_params()
    gb = 1 / 1e9
    weights = n * b * gb / num_gpus
    kv = 2 * cfg.num_layers * batch_size * seq_len * cfg.num_kv_heads * cfg.head_dim * b * gb / num_gpus if mode == "inference" else 0.0
    tokens = batch_size * seq_len
    inter = cfg.moe_intermediate_size * cfg.num_experts_per_tok if cfg.is_moe else cfg.intermediate_size
    per_layer = tokens * (4 * cfg.hidden_size + 2 * cfg.q_size // max(cfg.hidden_size, 1) * cfg.hidden_size + 3 * inter) * b * gb
    logits = tokens * cfg.vocab_size * 4 * gb
    if mode == "training":
        layers_kept = cfg.num_layers if keep_activations_of_layers is None else keep_activations_of_layers
        acts = per_layer * layers_kept + logits
        optimizer = n * (4 + 4 + 4) * gb / num_gpus              # fp32 master + two moments
        grads = n * b * gb / num_gpus
    elif mode == "analysis":
        acts = per_layer + (cfg.num_layers + 1) * tokens * cfg.hidden_size * 4 * gb + logits
        optimizer = grads = 0.0
    else:
        acts = per_layer + batch_size * cfg.vocab_size * 4 * gb   # logits of the last position only
        optimizer = grads = 0.0
    subtotal = weights + kv + acts + optimizer + grads
    total = subtotal * (1 + overhead)
    sharded_total = (weights + kv + optimizer + grads) * num_gpus * (1 + overhead)      # what divides over more GPUs
    room = gpu_gb - acts * (1 + overhead)                                                # what one GPU has left for its share
    min_gpus = max(1, math.ceil(sharded_total / room)) if room > 0 else None             # None: the activations alone do not fit
    return {"params_b": n / 1e9, "weights_gb": weights, "kv_cache_gb": kv, "activations_gb": acts, "optimizer_gb": optimizer, "gradients_gb": grads,
            "overhead_gb": subtotal * overhead, "total_gb_per_gpu": total, "fits": total <= gpu_gb, "gpu_gb": gpu_gb,
            "min_gpus": min_gpus}


def format_vram(est: dict) -> str:
    rows = [("weights", "weights_gb"), ("KV cache", "kv_cache_gb"), ("activations", "activations_gb"), ("optimizer state", "optimizer_gb"),
            ("gradients", "gradients_gb"), ("allocator / workspace", "overhead_gb")]
    lines = [f"{est['params_b']:.2f} B parameters"] + [f"  {name:<22}{est[key]:>9.2f} GB" for name, key in rows if est[key] > 0]
    lines.append(f"  {'total per GPU':<22}{est['total_gb_per_gpu']:>9.2f} GB  ({'fits in' if est['fits'] else 'does NOT fit in'} {est['gpu_gb']:g} GB; "
                 + (f"at least {est['min_gpus']} GPU(s) of that size)" if est["min_gpus"] else "the activations of one shard alone exceed it: lower batch or sequence length)"))
    return "\n".join(lines)


def main(argv=None) -> int:
    """``python -m research_b200.analysis.outlier_features vram --model llama-3-8b --mode training --seq-len 4096``
    ``python -m research_b200.analysis.outlier_features compare results/ [--csv | --plot num_outliers]``
    ``python -m research_b200.analysis.outlier_features run --model tiny-qwen2 --num-sequences 8 --seq-len 64 --out results/tiny``"""
    import argparse

    from ..models import get_preset, init_random_weights

    ap = argparse.ArgumentParser(prog="outlier_features")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("vram")
    p.add_argument("--model", required=True); p.add_argument("--dtype", default="bfloat16"); p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--seq-len", type=int, default=2048); p.add_argument("--mode", default="inference", choices=["inference", "analysis", "training"])
    p.add_argument("--num-gpus", type=int, default=1); p.add_argument("--gpu-gb", type=float, default=180.0)
    p = sub.add_parser("compare")
    p.add_argument("results_dir"); p.add_argument("--csv", action="store_true"); p.add_argument("--plot", default="")
    p = sub.add_parser("run")
    p.add_argument("--model", required=True); p.add_argument("--num-sequences", type=int, default=8); p.add_argument("--seq-len", type=int, default=128)
    p.add_argument("--batch-size", type=int, default=2); p.add_argument("--out", default=""); p.add_argument("--seed", type=int, default=0)
    p.add_argument("--magnitude", type=float, default=6.0)
    a = ap.parse_args(argv)
    if a.cmd == "vram":
        print(format_vram(estimate_vram(get_preset(a.model), a.dtype, a.batch_size, a.seq_len, a.mode, a.num_gpus, gpu_gb=a.gpu_gb)))
    elif a.cmd == "compare":
        rows = collect_results(a.results_dir)
        print(to_csv(rows) if a.csv else terminal_plot(rows, a.plot) if a.plot else format_table(rows))
    else:
        cfg = get_preset(a.model)
        ids = torch.randint(0, cfg.vocab_size, (a.num_sequences, a.seq_len), generator=torch.Generator().manual_seed(a.seed))
        r = run_analysis(init_random_weights(cfg, seed=a.seed), cfg, ids, a.batch_size, a.model, a.out or None, magnitude=a.magnitude)
        print(f"{r['model']}: {r['num_systematic']} systematic outlier feature(s) out of {r['candidate_dims']} candidates, perplexity {r['perplexity']:.1f}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
