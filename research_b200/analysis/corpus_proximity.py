"""Distance from model outputs to a text corpus (dev/corpus-proximity: chunking.py, search.py, cluster_corpus.py and the
GSM8K contamination analysis): chunk the corpus, embed the chunks, answer nearest-chunk queries under several
metrics, summarise how close a set of generations / benchmark items lies to the corpus, and build a recursive
cluster taxonomy. The embedding is pluggable; the default is a hashed character-n-gram vector, which needs no model
download and already separates verbatim or near-verbatim overlap from unrelated text."""

from __future__ import annotations

import re
import zlib
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch

EmbedFn = Callable[[Sequence[str]], torch.Tensor]


def chunk_text(text: str, strategy: str = "sentences", size: int = 3, overlap: int = 1) -> list[str]:
    """``sentences``: windows of ``size`` sentences stepping ``size - overlap``; ``words``: windows of ``size`` words;
    ``paragraphs``: blank-line separated blocks."""
    if strategy == "paragraphs":
        return [p.strip() for p in re.split(r"\n\s*\n", text) if p.strip()]
    units = re.findall(r"[^.!?\n]+[.!?]?", text) if strategy == "sentences" else text.split()
    units = [u.strip() for u in units if u.strip()]
    step = max(size - overlap, 1)
    return [" ".join(units[i:i + size]) for i in range(0, max(len(units) - overlap, 1), step) if units[i:i + size]]


def hashed_ngram_embedding(texts: Sequence[str], dim: int = 1024, n: int = 4) -> torch.Tensor:
    """L2-normalised bag of hashed character n-grams (lower-cased, whitespace collapsed)."""
    out = torch.zeros(len(texts), dim)
    for r, t in enumerate(texts):
        s = " " + re.sub(r"\s+", " ", t.lower()).strip() + " "
        for i in range(max(len(s) - n + 1, 1)):
            out[r, zlib.crc32(s[i:i + n].encode()) % dim] += 1.0
    return torch.nn.functional.normalize(out, dim=-1)


@dataclass
class CorpusIndex:
    chunks: list[str]
    vectors: torch.Tensor
    embed: EmbedFn = hashed_ngram_embedding
    sources: list[str] = field(default_factory=list)       # optional provenance per chunk

    @staticmethod
    def build(documents: Sequence[str], embed: EmbedFn = hashed_ngram_embedding, names: Sequence[str] | None = None,
              **chunk_kw) -> "CorpusIndex":
        chunks, src = [], []
        for i, doc in enumerate(documents):
            cs = chunk_text(doc, **chunk_kw)
            chunks += cs
            src += [names[i] if names else f"doc{i}"] * len(cs)
        return CorpusIndex(chunks, embed(chunks), embed, src)

    def search(self, queries: Sequence[str], k: int = 3, metric: str = "cosine") -> list[list[tuple[float, int]]]:
        """Per query the ``k`` nearest chunks as (distance, chunk index), nearest first."""
        q = self.embed(list(queries))
        if metric == "cosine":
            dist = 1.0 - torch.nn.functional.normalize(q, dim=-1) @ torch.nn.functional.normalize(self.vectors, dim=-1).T
        elif metric in ("euclidean", "manhattan"):
            dist = torch.cdist(q, self.vectors, p=2.0 if metric == "euclidean" else 1.0)
        else:
            raise ValueError(f"unknown metric {metric!r}")
        k = min(k, len(self.chunks))
        vals, idx = dist.topk(k, dim=-1, largest=False)
        return [[(float(v), int(i)) for v, i in zip(vr, ir)] for vr, ir in zip(vals, idx)]


def contamination_report(index: CorpusIndex, items: Sequence[str], threshold: float = 0.35, metric: str = "cosine") -> dict:
    """How close benchmark items (or generations) lie to the corpus: nearest distance per item, the share under
    ``threshold`` ("likely seen"), and the nearest chunk with its source for inspection."""
    hits = index.search(items, k=1, metric=metric)
    nearest = [h[0] for h in hits]
    dists = torch.tensor([d for d, _ in nearest])
    return {"n": len(items), "mean_distance": float(dists.mean()), "median_distance": float(dists.median()),
            "contaminated_fraction": float((dists < threshold).float().mean()),
            "items": [{"text": t, "distance": d, "nearest_chunk": index.chunks[i], "source": index.sources[i] if index.sources else ""}
                      for t, (d, i) in zip(items, nearest)]}


def cluster_recursively(vectors: torch.Tensor, max_depth: int = 3, branching: int = 4, min_size: int = 8, seed: int = 0,
                        _ids: torch.Tensor | None = None, _depth: int = 0) -> dict:
    """Hierarchy of k-means clusters: ``{"ids": [...], "centroid": tensor, "children": [...]}``; a node is split while it
    has at least ``min_size`` members and depth remains (the reference uses UMAP + HDBSCAN at each level)."""
    ids = _ids if _ids is not None else torch.arange(vectors.shape[0])
    x = vectors[ids]
    node = {"ids": ids.tolist(), "centroid": x.mean(0), "children": []}
    if _depth >= max_depth or len(ids) < max(min_size, branching):
        return node
    g = torch.Generator().manual_seed(seed + _depth)
    cent = x[torch.randperm(len(ids), generator=g)[:branching]].clone()
    for _ in range(20):
        assign = torch.cdist(x, cent).argmin(-1)
        for c in range(branching):
            if (assign == c).any():
                cent[c] = x[assign == c].mean(0)
    for c in range(branching):
        members = ids[assign == c]
        if 0 < len(members) < len(ids):
            node["children"].append(cluster_recursively(vectors, max_depth, branching, min_size, seed, members, _depth + 1))
    return node
