"""The second half of the corpus-proximity study (dev/corpus-proximity: chunking.py, cluster_corpus.py, name_clusters.py,
annotation.py, formatting.py, gsm8k_corpus_similarity.py): more ways to cut a corpus into chunks, a cluster TREE over the
chunk embeddings with coherence scores and noise points, names for the clusters written by a language model, and
annotation of a model's output sentence by sentence with the nearest training cluster ("this sentence sits 0.12 away
from 'grade-school word problems' in the SFT mix").

Everything numeric is torch on CPU; the clustering at each level is k-means with the number of clusters chosen by
silhouette score, and members far from every centroid are set aside as noise (the reference reduces with UMAP and
clusters with HDBSCAN, neither of which is available here; the tree, its ids and what is stored are the same).
"""

from __future__ import annotations

import asyncio
import json
import re
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Awaitable, Callable, Sequence

import torch

from .corpus_proximity import CorpusIndex, EmbedFn, hashed_ngram_embedding


# ------------------------------------------------------------------------------------------- chunking
_ABBREVIATIONS = {"mr", "mrs", "ms", "dr", "prof", "vs", "etc", "e.g", "i.e", "no", "fig", "st", "jr", "sr", "inc", "approx"}


def split_into_sentences(text: str) -> list[str]:
    """Sentence boundaries at ``. ! ?`` followed by whitespace and an upper-case letter, digit or quote; common
    abbreviations and decimal points do not end a sentence."""
    text = re.sub(r"\s+", " ", text).strip()
    if not text:
        return []
    parts = re.split(r"(?:(?<=[.!?])|(?<=[.!?][\"')\]]))\s+(?=[\"'(\[]*[A-Z0-9])", text)
    out: list[str] = []
    for p in parts:
        if out and out[-1].rsplit(" ", 1)[-1].lower().rstrip(".") in _ABBREVIATIONS and out[-1].endswith("."):
            out[-1] += " " + p.strip()                                  # "Dr." / "e.g." did not end the sentence
        elif p.strip():
            out.append(p.strip())
    return out


def chunk_paragraphs(text: str, min_chars: int = 1) -> list[str]:
    return [p.strip() for p in re.split(r"\n\s*\n", text) if len(p.strip()) >= min_chars]


def chunk_fixed_chars(text: str, size: int, overlap_pct: float = 0.15) -> list[str]:
    """Windows of ``size`` characters that overlap by ``overlap_pct`` and start / end at word boundaries where possible."""
    assert size > 0 and 0 <= overlap_pct < 1
    text = text.strip()
    step = max(int(size * (1 - overlap_pct)), 1)
    out, i, n = [], 0, len(text)
    while i < n:
        j = min(i + size, n)
        if j < n:
            k = text.rfind(" ", i + size // 2, j)
            j = k if k > i else j
        piece = text[i:j].strip()
        if piece:
            out.append(piece)
        if j >= n:
            break
        nxt = i + step
        sp = text.find(" ", nxt, j)
        i = sp + 1 if sp >= 0 else max(nxt, i + 1)
    return out


def chunk_fixed_tokens(text: str, tokenizer: Any, size: int, overlap_pct: float = 0.15) -> list[str]:
    """Windows of ``size`` tokens (overlapping by ``overlap_pct``), decoded back to text."""
    ids = list(tokenizer.encode(text))
    step = max(int(size * (1 - overlap_pct)), 1)
    out = []
    for i in range(0, max(len(ids), 1), step):
        window = ids[i:i + size]
        if window:
            out.append(tokenizer.decode(window).strip())
        if i + size >= len(ids):
            break
    return [c for c in out if c]


def chunk(text: str, strategy: str = "paragraph", size: int = 512, overlap_pct: float = 0.15, tokenizer: Any = None) -> list[str]:
    if strategy == "paragraph":
        return chunk_paragraphs(text)
    if strategy == "sentence":
        return split_into_sentences(text)
    if strategy == "fixed_chars":
        return chunk_fixed_chars(text, size, overlap_pct)
    if strategy == "fixed_tokens":
        assert tokenizer is not None, "fixed_tokens needs a tokenizer"
        return chunk_fixed_tokens(text, tokenizer, size, overlap_pct)
    raise ValueError(f"unknown chunking strategy {strategy!r}: paragraph | sentence | fixed_chars | fixed_tokens")


# ------------------------------------------------------------------------------------------- the cluster tree
@dataclass
class ClusterNode:
    cluster_id: str                          # "0", "0.1", "0.1.2": the path from the root
    depth: int
    parent_id: str | None
    indices: list[int]                       # members, as indices into the embedded chunks
    centroid: torch.Tensor
    silhouette: float = 0.0                  # coherence of the split BELOW this node (0 for leaves), in [0, 1]
    children: list["ClusterNode"] = field(default_factory=list)
    noise_indices: list[int] = field(default_factory=list)   # members that belong to none of the children
    name: str = ""

    @property
    def size(self) -> int:
        return len(self.indices)

    def walk(self):
        yield self
        for c in self.children:
            yield from c.walk()


def _kmeans(x: torch.Tensor, k: int, seed: int, iters: int = 25) -> tuple[torch.Tensor, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    cent = x[torch.randint(0, x.shape[0], (1,), generator=g)].clone()
    for _ in range(1, k):                                              # k-means++ seeding: far points first
        d2 = torch.cdist(x, cent).min(1).values ** 2
        if float(d2.sum()) <= 0:
            break
        cent = torch.cat([cent, x[torch.multinomial(d2 / d2.sum(), 1, generator=g)]])
    for _ in range(iters):
        assign = torch.cdist(x, cent).argmin(1)
        new = torch.stack([x[assign == c].mean(0) if (assign == c).any() else cent[c] for c in range(cent.shape[0])])
        if torch.allclose(new, cent, atol=1e-6):
            break
        cent = new
    return torch.cdist(x, cent).argmin(1), cent


def silhouette_score(x: torch.Tensor, assign: torch.Tensor) -> float:
    """Mean silhouette coefficient, clipped to [0, 1] (negative means the split is worse than none)."""
    labels = assign.unique()
    if len(labels) < 2 or x.shape[0] < 3:
        return 0.0
    d = torch.cdist(x, x)
    scores = []
    for i in range(x.shape[0]):
        same = assign == assign[i]
        if same.sum() <= 1:
            scores.append(0.0)
            continue
        a = float(d[i][same].sum() / (same.sum() - 1))
        b = min(float(d[i][assign == l].mean()) for l in labels if l != assign[i])
        scores.append((b - a) / max(a, b, 1e-12))
    return float(min(max(sum(scores) / len(scores), 0.0), 1.0))


def recursive_cluster(vectors: torch.Tensor, max_depth: int = 3, max_branching: int = 6, min_cluster_size: int = 6, min_silhouette: float = 0.05,
                      noise_quantile: float = 0.98, seed: int = 0, _indices: list[int] | None = None, _id: str = "0", _depth: int = 0,
                      _parent: str | None = None) -> ClusterNode:
    """Split a node with k-means, trying k = 2 .. ``max_branching`` and keeping the k with the best silhouette; stop when
    depth runs out, the node is small, or no split is coherent (``min_silhouette``). Members beyond the ``noise_quantile``
    of distance to their centroid are the node's noise points and go to no child."""
    idx = list(range(vectors.shape[0])) if _indices is None else _indices
    x = vectors[idx]
    node = ClusterNode(_id, _depth, _parent, idx, x.mean(0))
    if _depth >= max_depth or len(idx) < 2 * min_cluster_size:
        return node
    sample = x if x.shape[0] <= 400 else x[torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(seed))[:400]]
    best: tuple[float, int] | None = None
    for k in range(2, min(max_branching, len(idx) // min_cluster_size) + 1):
        a, _ = _kmeans(sample, k, seed + k)
        s = silhouette_score(sample, a)
        if best is None or s > best[0] + 1e-9:
            best = (s, k)
    if best is None or best[0] < min_silhouette:
        return node
    assign, cent = _kmeans(x, best[1], seed + best[1])
    node.silhouette = best[0]
    dist = (x - cent[assign]).norm(dim=1)
    cut = torch.quantile(dist, noise_quantile) if len(idx) >= 20 else dist.max() + 1
    child_no = 0
    for c in range(cent.shape[0]):
        members = [idx[i] for i in range(len(idx)) if assign[i] == c and dist[i] <= cut]
        if len(members) < min_cluster_size:
            node.noise_indices += [idx[i] for i in range(len(idx)) if assign[i] == c]
            continue
        node.noise_indices += [idx[i] for i in range(len(idx)) if assign[i] == c and dist[i] > cut]
        node.children.append(recursive_cluster(vectors, max_depth, max_branching, min_cluster_size, min_silhouette, noise_quantile, seed,
                                               members, f"{_id}.{child_no}", _depth + 1, _id))
        child_no += 1
    if len(node.children) < 2:                                         # one surviving child is not a split
        node.children, node.noise_indices, node.silhouette = [], [], 0.0
    return node


def build_chunk_to_cluster_map(tree: ClusterNode) -> dict[int, str]:
    """Chunk index -> id of the DEEPEST cluster that holds it (noise points stay with the node that set them aside)."""
    out: dict[int, str] = {}
    for node in tree.walk():                                           # parents before children: children overwrite
        for i in node.indices:
            out[i] = node.cluster_id
    return out


def get_max_depth(tree: ClusterNode) -> int:
    return max(n.depth for n in tree.walk())


def compute_cluster_stats(tree: ClusterNode) -> dict[str, Any]:
    nodes = list(tree.walk())
    leaves = [n for n in nodes if not n.children]
    split = [n for n in nodes if n.children]
    return {"total_clusters": len(nodes), "leaf_clusters": len(leaves), "max_depth": get_max_depth(tree),
            "mean_leaf_size": sum(n.size for n in leaves) / len(leaves), "noise_points": sum(len(n.noise_indices) for n in nodes),
            "mean_silhouette": sum(n.silhouette for n in split) / len(split) if split else 0.0,
            "clusters_per_depth": {d: sum(1 for n in nodes if n.depth == d) for d in range(get_max_depth(tree) + 1)}}


def find_node_by_id(tree: ClusterNode, cluster_id: str) -> ClusterNode | None:
    return next((n for n in tree.walk() if n.cluster_id == cluster_id), None)


def collect_nodes_at_depth(tree: ClusterNode, depth: int) -> list[ClusterNode]:
    return [n for n in tree.walk() if n.depth == depth]


def format_cluster_tree(tree: ClusterNode, max_depth: int | None = None) -> str:
    lines = []
    for n in tree.walk():
        if max_depth is not None and n.depth > max_depth:
            continue
        extra = f", silhouette {n.silhouette:.2f}" if n.children else ""
        extra += f", {len(n.noise_indices)} noise" if n.noise_indices else ""
        lines.append(f"{'  ' * n.depth}[{n.cluster_id}] {n.name or '(unnamed)'}  ({n.size} chunks{extra})")
    return "\n".join(lines)


def tree_to_dict(node: ClusterNode) -> dict[str, Any]:
    return {"cluster_id": node.cluster_id, "depth": node.depth, "parent_id": node.parent_id, "indices": node.indices, "size": node.size,
            "silhouette": node.silhouette, "noise_indices": node.noise_indices, "name": node.name, "centroid": node.centroid.tolist(),
            "children": [tree_to_dict(c) for c in node.children]}


def tree_from_dict(d: dict[str, Any]) -> ClusterNode:
    return ClusterNode(d["cluster_id"], d["depth"], d.get("parent_id"), list(d["indices"]), torch.tensor(d["centroid"]), d.get("silhouette", 0.0),
                       [tree_from_dict(c) for c in d.get("children", [])], list(d.get("noise_indices", [])), d.get("name", ""))


# ------------------------------------------------------------------------------------------- names from a model
Complete = Callable[[str], Awaitable[str]]

NAME_PROMPT = """These text excerpts were grouped together automatically. Give the group a short descriptive name (2-6 words) that says
what the texts have in common, specific enough to tell it apart from its sibling groups.
{parent}{siblings}
Excerpts:
{samples}

Answer with the name only."""


def sample_cluster_texts(node: ClusterNode, vectors: torch.Tensor, texts: Sequence[str], k: int = 5, strategy: str = "centroid", seed: int = 0) -> list[str]:
    """``centroid``: the ``k`` members nearest the cluster's centre (its most typical texts); ``random``: any ``k``."""
    assert strategy in ("centroid", "random")
    if node.size <= k:
        return [texts[i] for i in node.indices]
    if strategy == "random":
        g = torch.Generator().manual_seed(seed)
        return [texts[node.indices[int(j)]] for j in torch.randperm(node.size, generator=g)[:k]]
    d = (vectors[node.indices] - node.centroid).norm(dim=1)
    return [texts[node.indices[int(j)]] for j in d.argsort()[:k]]


def _clean_name(reply: str) -> str:
    line = next((ln.strip() for ln in reply.strip().splitlines() if ln.strip()), "")
    line = re.sub(r"^(name|group|cluster)\s*:\s*", "", line, flags=re.I).strip(" \"'*`.")
    return " ".join(line.split()[:10])


async def name_cluster_tree(tree: ClusterNode, vectors: torch.Tensor, texts: Sequence[str], complete: Complete, samples_per_cluster: int = 5,
                            max_chars: int = 400, max_concurrent: int = 8, rename: bool = False) -> int:
    """Name every cluster, level by level (a child's prompt names its parent and the siblings that already have names, so
    names at one level differ). ``complete(prompt) -> text`` is any model call. Returns how many names were written;
    a failing call leaves that cluster unnamed and does not stop the rest."""
    sem = asyncio.Semaphore(max_concurrent)
    parents = {n.cluster_id: n for n in tree.walk()}
    written = 0

    async def one(node: ClusterNode) -> None:
        nonlocal written
        if node.name and not rename:
            return
        parent = parents.get(node.parent_id) if node.parent_id else None
        sibs = [c.name for c in parent.children if c is not node and c.name] if parent else []
        samples = sample_cluster_texts(node, vectors, texts, samples_per_cluster)
        prompt = NAME_PROMPT.format(parent=f"\nThe group is part of the larger group \"{parent.name}\".\n" if parent and parent.name else "",
                                    siblings=f"Sibling groups already named: {', '.join(sibs)}.\n" if sibs else "",
                                    samples="\n".join(f"{i + 1}. {s[:max_chars]}" for i, s in enumerate(samples)))
        async with sem:
            try:
                name = _clean_name(await complete(prompt))
            except Exception:  # noqa: BLE001 - one failed call must not lose the names already written
                return
        if name:
            node.name = name
            written += 1

    for depth in range(get_max_depth(tree) + 1):
        level = collect_nodes_at_depth(tree, depth)
        if depth == 0 or len(level) == 1:
            await asyncio.gather(*[one(n) for n in level])
        else:                                                           # siblings one after another (they read each other's names),
            groups: dict[str | None, list[ClusterNode]] = {}            # different families in parallel
            for n in level:
                groups.setdefault(n.parent_id, []).append(n)

            async def family(nodes: list[ClusterNode]) -> None:
                for n in nodes:
                    await one(n)

            await asyncio.gather(*[family(ns) for ns in groups.values()])
    return written


def inspect_cluster(tree: ClusterNode, cluster_id: str, vectors: torch.Tensor, texts: Sequence[str], k: int = 5) -> str:
    node = find_node_by_id(tree, cluster_id)
    if node is None:
        return f"no cluster {cluster_id!r}"
    lines = [f"[{node.cluster_id}] {node.name or '(unnamed)'}: {node.size} chunks, depth {node.depth}, {len(node.children)} children, "
             f"{len(node.noise_indices)} noise points", "most typical:"]
    lines += [f"  - {t[:200]}" for t in sample_cluster_texts(node, vectors, texts, k)]
    if node.noise_indices:
        lines += ["set aside as noise:"] + [f"  - {texts[i][:200]}" for i in node.noise_indices[:k]]
    if node.children:
        lines += ["children:"] + [f"  [{c.cluster_id}] {c.name or '(unnamed)'} ({c.size})" for c in node.children]
    return "\n".join(lines)


# ------------------------------------------------------------------------------------------- a clustered, stored index
@dataclass
class ClusteredCorpus:
    """A corpus index with its cluster tree and per-chunk metadata (e.g. ``{"corpus_stage": "sft"}``), saved to and loaded
    from one folder: ``embeddings.pt``, ``chunks.jsonl``, ``tree.json``."""

    index: CorpusIndex
    tree: ClusterNode
    metadata: list[dict[str, Any]]
    path: str = ""

    def __post_init__(self) -> None:
        self.chunk_to_cluster = build_chunk_to_cluster_map(self.tree)
        self._nodes = {n.cluster_id: n for n in self.tree.walk()}

    @staticmethod
    def build(documents: Sequence[str], stages: Sequence[str] | None = None, embed: EmbedFn = hashed_ngram_embedding, strategy: str = "sentence",
              size: int = 512, overlap_pct: float = 0.15, tokenizer: Any = None, **cluster_kw: Any) -> "ClusteredCorpus":
        chunks, meta = [], []
        for d, doc in enumerate(documents):
            for c in chunk(doc, strategy, size, overlap_pct, tokenizer):
                chunks.append(c)
                meta.append({"doc": d, "corpus_stage": stages[d] if stages else None})
        vectors = embed(chunks)
        index = CorpusIndex(chunks, vectors, embed, [str(m["corpus_stage"] or f"doc{m['doc']}") for m in meta])
        return ClusteredCorpus(index, recursive_cluster(vectors, **cluster_kw), meta)

    def cluster_info(self, cluster_id: str) -> dict[str, Any]:
        n = self._nodes.get(cluster_id)
        return {"name": n.name or "(unnamed)", "depth": n.depth, "size": n.size} if n else {"name": "unknown", "depth": 0, "size": 0}

    def save(self, folder: str | Path) -> Path:
        d = Path(folder)
        d.mkdir(parents=True, exist_ok=True)
        torch.save(self.index.vectors, d / "embeddings.pt")
        with open(d / "chunks.jsonl", "w") as f:
            for text, m in zip(self.index.chunks, self.metadata):
                f.write(json.dumps({"text": text, **m}) + "\n")
        (d / "tree.json").write_text(json.dumps(tree_to_dict(self.tree)))
        self.path = str(d)
        return d

    @staticmethod
    def load(folder: str | Path, embed: EmbedFn = hashed_ngram_embedding) -> "ClusteredCorpus":
        d = Path(folder)
        rows = [json.loads(line) for line in (d / "chunks.jsonl").read_text().splitlines() if line.strip()]
        vectors = torch.load(d / "embeddings.pt", weights_only=True)
        meta = [{k: v for k, v in r.items() if k != "text"} for r in rows]
        index = CorpusIndex([r["text"] for r in rows], vectors, embed, [str(m.get("corpus_stage") or f"doc{m.get('doc')}") for m in meta])
        return ClusteredCorpus(index, tree_from_dict(json.loads((d / "tree.json").read_text())), meta, str(d))


# ------------------------------------------------------------------------------------------- annotating model output
@dataclass
class ClusterAnnotation:
    text_span: str
    cluster_id: str
    cluster_name: str
    cluster_depth: int
    distance: float
    rank: int
    corpus_stage: str | None
    nearest_chunk_idx: int
    nearest_chunk_text: str
    avg_logprob: float | None = None


@dataclass
class AnnotatedOutput:
    prompt: str | None
    text: str
    annotations: list[ClusterAnnotation]
    k: int
    phrase_level: bool
    corpus_path: str = ""

    def to_dict(self) -> dict[str, Any]:
        return {"prompt": self.prompt, "text": self.text, "annotations": [asdict(a) for a in self.annotations],
                "annotation_metadata": {"k": self.k, "phrase_level": self.phrase_level, "corpus_path": self.corpus_path}}

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "AnnotatedOutput":
        m = d.get("annotation_metadata", {})
        return AnnotatedOutput(d.get("prompt"), d.get("text", ""), [ClusterAnnotation(**a) for a in d.get("annotations", [])], m.get("k", 0),
                               m.get("phrase_level", False), m.get("corpus_path", ""))


def annotate_text(corpus: ClusteredCorpus, text: str, k: int = 3, phrase_level: bool = True, prompt: str | None = None,
                  token_logprobs: Sequence[tuple[str, float]] | None = None, preview_chars: int = 200, metric: str = "cosine") -> AnnotatedOutput:
    """For every sentence of ``text`` (or for the whole text) the ``k`` nearest corpus chunks, each with the cluster it
    belongs to. ``token_logprobs`` (the generation's ``(token text, logprob)`` pairs in order) adds the model's mean
    log-probability over each sentence: low confidence far from the corpus and high confidence close to it are the two
    patterns the study looks for."""
    assert k > 0
    phrases = (split_into_sentences(text) or ([text] if text.strip() else [])) if phrase_level else ([text] if text.strip() else [])
    out = AnnotatedOutput(prompt, text, [], k, phrase_level, corpus.path)
    if not phrases:
        return out
    spans_lp: list[float | None] = [None] * len(phrases)
    if token_logprobs:
        pos, cursor = 0, 0
        joined = "".join(t for t, _ in token_logprobs)
        offsets = []
        for t, lp in token_logprobs:
            offsets.append((pos, pos + len(t), lp))
            pos += len(t)
        for i, ph in enumerate(phrases):
            at = joined.find(ph[:20], cursor)
            if at < 0:
                continue
            end = at + len(ph)
            lps = [lp for a, b, lp in offsets if a < end and b > at]
            spans_lp[i] = sum(lps) / len(lps) if lps else None
            cursor = end
    hits = corpus.index.search(phrases, k=k, metric=metric)
    for i, (ph, near) in enumerate(zip(phrases, hits)):
        for rank, (dist, idx) in enumerate(near, 1):
            cid = corpus.chunk_to_cluster.get(idx, "unknown")
            info = corpus.cluster_info(cid)
            out.annotations.append(ClusterAnnotation(ph, cid, info["name"], info["depth"], dist, rank, corpus.metadata[idx].get("corpus_stage"), idx,
                                                     corpus.index.chunks[idx][:preview_chars], spans_lp[i]))
    return out


def format_annotations(a: AnnotatedOutput, show_chunks: bool = False) -> str:
    lines = []
    if a.prompt:
        lines += [f"Prompt: {a.prompt}", ""]
    last = None
    for ann in a.annotations:
        if ann.text_span != last:
            conf = f"  (mean logprob {ann.avg_logprob:.2f})" if ann.avg_logprob is not None else ""
            lines.append(f'"{ann.text_span}"{conf}')
            last = ann.text_span
        stage = f", {ann.corpus_stage}" if ann.corpus_stage else ""
        lines.append(f"   {ann.rank}. {ann.cluster_name} [{ann.cluster_id}{stage}]  distance {ann.distance:.3f}")
        if show_chunks:
            lines.append(f"      nearest: {ann.nearest_chunk_text}")
    return "\n".join(lines)


def format_annotations_compact(a: AnnotatedOutput) -> str:
    """One line per sentence: the text, then its nearest cluster and distance."""
    return "\n".join(f"{ann.text_span}  -> {ann.cluster_name} ({ann.distance:.2f})" for ann in a.annotations if ann.rank == 1)


def similarity_by_stage(corpus: ClusteredCorpus, items: Sequence[str], metric: str = "cosine") -> dict[str, dict[str, float]]:
    """For benchmark items against a staged corpus (pre-training / mid-training / SFT mixes): per stage, the distance from
    each item to its nearest chunk OF THAT STAGE, summarised (dev/corpus-proximity/gsm8k_corpus_similarity.py). Which stage
    sits closest to the benchmark says where its look-alikes entered training."""
    stages = sorted({str(m.get("corpus_stage")) for m in corpus.metadata if m.get("corpus_stage") is not None})
    out = {}
    for st in stages:
        ids = [i for i, m in enumerate(corpus.metadata) if str(m.get("corpus_stage")) == st]
        sub = CorpusIndex([corpus.index.chunks[i] for i in ids], corpus.index.vectors[ids], corpus.index.embed)
        d = torch.tensor([h[0][0] for h in sub.search(items, k=1, metric=metric)])
        out[st] = {"chunks": len(ids), "mean": float(d.mean()), "median": float(d.median()), "min": float(d.min()), "p10": float(torch.quantile(d, 0.1)),
                   "max": float(d.max())}
    return out
