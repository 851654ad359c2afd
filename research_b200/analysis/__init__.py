"""Model- and data-analysis utilities of the reference's dev tree: outlier-feature statistics of the residual stream
(dev/outlier-features) and distance from model outputs to a text corpus (dev/corpus-proximity)."""

from .corpus_proximity import (CorpusIndex, chunk_text, cluster_recursively, contamination_report, hashed_ngram_embedding)
from .outlier_features import OutlierReport, collect_residual_stream, find_outlier_features, perplexity

__all__ = ["CorpusIndex", "chunk_text", "cluster_recursively", "contamination_report", "hashed_ngram_embedding", "OutlierReport",
           "collect_residual_stream", "find_outlier_features", "perplexity"]
