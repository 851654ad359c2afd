from .config import CacheConfig
from .layer import Attention
from .mask import (causal_mask, causal_mask_mod, document_causal_mask, make_document_mask_mod,
                   make_sliding_window_mask_mod, sliding_window_causal_mask)
from .paged_backend import PagedAttentionBackend
from .protocol import AttentionBackend

__all__ = ["CacheConfig", "Attention", "causal_mask", "causal_mask_mod", "document_causal_mask", "make_document_mask_mod",
           "make_sliding_window_mask_mod", "sliding_window_causal_mask", "PagedAttentionBackend", "AttentionBackend"]
