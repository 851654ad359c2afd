"""Radix-tree prefix cache (SGLang style), backed by the C++ engine core.

The reference only sketches this class: ``RadixKVCache.__init__`` raises
``NotImplementedError`` (rollouts/inference/cache/radix.py:42-43). Here it is real: a
block-granular radix tree with edge splitting, per-path pin counts while sequences use a
prefix, and LRU eviction of unpinned leaves when the pool runs dry. Finished sequences publish
their blocks (prompt and generated tokens) into the tree on ``deallocate``.
"""

from __future__ import annotations

from .paged import MODE_RADIX, PagedKVCache


class RadixKVCache(PagedKVCache):
    _mode = MODE_RADIX
