"""Builders that turn block tables into an ``InferenceContext`` (rollouts/inference/context.py:10-154)."""

from __future__ import annotations

from .cache.protocol import KVCacheManager
from .types import InferenceContext


def _slots(blocks: tuple[int, ...], start: int, end: int, block_size: int) -> list[int]:
    out = []
    for pos in range(start, end):
        bi = pos // block_size
        out.append(blocks[bi] * block_size + pos % block_size if bi < len(blocks) else -1)
    return out


def build_prefill_context(cache: KVCacheManager, seq_ids: list[int], seq_lens: list[int],
                          block_tables: list[tuple[int, ...]], cached_lens: list[int] | None = None) -> InferenceContext:
    """Slot mapping for every NEW token of every sequence (all tokens when nothing is cached)."""
    cached_lens = cached_lens or [0] * len(seq_lens)
    slot_mapping: list[int] = []
    for n, blocks, c in zip(seq_lens, block_tables, cached_lens):
        slot_mapping.extend(_slots(blocks, c, n, cache.block_size))
    return InferenceContext(
        is_prefill=True, slot_mapping=tuple(slot_mapping), block_tables=tuple(tuple(b) for b in block_tables),
        seq_lens=tuple(seq_lens), max_seq_len=max(seq_lens) if seq_lens else 0,
        query_lens=tuple(n - c for n, c in zip(seq_lens, cached_lens)))


def build_decode_context(cache: KVCacheManager, seq_ids: list[int], seq_lens: list[int],
                         block_tables: list[tuple[int, ...]]) -> InferenceContext:
    """One new token per sequence: its slot is the position ``seq_len - 1``."""
    slot_mapping = [_slots(blocks, n - 1, n, cache.block_size)[0] for n, blocks in zip(seq_lens, block_tables)]
    return InferenceContext(
        is_prefill=False, slot_mapping=tuple(slot_mapping), block_tables=tuple(tuple(b) for b in block_tables),
        seq_lens=tuple(seq_lens), max_seq_len=max(seq_lens) if seq_lens else 0,
        query_lens=tuple(1 for _ in seq_lens))


def allocate_and_build_context(cache: KVCacheManager, seq_id: int, token_ids: list[int]) -> tuple[InferenceContext, tuple[int, ...]]:
    blocks = cache.allocate(seq_id, token_ids)
    cached = cache.get_cached_tokens(seq_id)
    return build_prefill_context(cache, [seq_id], [len(token_ids)], [blocks], [cached]), blocks


def extend_and_build_context(cache: KVCacheManager, seq_id: int, new_token: int, current_len: int) -> InferenceContext:
    cache.append_token(seq_id, new_token)
    blocks = cache.get_block_ids(seq_id)
    return build_decode_context(cache, [seq_id], [current_len + 1], [blocks])
