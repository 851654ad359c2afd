"""Paged KV block manager with hash-chain prefix reuse, backed by the C++ engine core.

API of the reference's ``PagedKVCache`` (rollouts/inference/cache/paged.py:57-230). Differences
that are deliberate: a block that fills up during decode is published to the prefix index too
(the reference's ``append_token`` never detects a full block, cache/paged.py:194), and a prompt
that is cached in full still recomputes its last block so the step has logits to sample from.
"""

from __future__ import annotations

import ctypes
import struct

from ... import _native

MODE_NONE, MODE_HASH, MODE_RADIX = 0, 1, 2
_LL, _I = ctypes.c_longlong, ctypes.c_int


def _core():
    lib = _native.load("rb_engine_core")
    if not getattr(lib, "_rbk_typed", False):
        lib.rbk_create.restype = ctypes.c_void_p
        lib.rbk_create.argtypes = [_I, _I, _I]
        lib.rbe_destroy.argtypes = [ctypes.c_void_p]
        lib.rbk_allocate.argtypes = [ctypes.c_void_p, _LL, ctypes.c_void_p, _I, ctypes.c_void_p, _I, ctypes.c_void_p]
        lib.rbk_append_token.argtypes = [ctypes.c_void_p, _LL, _I]
        lib.rbk_deallocate.argtypes = [ctypes.c_void_p, _LL, _I]
        lib.rbk_get_blocks.argtypes = [ctypes.c_void_p, _LL, ctypes.c_void_p, _I]
        lib.rbk_cached_tokens.argtypes = [ctypes.c_void_p, _LL]
        lib.rbk_ref_count.argtypes = [ctypes.c_void_p, _I]
        lib.rbe_num_free_blocks.argtypes = [ctypes.c_void_p]
        lib.rbe_check_invariants.argtypes = [ctypes.c_void_p]
        lib.rbe_flush_cache.argtypes = [ctypes.c_void_p]
        lib.rbe_stats.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib._rbk_typed = True
    return lib


def compute_block_hash(token_ids: list[int], prefix_hash: int = -1) -> int:
    """Chained 64-bit hash of one full block (same construction as the C++ core)."""
    mask = (1 << 64) - 1

    def mix(z: int) -> int:
        z = (z + 0x9E3779B97F4A7C15) & mask
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)

    prefix = 0 if prefix_hash == -1 else prefix_hash
    h = mix(prefix ^ 0xA0761D6478BD642F)
    for t in token_ids:
        (u,) = struct.unpack("<I", struct.pack("<i", t))
        h = mix(h ^ ((u * 0xE7037ED1A0B428DB) & mask))
    return h


class PagedKVCache:
    """Block table + prefix cache. Owns no GPU memory: it hands out block ids."""

    _mode = MODE_HASH

    def __init__(self, num_blocks: int, block_size: int = 16) -> None:
        assert num_blocks > 0 and block_size > 0
        self.num_blocks = num_blocks
        self.block_size = block_size
        self._lib = _core()
        self._h = self._lib.rbk_create(num_blocks, block_size, self._mode)
        assert self._h, "engine core allocation failed"

    def __del__(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rbe_destroy(h)

    def num_free_blocks(self) -> int:
        return self._lib.rbe_num_free_blocks(self._h)

    def can_allocate(self, num_tokens: int) -> bool:
        return -(-num_tokens // self.block_size) <= self.num_free_blocks()

    def allocate(self, seq_id: int, token_ids: list[int]) -> tuple[int, ...]:
        n = len(token_ids)
        assert n > 0
        toks = (_I * n)(*token_ids)
        cap = -(-n // self.block_size) + 1
        out = (_I * cap)()
        cached = _I(0)
        rc = self._lib.rbk_allocate(self._h, seq_id, toks, n, out, cap, ctypes.byref(cached))
        if rc == -1:
            raise AssertionError(f"Sequence {seq_id} already allocated")
        if rc < 0:
            raise RuntimeError("No free blocks")
        return tuple(out[:rc])

    def deallocate(self, seq_id: int, publish: bool = True) -> None:
        self._lib.rbk_deallocate(self._h, seq_id, int(publish))

    def append_token(self, seq_id: int, token_id: int) -> int | None:
        rc = self._lib.rbk_append_token(self._h, seq_id, token_id)
        if rc == -2:
            raise RuntimeError("No free blocks for token append")
        assert rc != -3, f"unknown sequence {seq_id}"
        return None if rc == -1 else rc

    def get_block_ids(self, seq_id: int) -> tuple[int, ...]:
        n = self._lib.rbk_get_blocks(self._h, seq_id, None, 0)
        if n <= 0:
            return ()
        out = (_I * n)()
        self._lib.rbk_get_blocks(self._h, seq_id, out, n)
        return tuple(out)

    def get_cached_tokens(self, seq_id: int) -> int:
        return max(0, self._lib.rbk_cached_tokens(self._h, seq_id))

    def ref_count(self, block_id: int) -> int:
        return self._lib.rbk_ref_count(self._h, block_id)

    def flush(self) -> None:
        self._lib.rbe_flush_cache(self._h)

    def check_invariants(self) -> int:
        """0 when refcounts are non-negative and free + used == total."""
        return self._lib.rbe_check_invariants(self._h)

    def stats(self) -> dict:
        s = (_LL * 5)()
        self._lib.rbe_stats(self._h, s)
        return {"hit_tokens": s[0], "miss_tokens": s[1], "evictions": s[2], "free_blocks": s[3], "evictable_blocks": s[4]}
