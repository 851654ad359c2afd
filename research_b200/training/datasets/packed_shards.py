"""Pre-tokenised shard files and BOS-aligned packing for pre-training runs (dev/speedrun/single-file.py:1154-1365:
``_load_data_shard``, ``BOSFinder``, ``distributed_data_generator``).

Shard format (the public one of the GPT-2 speedruns): 256 int32 header words (magic 20240520, version 1, token count),
then the tokens as uint16. A batch is a run of whole documents: every sequence starts at a BOS token, documents longer
than ``max_seq_len`` are cut, and the boundaries come back as ``cu_seqlens`` for varlen attention. Each rank takes its
own slice of the documents of a batch, so ranks never share a token.
"""

from __future__ import annotations

from pathlib import Path
from typing import Iterator, Sequence

import numpy as np
import torch

MAGIC, VERSION, HEADER_WORDS = 20240520, 1, 256


def write_shard(path: str | Path, tokens: Sequence[int] | np.ndarray) -> None:
    arr = np.asarray(tokens, dtype=np.uint16)
    header = np.zeros(HEADER_WORDS, dtype=np.int32)
    header[0], header[1], header[2] = MAGIC, VERSION, arr.size
    with open(path, "wb") as f:
        f.write(header.tobytes())
        f.write(arr.tobytes())


def load_shard(path: str | Path) -> torch.Tensor:
    """uint16 tokens of one shard as an int32 tensor (memory-mapped read, header checked)."""
    header = np.fromfile(path, dtype=np.int32, count=HEADER_WORDS)
    if header.size < 3 or header[0] != MAGIC or header[1] != VERSION:
        raise ValueError(f"{path}: not a token shard (magic {header[:2].tolist()})")
    n = int(header[2])
    tokens = np.memmap(path, dtype=np.uint16, mode="r", offset=HEADER_WORDS * 4, shape=(n,))
    return torch.from_numpy(tokens.astype(np.int32))


def document_starts(tokens: torch.Tensor, bos_id: int) -> torch.Tensor:
    return torch.nonzero(tokens == bos_id).flatten()


def pack_documents(tokens: torch.Tensor, starts: torch.Tensor, first_doc: int, num_tokens: int, max_seq_len: int):
    """Whole documents from ``first_doc`` on until ``num_tokens`` inputs are filled (the last one cut to fit).
    Returns (inputs, targets, cu_seqlens, next_doc) or None when the shard has too few tokens left."""
    spans, total, d = [], 0, first_doc
    while total < num_tokens and d < len(starts):
        a = int(starts[d])
        b = int(starts[d + 1]) if d + 1 < len(starts) else tokens.numel()
        length = min(b - a, max_seq_len, num_tokens - total)
        if a + length + 1 > tokens.numel():                       # targets need one token beyond the inputs
            length = tokens.numel() - 1 - a
        if length <= 0:
            break
        spans.append((a, length))
        total += length
        d += 1
    if total < num_tokens:
        return None
    inputs = torch.cat([tokens[a:a + n] for a, n in spans])
    targets = torch.cat([tokens[a + 1:a + n + 1] for a, n in spans])
    cu = torch.tensor([0] + list(np.cumsum([n for _, n in spans])), dtype=torch.int32)
    return inputs, targets, cu, d


def packed_batches(files: Sequence[str | Path], num_tokens: int, max_seq_len: int, bos_id: int, rank: int = 0, world: int = 1,
                   loop: bool = False) -> Iterator[tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
    """Yields (inputs [num_tokens], targets [num_tokens], cu_seqlens) for this rank. One global step consumes
    ``world`` consecutive packs from the shard; rank r keeps the r-th, so the ranks stay in step through a shard."""
    assert files, "no shard files"
    while True:
        for path in files:
            tokens = load_shard(path)
            starts = document_starts(tokens, bos_id)
            doc = 0
            while True:
                packs = []
                for _ in range(world):
                    got = pack_documents(tokens, starts, doc, num_tokens, max_seq_len)
                    if got is None:
                        packs = None
                        break
                    packs.append(got[:3])
                    doc = got[3]
                if packs is None:
                    break
                yield packs[rank]
        if not loop:
            return
