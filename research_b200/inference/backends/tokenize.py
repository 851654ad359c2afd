"""Chat tokenisation helpers for multi-turn token-level rollouts
(rollouts/inference/backends/tokenize.py:59-378): the "prefix trick" for tokenising one message
in context, cached suffix ids, overlap-safe suffix appending, loss masks, mismatch diagnostics."""

from __future__ import annotations

import logging
from typing import Any

logger = logging.getLogger(__name__)

_DUMMY = [{"role": "user", "content": "x"}]


def tokenize_chat(tokenizer: Any, messages: list[dict[str, str]], add_generation_prompt: bool = False) -> list[int]:
    return list(tokenizer.apply_chat_template(messages, tokenize=True, add_generation_prompt=add_generation_prompt))


def tokenize_message_with_delimiter(tokenizer: Any, message: dict[str, str], add_generation_prompt: bool = False) -> list[int]:
    """Tokens one message contributes when it FOLLOWS other messages: tokenise [dummy, message]
    and strip the dummy's tokens, so role delimiters come out as in context rather than as at
    the start of a conversation."""
    base = tokenize_chat(tokenizer, _DUMMY)
    full = tokenize_chat(tokenizer, _DUMMY + [message], add_generation_prompt)
    assert full[:len(base)] == base, "chat template is not prefix-stable for this tokenizer"
    return full[len(base):]


def build_loss_mask(segments: list[tuple[list[int], bool]]) -> tuple[list[int], list[float]]:
    """Concatenate ``(token_ids, trainable)`` segments into tokens + mask."""
    tokens: list[int] = []
    mask: list[float] = []
    for ids, train in segments:
        tokens += ids
        mask += [1.0 if train else 0.0] * len(ids)
    return tokens, mask


def compute_suffix_ids(tokenizer: Any) -> list[int]:
    """Tokens the template appends after an assistant message's content (end-of-turn markers)."""
    a = tokenize_chat(tokenizer, _DUMMY + [{"role": "assistant", "content": "y"}])
    content = list(tokenizer.encode("y", add_special_tokens=False))
    for i in range(len(a) - len(content), -1, -1):
        if a[i:i + len(content)] == content:
            return a[i + len(content):]
    return []


def find_largest_overlap(a: list[int], b: list[int]) -> int:
    """Largest n with ``a[-n:] == b[:n]``."""
    for n in range(min(len(a), len(b)), 0, -1):
        if a[-n:] == b[:n]:
            return n
    return 0


def append_suffix_with_overlap(tokens: list[int], suffix: list[int]) -> list[int]:
    """Append ``suffix`` without duplicating the part the generation already ended with
    (a model that emitted its own end-of-turn token must not get a second one)."""
    return tokens + suffix[find_largest_overlap(tokens, suffix):]


def check_token_mismatch(engine_ids: list[int], retokenized_ids: list[int]) -> dict[str, Any] | None:
    """First divergence between what the engine produced and what re-tokenising its text gives."""
    n = min(len(engine_ids), len(retokenized_ids))
    for i in range(n):
        if engine_ids[i] != retokenized_ids[i]:
            return {"position": i, "engine": engine_ids[i], "retokenized": retokenized_ids[i],
                    "engine_len": len(engine_ids), "retokenized_len": len(retokenized_ids)}
    if len(engine_ids) != len(retokenized_ids):
        return {"position": n, "engine": None, "retokenized": None, "engine_len": len(engine_ids),
                "retokenized_len": len(retokenized_ids)}
    return None


def log_token_mismatch(mismatch: dict[str, Any] | None, tokenizer: Any = None, context: str = "") -> None:
    if mismatch is None:
        return
    detail = ""
    if tokenizer is not None and mismatch.get("engine") is not None:
        detail = f" engine={tokenizer.decode([mismatch['engine']])!r} retokenized={tokenizer.decode([mismatch['retokenized']])!r}"
    logger.warning("token mismatch %s at %d (lengths %d vs %d)%s", context, mismatch["position"], mismatch["engine_len"],
                   mismatch["retokenized_len"], detail)
