"""SFT data preparation: conversations -> token ids + loss mask -> ``Sample``
(rollouts/training/datasets/sft.py:14-248, dataset_loaders.py:39-365).

The mask trains on assistant turns only. Message boundaries are found by tokenising growing
prefixes of the conversation with the chat template (prefix-stable templates give exact spans
without any string matching). Loaders accept lists, JSONL and (when the libraries and files exist
locally) parquet / Hugging Face datasets; conversations may use ``messages`` or the
``conversations`` / ``from`` / ``value`` (ShareGPT) convention or ``prompt`` + ``response``.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Iterable

from ..types import Sample, Status

_ROLE_ALIASES = {"human": "user", "gpt": "assistant", "bot": "assistant", "model": "assistant"}


def extract_conversation(example: dict[str, Any]) -> list[dict[str, str]] | None:
    if isinstance(example.get("messages"), list):
        return [{"role": m["role"], "content": m.get("content", "")} for m in example["messages"]]
    if isinstance(example.get("conversations"), list):
        return [{"role": _ROLE_ALIASES.get(m.get("from", m.get("role", "user")), m.get("from", m.get("role", "user"))),
                 "content": m.get("value", m.get("content", ""))} for m in example["conversations"]]
    prompt = next((example[k] for k in ("prompt", "question", "instruction", "input") if example.get(k)), None)
    response = next((example[k] for k in ("response", "answer", "output", "completion") if example.get(k)), None)
    if prompt is not None and response is not None:
        return [{"role": "user", "content": str(prompt)}, {"role": "assistant", "content": str(response)}]
    return None


def extract_prompt(example: dict[str, Any]) -> str | None:
    for k in ("prompt", "question", "problem", "instruction", "input", "query"):
        if example.get(k):
            return str(example[k])
    conv = extract_conversation(example)
    return next((m["content"] for m in conv if m["role"] == "user"), None) if conv else None


def extract_answer(example: dict[str, Any]) -> str | None:
    for k in ("answer", "ground_truth", "solution", "target", "label", "response"):
        if example.get(k) is not None:
            return str(example[k])
    return None


def tokenize_conversation(tokenizer: Any, messages: list[dict[str, str]], max_length: int | None = None) -> tuple[list[int], list[tuple[int, int, str]]]:
    """Token ids of the whole conversation and ``(start, end, role)`` spans of every message."""
    ids: list[int] = []
    spans = []
    for i in range(len(messages)):
        cur = list(tokenizer.apply_chat_template(messages[: i + 1], tokenize=True, add_generation_prompt=False))
        if cur[: len(ids)] != ids:         # template rewrote earlier tokens: fall back to whole-conversation ids
            ids = cur
            spans = [(0, len(cur), messages[i]["role"])] if i == 0 else spans[:-1] + [(spans[-1][0], len(cur), messages[i]["role"])]
            continue
        spans.append((len(ids), len(cur), messages[i]["role"]))
        ids = cur
    if max_length is not None and len(ids) > max_length:
        ids = ids[:max_length]
        spans = [(s, min(e, max_length), r) for s, e, r in spans if s < max_length]
    return ids, spans


def compute_loss_mask(n_tokens: int, spans: list[tuple[int, int, str]], train_roles: tuple[str, ...] = ("assistant",)) -> list[float]:
    mask = [0.0] * n_tokens
    for s, e, role in spans:
        if role in train_roles:
            for i in range(s, min(e, n_tokens)):
                mask[i] = 1.0
    return mask


def prepare_sft_sample(tokenizer: Any, messages: list[dict[str, str]], max_length: int | None = None, index: int = 0) -> Sample:
    ids, spans = tokenize_conversation(tokenizer, messages, max_length)
    mask = compute_loss_mask(len(ids), spans)
    n_resp = int(sum(mask))
    return Sample(id=f"sft_{index}", index=index, prompt=messages, tokens=ids, loss_mask=mask, response_length=n_resp,
                  status=Status.COMPLETED, metadata={"num_messages": len(messages)})


def _rows(source: str | Path | Iterable[dict[str, Any]], split: str = "train") -> Iterable[dict[str, Any]]:
    if not isinstance(source, (str, Path)):
        return source
    p = Path(source)
    if p.suffix in (".jsonl", ".json") and p.exists():
        text = p.read_text()
        return json.loads(text) if p.suffix == ".json" else [json.loads(line) for line in text.splitlines() if line.strip()]
    if p.suffix == ".parquet" and p.exists():
        import pandas as pd

        return pd.read_parquet(p).to_dict("records")
    from datasets import load_dataset  # needs the dataset in the local cache (no network here)

    return load_dataset(str(source), split=split)


def load_sft_dataset(source, tokenizer: Any, max_length: int | None = 2048, max_samples: int | None = None, split: str = "train",
                     skip_too_long: bool = False) -> list[Sample]:
    out = []
    for i, row in enumerate(_rows(source, split)):
        if max_samples is not None and len(out) >= max_samples:
            break
        conv = extract_conversation(row)
        if not conv or not any(m["role"] == "assistant" for m in conv):
            continue
        s = prepare_sft_sample(tokenizer, conv, None if skip_too_long else max_length, i)
        if skip_too_long and max_length is not None and len(s.tokens) > max_length:
            continue
        if s.response_length > 0:
            out.append(s)
    return out


def load_rl_prompts(source, max_samples: int | None = None, split: str = "train") -> list[Sample]:
    out = []
    for i, row in enumerate(_rows(source, split)):
        if max_samples is not None and len(out) >= max_samples:
            break
        prompt = extract_prompt(row)
        if prompt:
            out.append(Sample(id=f"prompt_{i}", index=i, prompt=prompt, ground_truth=extract_answer(row), input=dict(row)))
    return out


def export_samples_to_jsonl(samples: list[Sample], path: str | Path) -> None:
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as f:
        for s in samples:
            f.write(json.dumps({"id": s.id, "index": s.index, "prompt": s.prompt, "tokens": s.tokens, "loss_mask": s.loss_mask,
                                "response_length": s.response_length, "reward": s.reward, "ground_truth": s.ground_truth,
                                "metadata": s.metadata}) + "\n")


def load_samples_from_export(path: str | Path) -> list[Sample]:
    out = []
    for line in Path(path).read_text().splitlines():
        if line.strip():
            d = json.loads(line)
            out.append(Sample(id=d.get("id", ""), index=d.get("index"), prompt=d.get("prompt", ""), tokens=d.get("tokens", []),
                              loss_mask=d.get("loss_mask", []), response_length=d.get("response_length", 0), reward=d.get("reward", 0.0),
                              ground_truth=d.get("ground_truth"), metadata=d.get("metadata", {}), status=Status.COMPLETED))
    return out
