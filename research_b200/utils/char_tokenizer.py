"""A dependency-free character tokenizer with the subset of the Hugging Face tokenizer interface this framework calls
(``encode``, ``decode``, ``apply_chat_template``, ``eos_token_id``, ``__call__``). It lets the examples and smoke runs
work end to end (chat templates, loss masks, token-in / token-out rollouts, stop on EOS) where no pretrained tokenizer
is on disk. Ids: 0 pad, 1 bos, 2 eos, 3.. role markers, then the printable ASCII characters and newline / tab; any
other character maps to ``<unk>``. The chat template is prefix-stable (``<|role|>text<|eos|>`` per message), which the
loss-mask and suffix logic of ``inference/backends/tokenize.py`` relies on."""

from __future__ import annotations

from typing import Any, Iterable, Sequence

SPECIALS = ["<|pad|>", "<|bos|>", "<|eos|>", "<|unk|>", "<|system|>", "<|user|>", "<|assistant|>", "<|tool|>"]
ROLES = {"system": "<|system|>", "user": "<|user|>", "assistant": "<|assistant|>", "tool": "<|tool|>"}


class CharTokenizer:
    def __init__(self) -> None:
        chars = [chr(c) for c in range(32, 127)] + ["\n", "\t"]
        self.itos: list[str] = SPECIALS + chars
        self.stoi = {s: i for i, s in enumerate(self.itos)}
        self.pad_token_id, self.bos_token_id, self.eos_token_id, self.unk_token_id = 0, 1, 2, 3
        self.pad_token, self.bos_token, self.eos_token = SPECIALS[0], SPECIALS[1], SPECIALS[2]
        self.name_or_path = "char-tokenizer"

    @property
    def vocab_size(self) -> int:
        return len(self.itos)

    def __len__(self) -> int:
        return len(self.itos)

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        out = [self.bos_token_id] if add_special_tokens else []
        i, n = 0, len(text)
        while i < n:
            if text[i] == "<" and text.startswith("<|", i):
                j = text.find("|>", i)
                if j != -1 and text[i:j + 2] in self.stoi:
                    out.append(self.stoi[text[i:j + 2]])
                    i = j + 2
                    continue
            out.append(self.stoi.get(text[i], self.unk_token_id))
            i += 1
        return out

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = False) -> str:
        n_special = len(SPECIALS)
        return "".join(self.itos[i] for i in ids if 0 <= i < len(self.itos) and not (skip_special_tokens and i < n_special))

    def apply_chat_template(self, messages: Sequence[dict[str, Any]], tokenize: bool = True, add_generation_prompt: bool = False,
                            **_: Any) -> list[int] | str:
        text = "".join(f"{ROLES.get(m['role'], ROLES['user'])}{m.get('content') or ''}{self.eos_token}" for m in messages)
        if add_generation_prompt:
            text += ROLES["assistant"]
        return self.encode(text) if tokenize else text

    def __call__(self, text: str | list[str], add_special_tokens: bool = False, **_: Any) -> dict[str, Any]:
        if isinstance(text, str):
            return {"input_ids": self.encode(text, add_special_tokens)}
        return {"input_ids": [self.encode(t, add_special_tokens) for t in text]}

    def convert_ids_to_tokens(self, ids: Iterable[int]) -> list[str]:
        return [self.itos[i] if 0 <= i < len(self.itos) else SPECIALS[3] for i in ids]
