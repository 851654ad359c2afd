"""Trigram-indexed code search (csearch/csearch/index.py:67-189).

The index maps every 3-character substring to the files that contain it; a literal query is answered
by intersecting the posting lists of its trigrams and confirming candidates by reading them, a regex
query uses the literal fragments it can prove are required. Symbol lookup (``def`` / ``class`` /
``struct`` / ``__global__`` definitions) is a cheap regex pass over the same file set.
"""

from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from pathlib import Path

TEXT_EXT = {".py", ".cu", ".cuh", ".h", ".hpp", ".cpp", ".cc", ".c", ".md", ".toml", ".json", ".yaml", ".yml", ".sh", ".txt", ".rs", ".js", ".ts"}
SKIP_DIRS = {".git", "__pycache__", "node_modules", ".venv", "build", "dist"}
_DEF = re.compile(r"^\s*(?:async\s+def|def|class|struct|enum|fn|function|__global__\s+\w+|template\s*<[^>]*>\s*__global__\s+\w+)\s+(\w+)", re.MULTILINE)


@dataclass(frozen=True)
class Hit:
    path: str
    line: int
    text: str


def trigrams(s: str) -> set[str]:
    s = s.lower()
    return {s[i:i + 3] for i in range(len(s) - 2)}


class CodeIndex:
    def __init__(self, root: str | Path):
        self.root = Path(root)
        self.files: list[str] = []
        self.postings: dict[str, set[int]] = {}
        self.mtimes: dict[str, float] = {}

    def build(self, max_bytes: int = 2_000_000) -> "CodeIndex":
        self.files, self.postings, self.mtimes = [], {}, {}
        for dirpath, dirnames, filenames in os.walk(self.root):
            dirnames[:] = [d for d in dirnames if d not in SKIP_DIRS and not d.startswith(".")]
            for fn in filenames:
                p = Path(dirpath) / fn
                if p.suffix not in TEXT_EXT or p.stat().st_size > max_bytes:
                    continue
                try:
                    text = p.read_text(errors="ignore")
                except OSError:
                    continue
                idx = len(self.files)
                rel = str(p.relative_to(self.root))
                self.files.append(rel)
                self.mtimes[rel] = p.stat().st_mtime
                for t in trigrams(text):
                    self.postings.setdefault(t, set()).add(idx)
        return self

    def _candidates(self, literal: str) -> set[int]:
        tg = trigrams(literal)
        if not tg:
            return set(range(len(self.files)))
        sets = [self.postings.get(t, set()) for t in tg]
        return set.intersection(*sets) if sets else set()

    @staticmethod
    def _required_literals(pattern: str) -> list[str]:
        """Literal runs of length >= 3 outside any alternation, class, group or quantified atom."""
        if "|" in pattern:
            return []
        out, cur, i = [], "", 0
        while i < len(pattern):
            c = pattern[i]
            if c == "\\" and i + 1 < len(pattern) and not pattern[i + 1].isalnum():
                cur += pattern[i + 1]
                i += 2
                continue
            if c in "[(":                                   # skip the whole class / group
                close = {"[": "]", "(": ")"}[c]
                out.append(cur)
                cur = ""
                depth = 1
                i += 1
                while i < len(pattern) and depth:
                    depth += pattern[i] == c
                    depth -= pattern[i] == close
                    i += 1
                continue
            if c in ".*+?{}^$\\":
                if c in "*?{" and cur:
                    cur = cur[:-1]                          # the quantified character is optional
                out.append(cur)
                cur = ""
            else:
                cur += c
            i += 1
        out.append(cur)
        return [s for s in out if len(s) >= 3]

    def search(self, query: str, regex: bool = False, ignore_case: bool = True, max_hits: int = 200) -> list[Hit]:
        flags = re.IGNORECASE if ignore_case else 0
        rx = re.compile(query if regex else re.escape(query), flags)
        lits = self._required_literals(query) if regex else [query]
        cand = set(range(len(self.files)))
        for lit in lits:
            cand &= self._candidates(lit)
        hits = []
        for idx in sorted(cand):
            try:
                lines = (self.root / self.files[idx]).read_text(errors="ignore").splitlines()
            except OSError:
                continue
            for n, line in enumerate(lines, 1):
                if rx.search(line):
                    hits.append(Hit(self.files[idx], n, line.strip()[:240]))
                    if len(hits) >= max_hits:
                        return hits
        return hits

    def symbols(self, name: str | None = None) -> list[Hit]:
        out = []
        for rel in self.files:
            text = (self.root / rel).read_text(errors="ignore")
            for m in _DEF.finditer(text):
                if name is None or m.group(1) == name:
                    out.append(Hit(rel, text.count("\n", 0, m.start(1)) + 1, m.group(0).strip()))   # the match may begin on blank lines above
        return out

    def stale_files(self) -> list[str]:
        return [f for f in self.files if not (self.root / f).exists() or (self.root / f).stat().st_mtime != self.mtimes[f]]

    def save(self, path: str | Path) -> None:
        Path(path).write_text(json.dumps({"root": str(self.root), "files": self.files, "mtimes": self.mtimes,
                                          "postings": {k: sorted(v) for k, v in self.postings.items()}}))

    @staticmethod
    def load(path: str | Path) -> "CodeIndex":
        d = json.loads(Path(path).read_text())
        ix = CodeIndex(d["root"])
        ix.files, ix.mtimes = d["files"], d["mtimes"]
        ix.postings = {k: set(v) for k, v in d["postings"].items()}
        return ix
