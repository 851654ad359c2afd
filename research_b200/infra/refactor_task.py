"""Comment-driven multi-file refactoring with a language model (rollouts/tools/refactor-artillery/refactor.py, blocks.py,
imports.py, commands.py): the task is written as trailing comments of a file, the tool gathers that file and the files
it imports (recursively), asks a model for edits in a small tagged format, and applies them.

Reply format the model is asked for (any number of blocks, in any order)::

    <write file="pkg/new.py">...whole new content...</write>
    <patch file="pkg/a.py"><search>exact old text</search><replace>new text</replace></patch>
    <delete file="pkg/old.py"/>

Paths are relative to the root directory and may not leave it. ``dry_run`` returns the planned edits untouched.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from pathlib import Path
from typing import Awaitable, Callable

COMMENT_PREFIX = {".py": "#", ".js": "//", ".ts": "//", ".tsx": "//", ".jsx": "//", ".lua": "--", ".go": "//", ".rs": "//",
                  ".c": "//", ".h": "//", ".cpp": "//", ".cu": "//", ".sh": "#"}


def extract_task(source: str, suffix: str = ".py") -> tuple[str, str]:
    """Split ``source`` into (code without the trailing comment block, task text). The task is the run of comment
    lines at the very end of the file (blank lines between them allowed)."""
    mark = COMMENT_PREFIX.get(suffix, "#")
    lines = source.rstrip("\n").split("\n")
    i = len(lines)
    task: list[str] = []
    while i > 0:
        s = lines[i - 1].strip()
        if s.startswith(mark):
            task.append(s[len(mark):].strip())
            i -= 1
        elif not s and task:
            i -= 1
        else:
            break
    code = "\n".join(lines[:i]).rstrip("\n") + "\n"
    return code, "\n".join(reversed([t for t in task if t]))


_PY_FROM = re.compile(r"^\s*from\s+(\.*)([\w.]*)\s+import\s+", re.M)
_PY_IMPORT = re.compile(r"^\s*import\s+([\w.]+)", re.M)
_JS_IMPORT = re.compile(r"""(?:import\s[^'"]*?from\s*|import\s*|require\()\s*['"](\.{1,2}/[^'"]+)['"]""")
_LUA_REQUIRE = re.compile(r"""require\s*\(?\s*['"]([\w./]+)['"]""")
_C_INCLUDE = re.compile(r'^\s*#\s*include\s*"([^"]+)"', re.M)
# a file named on a comment line of its own, "#[./rel/path]" ("//[...]", "--[...]"): context the imports do not reach
_MARKER = re.compile(r"^\s*(?:#|//|--)\[(\.{1,2}/[^\]]+)\]\s*$", re.M)


def imported_files(path: Path, root: Path) -> list[Path]:
    """Files of the project that ``path`` imports (only those that exist under ``root``)."""
    text = path.read_text(errors="replace")
    out: list[Path] = []

    def add(p: Path) -> None:
        for cand in (p, p.with_suffix(path.suffix), p / "__init__.py", p / f"index{path.suffix}"):
            if cand.is_file() and root in cand.resolve().parents and cand.resolve() not in out:
                out.append(cand.resolve())
                return

    if path.suffix == ".py":
        for dots, mod in _PY_FROM.findall(text):
            base = path.parent
            for _ in range(max(len(dots) - 1, 0)):
                base = base.parent
            start = base if dots else root
            add(start.joinpath(*mod.split(".")) if mod else start)
        for mod in _PY_IMPORT.findall(text):
            add(root.joinpath(*mod.split(".")))
    elif path.suffix in (".js", ".ts", ".tsx", ".jsx"):
        for rel in _JS_IMPORT.findall(text):
            add((path.parent / rel))
    elif path.suffix == ".lua":
        for mod in _LUA_REQUIRE.findall(text):
            add(root.joinpath(*mod.replace("/", ".").split(".")))
    elif path.suffix in (".c", ".h", ".cpp", ".hpp", ".cc", ".cu", ".cuh"):
        for inc in _C_INCLUDE.findall(text):
            for base in (path.parent, root):
                if (base / inc).is_file():
                    add(base / inc)
                    break
    for rel in _MARKER.findall(text):
        if (path.parent / rel).is_file():
            add(path.parent / rel)
    return out


def collect_context(entry: Path, root: Path | None = None, max_files: int = 20, max_bytes: int = 400_000) -> dict[str, str]:
    """``{relative path: content}`` of ``entry`` and everything it imports, breadth first, bounded."""
    entry = entry.resolve()
    root = (root or entry.parent).resolve()
    order, seen, size = [entry], {entry}, 0
    out: dict[str, str] = {}
    while order and len(out) < max_files:
        p = order.pop(0)
        text = p.read_text(errors="replace")
        if size + len(text) > max_bytes and out:
            break
        size += len(text)
        out[str(p.relative_to(root))] = text
        for q in imported_files(p, root):
            if q not in seen:
                seen.add(q)
                order.append(q)
    return out


@dataclass(frozen=True)
class Edit:
    kind: str                      # write | patch | delete
    file: str
    content: str = ""              # write: new content; patch: replacement
    search: str = ""               # patch only


_BLOCK = re.compile(r'<write file="([^"]+)">\n?(.*?)</write>|<patch file="([^"]+)">\s*<search>\n?(.*?)</search>\s*<replace>\n?(.*?)</replace>\s*</patch>'
                    r'|<delete file="([^"]+)"\s*/>', re.S)


def parse_edits(reply: str) -> list[Edit]:
    edits = []
    for w_file, w_body, p_file, p_search, p_repl, d_file in _BLOCK.findall(reply):
        if w_file:
            edits.append(Edit("write", w_file, w_body))
        elif p_file:
            edits.append(Edit("patch", p_file, p_repl, p_search))
        elif d_file:
            edits.append(Edit("delete", d_file))
    return edits


def apply_edits(edits: list[Edit], root: Path, dry_run: bool = False, initial: dict[Path, str] | None = None) -> list[str]:
    """Apply in order; returns one line per edit. Nothing is written unless every edit is valid (paths inside
    ``root``, patch targets exist and contain their search text exactly once). ``initial`` gives contents to start
    from instead of what is on disk (they are written too)."""
    root = root.resolve()
    staged: dict[Path, str | None] = {p.resolve(): c for p, c in (initial or {}).items()}
    log = []
    for e in edits:
        target = (root / e.file).resolve()
        if root != target and root not in target.parents:
            raise ValueError(f"edit leaves the project root: {e.file}")
        current = staged[target] if target in staged else (target.read_text() if target.is_file() else None)
        if e.kind == "write":
            staged[target] = e.content
            log.append(f"write {e.file} ({len(e.content)} bytes)")
        elif e.kind == "delete":
            if current is None:
                raise ValueError(f"cannot delete missing file {e.file}")
            staged[target] = None
            log.append(f"delete {e.file}")
        else:
            if current is None:
                raise ValueError(f"cannot patch missing file {e.file}")
            n = current.count(e.search)
            if n != 1:
                raise ValueError(f"patch for {e.file}: search text found {n} times, expected once")
            staged[target] = current.replace(e.search, e.content)
            log.append(f"patch {e.file}")
    if not dry_run:
        for target, content in staged.items():
            if content is None:
                target.unlink()
            else:
                target.parent.mkdir(parents=True, exist_ok=True)
                target.write_text(content)
    return log


PROMPT = """You are a refactoring tool. Apply the TASK to the FILES and answer ONLY with edit blocks:
<write file="path">whole new content</write>
<patch file="path"><search>exact old text</search><replace>new text</replace></patch>
<delete file="path"/>
Keep behaviour unchanged apart from the task. Paths are relative to the project root.

TASK:
{task}

FILES:
{files}"""


COMPACTION_THRESHOLD_TOKENS = 32_000

COMPACT_PROMPT = """You are preparing context for a refactoring. Below are the TASK and the FILES gathered for it. Name the files
that are NOT needed to carry out the task, one per line, as <omit file="path"/>. Omit nothing you are unsure about; answer
with no <omit> line if everything is needed.

TASK:
{task}

FILES:
{files}"""


def estimate_tokens(text: str) -> int:
    return len(text) // 4


def _render(ctx: dict[str, str]) -> str:
    return "\n".join(f'<file path="{p}">\n{c}</file>' for p, c in ctx.items())


async def compact_context(ctx: dict[str, str], task: str, complete: Callable[[str], Awaitable[str]], keep: set[str] = frozenset(),
                          threshold_tokens: int = COMPACTION_THRESHOLD_TOKENS) -> dict[str, str]:
    """When the gathered files exceed ``threshold_tokens``, ask the model which of them the task does not need and
    drop those (never a file in ``keep``, never a path that was not offered)."""
    if estimate_tokens(_render(ctx)) <= threshold_tokens:
        return ctx
    reply = await complete(COMPACT_PROMPT.format(task=task, files=_render(ctx)))
    omit = set(re.findall(r'<omit file="([^"]+)"\s*/>', reply)) & set(ctx) - set(keep)
    return {p: c for p, c in ctx.items() if p not in omit}


def save_run_log(log_dir: Path, entry: str, task: str, prompt: str, reply: str, applied: list[str], now: float | None = None) -> Path:
    """One text file per run (prompt, reply, what was applied) under ``log_dir``, named by time and entry file."""
    import time

    log_dir.mkdir(parents=True, exist_ok=True)
    stamp = time.strftime("%Y%m%d-%H%M%S", time.localtime(now if now is not None else time.time()))
    f = log_dir / f"{stamp}_{Path(entry).stem}.log"
    f.write_text(f"# task\n{task}\n\n# prompt\n{prompt}\n\n# reply\n{reply}\n\n# applied\n" + "\n".join(applied) + "\n")
    return f


async def refactor(entry: str | Path, complete: Callable[[str], Awaitable[str]], root: str | Path | None = None,
                   dry_run: bool = False, compaction_threshold_tokens: int = COMPACTION_THRESHOLD_TOKENS,
                   log_dir: str | Path | None = None) -> list[str]:
    """Run the whole loop for ``entry``: task from its trailing comments, context from its imports, ``complete(prompt)``
    (any async text-in / text-out model call) for the edits, then apply. The task comment is removed from ``entry``
    before the model sees it; the edits apply to that cleaned text."""
    entry = Path(entry).resolve()
    root_p = Path(root).resolve() if root else entry.parent
    code, task = extract_task(entry.read_text(), entry.suffix)
    if not task:
        raise ValueError(f"{entry} has no trailing comment describing a task")
    ctx = collect_context(entry, root_p)
    rel = str(entry.relative_to(root_p))
    ctx[rel] = code
    ctx = await compact_context(ctx, task, complete, keep={rel}, threshold_tokens=compaction_threshold_tokens)
    prompt = PROMPT.format(task=task, files=_render(ctx))
    reply = await complete(prompt)
    edits = parse_edits(reply)
    if not edits:
        raise ValueError("the model returned no edit blocks")
    applied = apply_edits(edits, root_p, dry_run, initial={entry: code})
    if log_dir is not None:
        save_run_log(Path(log_dir), rel, task, prompt, reply, applied)
    return applied
