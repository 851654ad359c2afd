"""Symbol search: where is a name DEFINED, where is it USED (csearch/csearch: ``types.py``, ``search.py``,
``backends/tree_sitter.py:146-343``, ``backends/ctags.py:19-266``).

Backends, tried in this order by ``backend="auto"``:

* ``tree-sitter``  the reference's first choice; used when the ``tree_sitter`` package and a grammar for the file's
                   language can be imported, otherwise reported unavailable (nothing is downloaded);
* ``ast``          Python files through the standard ``ast`` module: exact start / end lines, functions, methods,
                   classes, module and class level assignments; references are name / attribute / call nodes;
* ``scan``         every other language (C, C++, CUDA, Rust, Go, JS / TS): a definition scanner with brace matching
                   for the end line (functions, ``__global__`` kernels, struct / class / enum / namespace, macros);
* ``ctags``        a ``tags`` file built by an installed ``ctags`` binary (``ctags -R --fields=+ne``), parsed here;
                   without the binary the backend is unavailable.

All functions are pure: query + ``SearchOptions`` in, list of ``SearchResult`` out.
"""

from __future__ import annotations

import ast
import os
import re
import shutil
import subprocess
from dataclasses import dataclass
from pathlib import Path

SKIP_DIRS = {".git", "__pycache__", "node_modules", ".venv", "venv", "build", "dist", ".mypy_cache", ".pytest_cache", "target"}
LANG_BY_EXT = {".py": "python", ".c": "c", ".h": "c", ".cc": "cpp", ".cpp": "cpp", ".hpp": "cpp", ".cu": "cuda", ".cuh": "cuda",
               ".rs": "rust", ".go": "go", ".js": "javascript", ".ts": "typescript", ".tsx": "typescript", ".java": "java"}


@dataclass(frozen=True)
class Location:
    path: Path
    line_start: int
    line_end: int

    def __str__(self) -> str:
        return f"{self.path}:{self.line_start}" if self.line_start == self.line_end else f"{self.path}:{self.line_start}-{self.line_end}"


@dataclass(frozen=True)
class SearchResult:
    location: Location
    name: str
    kind: str                      # function | method | class | struct | enum | variable | kernel | macro | namespace | reference | call
    snippet: str | None = None

    def format_compact(self) -> str:
        return f"{self.location} {self.kind} {self.name}"

    def format_with_snippet(self) -> str:
        return str(self.location) + ("\n" + self.snippet if self.snippet else "")


@dataclass(frozen=True)
class SearchOptions:
    path: Path = Path(".")
    backend: str = "auto"          # auto | tree-sitter | ast | scan | ctags
    include_snippet: bool = False
    limit: int | None = None
    exact: bool = True             # False: the query may be a substring of the symbol name


def find_files(root: Path, extensions: set[str] | None = None) -> list[Path]:
    root = Path(root)
    if root.is_file():
        return [root]
    out = []
    for dirpath, dirnames, filenames in os.walk(root):
        dirnames[:] = sorted(d for d in dirnames if d not in SKIP_DIRS and not d.startswith("."))
        for fn in sorted(filenames):
            p = Path(dirpath) / fn
            if p.suffix in (extensions or LANG_BY_EXT):
                out.append(p)
    return out


def extract_snippet(path: Path, start: int, end: int, max_lines: int = 40) -> str:
    try:
        lines = Path(path).read_text(errors="replace").splitlines()
    except OSError:
        return ""
    end = min(end, start + max_lines - 1, len(lines))
    return "\n".join(lines[start - 1:end])


def _match(name: str, query: str, exact: bool) -> bool:
    return name == query if exact else query.lower() in name.lower()


def _finish(results: list[SearchResult], o: SearchOptions) -> list[SearchResult]:
    results = results[:o.limit] if o.limit is not None else results
    if o.include_snippet:
        results = [SearchResult(r.location, r.name, r.kind, extract_snippet(r.location.path, r.location.line_start, r.location.line_end))
                   for r in results]
    return results


# ------------------------------------------------------------------------------------------ python: ast
def _py_definitions(path: Path):
    try:
        tree = ast.parse(path.read_text(errors="replace"))
    except (SyntaxError, OSError, ValueError):
        return

    def walk(node, in_class: bool):
        for ch in ast.iter_child_nodes(node):
            if isinstance(ch, (ast.FunctionDef, ast.AsyncFunctionDef)):
                first = min([d.lineno for d in ch.decorator_list] + [ch.lineno])
                yield ch.name, "method" if in_class else "function", first, ch.end_lineno or ch.lineno
                yield from walk(ch, False)
            elif isinstance(ch, ast.ClassDef):
                first = min([d.lineno for d in ch.decorator_list] + [ch.lineno])
                yield ch.name, "class", first, ch.end_lineno or ch.lineno
                yield from walk(ch, True)
            elif isinstance(ch, (ast.Assign, ast.AnnAssign)) and isinstance(node, (ast.Module, ast.ClassDef)):
                targets = ch.targets if isinstance(ch, ast.Assign) else [ch.target]
                for t in targets:
                    for n in ast.walk(t):
                        if isinstance(n, ast.Name):
                            yield n.id, "variable", ch.lineno, ch.end_lineno or ch.lineno
            elif isinstance(ch, (ast.If, ast.Try, ast.With, ast.For, ast.While)):
                yield from walk(ch, in_class)

    yield from walk(tree, False)


def _py_references(path: Path, query: str):
    try:
        tree = ast.parse(path.read_text(errors="replace"))
    except (SyntaxError, OSError, ValueError):
        return
    calls = set()
    for n in ast.walk(tree):
        if isinstance(n, ast.Call):
            f = n.func
            if (isinstance(f, ast.Name) and f.id == query) or (isinstance(f, ast.Attribute) and f.attr == query):
                calls.add((f.lineno, f.col_offset))
    seen = set()
    for n in ast.walk(tree):
        hit = (isinstance(n, ast.Name) and n.id == query and not isinstance(n.ctx, ast.Store)) or (isinstance(n, ast.Attribute) and n.attr == query)
        if hit and (n.lineno, n.col_offset) not in seen:
            seen.add((n.lineno, n.col_offset))
            yield ("call" if (n.lineno, n.col_offset) in calls else "reference"), n.lineno


# ------------------------------------------------------------------------------------------ other languages: scan
_SCAN = [
    ("kernel", re.compile(r"^\s*(?:template\s*<[^>]*>\s*)?(?:static\s+|extern\s+\"C\"\s+)*__global__\s+[\w:<>\s\*&]+?\b(\w+)\s*\(")),
    ("macro", re.compile(r"^\s*#\s*define\s+(\w+)")),
    ("struct", re.compile(r"^\s*(?:typedef\s+)?(?:pub\s+)?struct\s+(\w+)")),
    ("class", re.compile(r"^\s*(?:export\s+)?(?:abstract\s+)?class\s+(\w+)")),
    ("enum", re.compile(r"^\s*(?:pub\s+)?enum\s+(?:class\s+)?(\w+)")),
    ("namespace", re.compile(r"^\s*namespace\s+(\w+)")),
    ("function", re.compile(r"^\s*(?:pub(?:\([a-z]+\))?\s+)?(?:async\s+)?(?:fn|func|function)\s+(?:\([^)]*\)\s*)?(\w+)")),
    # C-family function definition: return type, name, argument list, no semicolon before the brace
    ("function", re.compile(r"^\s*(?:template\s*<[^>]*>\s*)?(?:(?:static|inline|extern|constexpr|virtual|__device__|__host__|__forceinline__|"
                            r"extern\s+\"C\")\s+)*[\w:<>,\*&\s]+?[\s\*&](\w+)\s*\([^;{}]*\)\s*(?:const\s*)?(?:noexcept\s*)?(?:->\s*[\w:<>]+\s*)?\{?\s*$")),
]
_NOT_FUNCTIONS = {"if", "for", "while", "switch", "return", "sizeof", "else", "do", "catch", "defined"}


def _block_end(lines: list[str], start: int) -> int:
    """Line (1-based) on which the brace block opened at or after line ``start`` closes; ``start`` when there is none."""
    depth, opened = 0, False
    for i in range(start - 1, min(len(lines), start + 2000)):
        code = re.sub(r'"(?:\\.|[^"\\])*"|//.*$', "", lines[i])
        for ch in code:
            if ch == "{":
                depth, opened = depth + 1, True
            elif ch == "}":
                depth -= 1
                if opened and depth == 0:
                    return i + 1
        if not opened and code.rstrip().endswith(";"):
            return i + 1
        if not opened and i > start + 3:
            return start
    return start


def _scan_definitions(path: Path):
    try:
        lines = path.read_text(errors="replace").splitlines()
    except OSError:
        return
    for i, line in enumerate(lines, 1):
        if not line.strip() or line.lstrip().startswith(("//", "*", "/*")):
            continue
        for kind, rx in _SCAN:
            m = rx.match(line)
            if not m:
                continue
            name = m.group(1)
            if kind == "function" and (name in _NOT_FUNCTIONS or line.rstrip().endswith(";")):
                continue
            end = i if kind == "macro" else _block_end(lines, i)
            if kind == "function" and end == i and "{" not in line:
                continue            # a declaration or a call that merely looked like a definition
            yield name, kind, i, end
            break


def _scan_references(path: Path, query: str):
    rx = re.compile(rf"(?<![\w]){re.escape(query)}(?![\w])")
    try:
        lines = path.read_text(errors="replace").splitlines()
    except OSError:
        return
    for i, line in enumerate(lines, 1):
        for m in rx.finditer(line):
            yield ("call" if line[m.end():].lstrip().startswith("(") else "reference"), i
            break


# ------------------------------------------------------------------------------------------ tree-sitter (optional)
def tree_sitter_available(lang: str = "python") -> bool:
    try:
        import tree_sitter  # noqa: F401
        __import__(f"tree_sitter_{lang}")
        return True
    except Exception:  # noqa: BLE001 - any import problem means "not available"
        return False


_TS_DEF_NODES = {"function_definition": "function", "class_definition": "class", "function_declaration": "function",
                 "method_definition": "method", "class_declaration": "class", "struct_specifier": "struct", "function_item": "function",
                 "struct_item": "struct", "enum_item": "enum", "impl_item": "class"}


def _ts_definitions(path: Path, lang: str):
    import tree_sitter

    mod = __import__(f"tree_sitter_{lang}")
    parser = tree_sitter.Parser(tree_sitter.Language(mod.language()))
    src = path.read_bytes()
    stack = [parser.parse(src).root_node]
    while stack:
        node = stack.pop()
        kind = _TS_DEF_NODES.get(node.type)
        if kind:
            ident = node.child_by_field_name("name")
            if ident is None:
                decl = node.child_by_field_name("declarator")
                while decl is not None and decl.type not in ("identifier", "field_identifier"):
                    decl = decl.child_by_field_name("declarator")
                ident = decl
            if ident is not None:
                yield src[ident.start_byte:ident.end_byte].decode(errors="replace"), kind, node.start_point[0] + 1, node.end_point[0] + 1
        stack.extend(reversed(node.children))


# ------------------------------------------------------------------------------------------ ctags (optional)
def ctags_available() -> bool:
    exe = shutil.which("ctags")
    if not exe:
        return False
    try:
        return "Universal Ctags" in subprocess.run([exe, "--version"], capture_output=True, text=True, timeout=5).stdout
    except (OSError, subprocess.SubprocessError):
        return False


_CTAGS_KINDS = {"f": "function", "c": "class", "m": "method", "v": "variable", "s": "struct", "g": "enum", "d": "macro",
                "n": "namespace", "t": "typedef", "p": "prototype", "e": "enumerator"}


def expand_ctags_kind(short: str) -> str:
    return _CTAGS_KINDS.get(short, short)


def parse_tags_file(tags_path: Path, query: str, exact: bool = True) -> list[dict]:
    """Entries of a ``tags`` file (``name<TAB>file<TAB>pattern;"<TAB>kind<TAB>line:N<TAB>end:M``) whose name matches."""
    out = []
    for line in Path(tags_path).read_text(errors="replace").splitlines():
        if line.startswith("!_TAG_"):
            continue
        parts = line.split("\t")
        if len(parts) < 4 or not _match(parts[0], query, exact):
            continue
        fields = {p.split(":", 1)[0]: p.split(":", 1)[1] for p in parts[3:] if ":" in p}
        kind = next((p for p in parts[3:] if ":" not in p), fields.get("kind", ""))
        ln = int(fields.get("line", "0") or 0)
        out.append({"name": parts[0], "file": parts[1], "kind": expand_ctags_kind(kind), "line": ln, "end": int(fields.get("end", ln) or ln)})
    return out


def build_ctags_index(root: Path) -> Path | None:
    if not ctags_available():
        return None
    tags = Path(root) / ".csearch.tags"
    rc = subprocess.run(["ctags", "-R", "--fields=+ne", "-f", str(tags), "."], cwd=root, capture_output=True, timeout=300)
    return tags if rc.returncode == 0 and tags.exists() else None


def search_definitions_ctags(query: str, options: SearchOptions) -> list[SearchResult]:
    root = options.path if Path(options.path).is_dir() else Path(options.path).parent
    tags = Path(root) / ".csearch.tags"
    if not tags.exists():
        tags = Path(root) / "tags" if (Path(root) / "tags").exists() else (build_ctags_index(root) or tags)
    if not tags.exists():
        return []
    res = [SearchResult(Location(Path(root) / e["file"], e["line"], e["end"]), e["name"], e["kind"])
           for e in parse_tags_file(tags, query, options.exact) if e["line"] > 0]
    return _finish(res, options)


# ------------------------------------------------------------------------------------------ public entry points
def _definitions_in(path: Path, backend: str):
    lang = LANG_BY_EXT.get(path.suffix)
    if backend in ("auto", "tree-sitter") and lang and tree_sitter_available("cpp" if lang == "cuda" else lang):
        try:
            yield from _ts_definitions(path, "cpp" if lang == "cuda" else lang)
            return
        except Exception:  # noqa: BLE001 - a grammar / API mismatch falls through to the built-in scanners
            pass
    if backend == "tree-sitter":
        return
    if lang == "python":
        if backend in ("auto", "ast"):
            yield from _py_definitions(path)
    elif backend in ("auto", "scan"):
        yield from _scan_definitions(path)


def search_definitions(query: str, options: SearchOptions = SearchOptions()) -> list[SearchResult]:
    """Definitions of ``query`` under ``options.path``."""
    if options.backend == "ctags":
        return search_definitions_ctags(query, options)
    res = []
    for f in find_files(options.path):
        for name, kind, a, b in _definitions_in(f, options.backend):
            if _match(name, query, options.exact):
                res.append(SearchResult(Location(f, a, b), name, kind))
    if not res and options.backend == "auto":
        return search_definitions_ctags(query, options)
    return _finish(res, options)


def list_symbols(options: SearchOptions = SearchOptions()) -> list[SearchResult]:
    """Every definition under ``options.path`` (an outline)."""
    res = [SearchResult(Location(f, a, b), name, kind) for f in find_files(options.path)
           for name, kind, a, b in _definitions_in(f, options.backend if options.backend != "ctags" else "auto")]
    return _finish(res, options)


def search_references(query: str, options: SearchOptions = SearchOptions()) -> list[SearchResult]:
    """Uses of ``query`` (reads, attribute accesses, calls) - syntactic, not type-resolved. Definitions themselves
    are not listed."""
    res = []
    for f in find_files(options.path):
        it = _py_references(f, query) if LANG_BY_EXT.get(f.suffix) == "python" else _scan_references(f, query)
        defs = {a for name, _, a, _ in _definitions_in(f, "auto") if name == query} if LANG_BY_EXT.get(f.suffix) != "python" else set()
        for kind, line in it or ():
            if line not in defs:
                res.append(SearchResult(Location(f, line, line), query, kind))
    return _finish(res, options)


def available_backends() -> dict[str, bool]:
    return {"tree-sitter": tree_sitter_available("python"), "ast": True, "scan": True, "ctags": ctags_available()}
