"""Symbol search backends: Python ``ast``, the brace-matching scanner for C-family sources, the tags-file parser."""

from pathlib import Path

from research_b200.infra.csearch_symbols import (Location, SearchOptions, SearchResult, available_backends, expand_ctags_kind,
                                                 list_symbols, parse_tags_file, search_definitions, search_references)

PY = '''import os
LIMIT = 3

class Pool:
    size: int = 4

    @staticmethod
    def make():
        return Pool()

    def take(self, n):
        def helper(x):
            return x + LIMIT
        return helper(n)

async def fetch(url):
    p = Pool.make()
    return p.take(os.getpid())
'''

CU = '''#include <cuda.h>
#define TILE 128
namespace rb {
struct Params { int n; };
template <int BN>
__global__ void scale_kernel(const float* x, float* y, Params p) {
  int i = blockIdx.x;
  if (i < p.n) { y[i] = x[i] * 2.f; }
}
static inline int helper(int a, int b);
static inline int helper(int a, int b) {
  return a + b;
}
}  // namespace rb
extern "C" int launch(const float* x, float* y, int n) {
  rb::Params p{n};
  rb::scale_kernel<128><<<n, 1>>>(x, y, p);
  return rb::helper(n, TILE);
}
'''


def _tree(tmp_path: Path) -> Path:
    (tmp_path / "pkg").mkdir()
    (tmp_path / "pkg" / "pool.py").write_text(PY)
    (tmp_path / "pkg" / "k.cu").write_text(CU)
    (tmp_path / "pkg" / "__pycache__").mkdir()
    (tmp_path / "pkg" / "__pycache__" / "junk.py").write_text("def take(): pass\n")
    (tmp_path / "broken.py").write_text("def oops(:\n")
    return tmp_path


def test_python_definitions_and_references(tmp_path):
    root = _tree(tmp_path)
    o = SearchOptions(path=root)
    take = search_definitions("take", o)
    assert [(r.kind, r.location.line_start, r.location.line_end, r.location.path.name) for r in take] == [("method", 11, 14, "pool.py")]
    assert search_definitions("make", o)[0].location.line_start == 7            # the decorator belongs to the definition
    assert {(r.name, r.kind) for r in search_definitions("Pool", o)} == {("Pool", "class")}
    assert [(r.kind, r.location.line_start) for r in search_definitions("LIMIT", o)] == [("variable", 2)]
    assert search_definitions("helper", SearchOptions(path=root / "pkg" / "pool.py"))[0].kind == "function"
    assert {r.name for r in search_definitions("e", SearchOptions(path=root, exact=False, backend="ast"))} >= {"take", "make", "helper", "fetch", "size"}
    refs = search_references("take", o)
    assert [(r.kind, r.location.line_start) for r in refs if r.location.path.suffix == ".py"] == [("call", 18)]
    assert {(r.kind, r.location.line_start) for r in search_references("LIMIT", SearchOptions(path=root / "pkg" / "pool.py"))} == {("reference", 13)}
    with_snip = search_definitions("fetch", SearchOptions(path=root, include_snippet=True))[0]
    assert with_snip.snippet.startswith("async def fetch") and "16-18" in str(with_snip.location)
    assert "async def fetch" in with_snip.format_with_snippet() and with_snip.format_compact().endswith("function fetch")


def test_c_family_scanner(tmp_path):
    root = _tree(tmp_path)
    o = SearchOptions(path=root / "pkg" / "k.cu")
    out = {(r.name, r.kind): (r.location.line_start, r.location.line_end) for r in list_symbols(o)}
    assert out[("scale_kernel", "kernel")] == (6, 9) and out[("Params", "struct")] == (4, 4) and out[("TILE", "macro")] == (2, 2)
    assert out[("helper", "function")] == (11, 13)            # the definition, not the declaration on line 10
    assert out[("launch", "function")] == (15, 19) and out[("rb", "namespace")][0] == 3
    refs = search_references("helper", o)
    assert [(r.kind, r.location.line_start) for r in refs] == [("call", 10), ("call", 18)] or \
        [(r.kind, r.location.line_start) for r in refs] == [("call", 18)]
    assert [r.location.line_start for r in search_references("scale_kernel", o)] == [17]
    assert search_definitions("scale_kernel", SearchOptions(path=root, limit=1))[0].kind == "kernel"


def test_tags_parser_and_backends(tmp_path):
    tags = tmp_path / "tags"
    tags.write_text("!_TAG_FILE_FORMAT\t2\n"
                    "take\tpkg/pool.py\t/^    def take(self, n):$/;\"\tm\tline:11\tclass:Pool\tend:14\n"
                    "Pool\tpkg/pool.py\t/^class Pool:$/;\"\tc\tline:4\tend:14\n"
                    "taken\tpkg/x.c\t/^int taken;$/;\"\tv\tline:3\n")
    e = parse_tags_file(tags, "take")
    assert e == [{"name": "take", "file": "pkg/pool.py", "kind": "method", "line": 11, "end": 14}]
    assert [x["name"] for x in parse_tags_file(tags, "take", exact=False)] == ["take", "taken"]
    assert expand_ctags_kind("s") == "struct" and expand_ctags_kind("zz") == "zz"
    res = search_definitions("Pool", SearchOptions(path=tmp_path, backend="ctags"))
    assert [(r.kind, str(r.location)) for r in res] == [("class", f"{tmp_path / 'pkg/pool.py'}:4-14")]
    b = available_backends()
    assert b["ast"] and b["scan"] and set(b) == {"tree-sitter", "ast", "scan", "ctags"}
    assert search_definitions("anything", SearchOptions(path=tmp_path / "nothing_here")) == []
    assert str(Location(Path("a.py"), 3, 3)) == "a.py:3" and isinstance(res[0], SearchResult)
