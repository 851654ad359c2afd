"""Syntax-aware refactorings and the comment-driven multi-file refactor tool."""

import asyncio

import pytest

from research_b200.infra.refactor_snipe import (RefactorError, extract_function, extract_variable, inline_function,
                                                inline_variable)

SRC = '''import math


def area(r, scale=2):
    k = math.pi * r * r
    total = k * scale + 1
    print(total)
    return total


def double(x, y=1):
    """Twice x plus y."""
    return 2 * x + y


z = double(3 + 1) * 5
'''


def run(src):
    ns = {}
    exec(compile(src, "<t>", "exec"), ns)
    return ns


def test_extract_and_inline_variable():
    out = extract_variable(SRC, "math.pi * r", "pr", 5)
    assert "    pr = math.pi * r\n    k = pr * r\n" in out
    assert run(out)["area"](2.0) == run(SRC)["area"](2.0)
    back = inline_variable(out, "pr", 5)
    assert "k = (math.pi * r) * r" in back and "pr =" not in back and run(back)["area"](2.0) == run(SRC)["area"](2.0)
    out2 = inline_variable(SRC, "k", 5)
    assert "total = (math.pi * r * r) * scale + 1" in out2 and "k =" not in out2
    with pytest.raises(RefactorError):
        inline_variable(SRC + "\nz = 1\nz = 2\nprint(z)\n", "z", 18)
    with pytest.raises(RefactorError):
        extract_variable(SRC, "nothing + here", "v", 5)


def test_extract_function():
    out = extract_function(SRC, 5, 6, "compute_total")
    assert "def compute_total(r, scale):\n    k = math.pi * r * r\n    total = k * scale + 1\n    return total\n" in out
    assert "    total = compute_total(r, scale)\n" in out
    assert run(out)["area"](3.0, 4) == run(SRC)["area"](3.0, 4)
    assert out.index("def compute_total") < out.index("def area")
    with pytest.raises(RefactorError):
        extract_function(SRC, 7, 8, "f")            # contains a return
    with pytest.raises(RefactorError):
        extract_function(SRC, 5, 5 + 10, "f")       # not whole statements of one block


def test_inline_function():
    out = inline_function(SRC, "double", 16)
    assert "z = (2 * (3 + 1) + 1) * 5" in out
    assert run(out)["z"] == run(SRC)["z"] == 45
    kw = inline_function(SRC.replace("double(3 + 1)", "double(y=4, x=2)"), "double", 16)
    assert "z = (2 * 2 + 4) * 5" in kw
    with pytest.raises(RefactorError):
        inline_function(SRC, "area", 16)


def test_task_extraction_context_and_edits(tmp_path):
    from research_b200.infra.refactor_task import apply_edits, collect_context, extract_task, parse_edits, refactor

    (tmp_path / "pkg").mkdir()
    (tmp_path / "pkg" / "__init__.py").write_text("")
    (tmp_path / "pkg" / "utils.py").write_text("from .deep import leaf\n\ndef helper(x):\n    return leaf(x) + 1\n")
    (tmp_path / "pkg" / "deep.py").write_text("def leaf(x):\n    return x * 2\n")
    main = tmp_path / "main.py"
    main.write_text("from pkg.utils import helper\n\nprint(helper(2))\n\n# move helper to pkg/helpers.py\n\n# and update the import\n")

    code, task = extract_task(main.read_text())
    assert task == "move helper to pkg/helpers.py\nand update the import" and code.endswith("print(helper(2))\n") and "#" not in code
    assert extract_task("x = 1\n")[1] == "" and extract_task("a()\n// do it\n", ".js")[1] == "do it"
    ctx = collect_context(main, tmp_path)
    assert set(ctx) == {"main.py", "pkg/utils.py", "pkg/deep.py"}

    reply = ('<write file="pkg/helpers.py">from .deep import leaf\n\ndef helper(x):\n    return leaf(x) + 1\n</write>\n'
             '<patch file="main.py"><search>from pkg.utils import helper</search><replace>from pkg.helpers import helper</replace></patch>\n'
             '<delete file="pkg/utils.py"/>')
    edits = parse_edits(reply)
    assert [e.kind for e in edits] == ["write", "patch", "delete"]
    seen = {}

    async def complete(prompt):
        seen["prompt"] = prompt
        return reply

    planned = asyncio.run(refactor(main, complete, root=tmp_path, dry_run=True))
    assert len(planned) == 3 and (tmp_path / "pkg" / "utils.py").exists() and "# move helper" in main.read_text()
    assert "TASK:\nmove helper" in seen["prompt"] and '<file path="pkg/deep.py">' in seen["prompt"] and "# move helper" not in seen["prompt"]
    asyncio.run(refactor(main, complete, root=tmp_path))
    assert not (tmp_path / "pkg" / "utils.py").exists() and (tmp_path / "pkg" / "helpers.py").exists()
    assert main.read_text() == "from pkg.helpers import helper\n\nprint(helper(2))\n"
    with pytest.raises(ValueError):
        apply_edits(parse_edits('<write file="../escape.py">x</write>'), tmp_path)
    with pytest.raises(ValueError):
        apply_edits(parse_edits('<patch file="main.py"><search>absent</search><replace>y</replace></patch>'), tmp_path)
    assert main.read_text() == "from pkg.helpers import helper\n\nprint(helper(2))\n"      # failed edits wrote nothing


def test_context_from_includes_and_markers_compaction_and_run_log(tmp_path):
    from research_b200.infra.refactor_task import collect_context, compact_context, refactor

    (tmp_path / "inc").mkdir()
    (tmp_path / "inc" / "tile.h").write_text('#include "util.h"\nint tile();\n')
    (tmp_path / "inc" / "util.h").write_text("int util();\n")
    (tmp_path / "notes.txt").write_text("layout notes " * 20)
    (tmp_path / "big.py").write_text("X = 1\n" + "# filler\n" * 400 + "Y = 2\n")
    kern = tmp_path / "kern.cu"
    kern.write_text('#include <cuda.h>\n#include "inc/tile.h"\n//[./notes.txt]\n//[./absent.txt]\nint main() { return tile(); }\n')
    assert set(collect_context(kern, tmp_path)) == {"kern.cu", "inc/tile.h", "inc/util.h", "notes.txt"}

    main = tmp_path / "main.py"
    main.write_text("import big\n#[./notes.txt]\nprint(big.X)\n\n# rename X to WIDTH\n")
    prompts = []

    async def complete(prompt):
        prompts.append(prompt)
        if "NOT needed" in prompt:
            return '<omit file="notes.txt"/>\n<omit file="main.py"/>\n<omit file="never/offered.py"/>'
        return '<patch file="main.py"><search>big.X</search><replace>big.WIDTH</replace></patch>'

    # under the threshold nothing is asked; above it the model's omissions apply, except to the entry file
    ctx = collect_context(main, tmp_path)
    assert asyncio.run(compact_context(ctx, "t", complete, threshold_tokens=10**6)) is ctx and not prompts
    log = asyncio.run(refactor(main, complete, root=tmp_path, compaction_threshold_tokens=200, log_dir=tmp_path / "logs"))
    assert log == ["patch main.py"] and len(prompts) == 2 and "notes.txt" in prompts[0]
    assert '<file path="notes.txt">' not in prompts[1] and '<file path="main.py">' in prompts[1] and '<file path="big.py">' in prompts[1]
    assert "big.WIDTH" in main.read_text()
    saved = list((tmp_path / "logs").iterdir())
    assert len(saved) == 1 and saved[0].name.endswith("_main.log") and "# applied\npatch main.py" in saved[0].read_text()
