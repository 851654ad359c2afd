"""Single-file, syntax-aware refactorings for Python source: extract / inline variable, extract / inline function
(the operations of rollouts/tools/refactor-snipe/refactors/*.py). The reference drives tree-sitter; Python's own
``ast`` gives the same positions for the one language it supports, with nothing to install. Every function takes
source text and returns new source text, or raises ``RefactorError`` when the edit would not be safe."""

from __future__ import annotations

import ast


class RefactorError(ValueError):
    pass


def _lines(src: str) -> list[str]:
    return src.splitlines(keepends=True)


def _indent_of(line: str) -> str:
    return line[: len(line) - len(line.lstrip())]


def _replace_span(src: str, node: ast.AST, text: str) -> str:
    ls = _lines(src)
    a, b = node.lineno - 1, node.end_lineno - 1
    head, tail = ls[a][: _byte_to_col(ls[a], node.col_offset)], ls[b][_byte_to_col(ls[b], node.end_col_offset):]
    return "".join(ls[:a]) + head + text + tail + "".join(ls[b + 1:])


def _byte_to_col(line: str, byte_off: int) -> int:
    return len(line.encode()[:byte_off].decode())


def _stmt_containing(tree: ast.AST, node: ast.AST) -> ast.stmt:
    best = None
    for st in ast.walk(tree):
        if isinstance(st, ast.stmt) and st.lineno <= node.lineno and st.end_lineno >= node.end_lineno:
            if any(n is node for n in ast.walk(st)) and (best is None or st.lineno >= best.lineno):
                if not isinstance(st, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)) or st is node:
                    best = st if best is None or (st.end_lineno - st.lineno) <= (best.end_lineno - best.lineno) else best
    if best is None:
        raise RefactorError("expression is not inside a statement")
    return best


def _needs_parens(expr: ast.expr) -> bool:
    return not isinstance(expr, (ast.Name, ast.Constant, ast.Call, ast.Attribute, ast.Subscript, ast.List, ast.Tuple, ast.Dict,
                                 ast.Set, ast.ListComp, ast.DictComp, ast.SetComp, ast.GeneratorExp, ast.JoinedStr))


def extract_variable(src: str, expr_text: str, name: str, line: int) -> str:
    """Bind the expression ``expr_text`` found on ``line`` (1-based) to ``name`` just before its statement."""
    if not name.isidentifier():
        raise RefactorError(f"{name!r} is not an identifier")
    tree = ast.parse(src)
    want = ast.dump(ast.parse(expr_text.strip(), mode="eval").body)
    hits = [n for n in ast.walk(tree) if isinstance(n, ast.expr) and n.lineno <= line <= n.end_lineno and ast.dump(n) == want]
    if not hits:
        raise RefactorError(f"no expression {expr_text!r} on line {line}")
    node = min(hits, key=lambda n: (n.lineno != line, n.col_offset))
    stmt = _stmt_containing(tree, node)
    if isinstance(stmt, (ast.For, ast.While, ast.If, ast.With)) and node.lineno != stmt.lineno:
        raise RefactorError("expression spans a compound statement header and its body")
    out = _replace_span(src, node, name)
    ls = _lines(out)
    ind = _indent_of(ls[stmt.lineno - 1])
    ls.insert(stmt.lineno - 1, f"{ind}{name} = {ast.get_source_segment(src, node)}\n")
    return "".join(ls)


def _scope_of(tree: ast.AST, line: int) -> ast.AST:
    scope: ast.AST = tree
    for n in ast.walk(tree):
        if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)) and n.lineno <= line <= n.end_lineno:
            if scope is tree or n.lineno >= scope.lineno:  # innermost
                scope = n
    return scope


def inline_variable(src: str, name: str, line: int) -> str:
    """Replace the uses of ``name`` (assigned once, on ``line``) by its value and drop the assignment."""
    tree = ast.parse(src)
    scope = _scope_of(tree, line)
    assigns = [n for n in ast.walk(scope) if isinstance(n, ast.Assign) and n.lineno == line and len(n.targets) == 1
               and isinstance(n.targets[0], ast.Name) and n.targets[0].id == name]
    if not assigns:
        raise RefactorError(f"no simple assignment to {name!r} on line {line}")
    asg = assigns[0]
    stores = [n for n in ast.walk(scope) if isinstance(n, ast.Name) and n.id == name and isinstance(n.ctx, (ast.Store, ast.Del))]
    if len(stores) != 1 or any(isinstance(n, ast.AugAssign) and isinstance(n.target, ast.Name) and n.target.id == name
                               for n in ast.walk(scope)):
        raise RefactorError(f"{name!r} is bound more than once in its scope")
    value = ast.get_source_segment(src, asg.value)
    text = f"({value})" if _needs_parens(asg.value) else value
    loads = sorted((n for n in ast.walk(scope) if isinstance(n, ast.Name) and n.id == name and isinstance(n.ctx, ast.Load)),
                   key=lambda n: (n.lineno, n.col_offset), reverse=True)
    if any((n.lineno, n.col_offset) < (asg.end_lineno, asg.end_col_offset) for n in loads):
        raise RefactorError(f"{name!r} is read before its assignment")
    out = src
    for n in loads:                                   # back to front: earlier positions stay valid
        out = _replace_span(out, n, text)
    ls = _lines(out)
    del ls[asg.lineno - 1:asg.end_lineno]
    return "".join(ls)


def _names(nodes, ctx_types) -> list[str]:
    seen: list[str] = []
    for root in nodes:
        for n in ast.walk(root):
            if isinstance(n, ast.Name) and isinstance(n.ctx, ctx_types) and n.id not in seen:
                seen.append(n.id)
    return seen


def extract_function(src: str, start_line: int, end_line: int, name: str) -> str:
    """Move the whole statements on lines ``start_line..end_line`` into a new module-level function ``name``.
    Parameters are the names the block reads that its enclosing function bound earlier; returned are the names the
    block binds that are read afterwards."""
    if not name.isidentifier():
        raise RefactorError(f"{name!r} is not an identifier")
    tree = ast.parse(src)
    scope = _scope_of(tree, start_line)
    body_owner = None
    for n in ast.walk(scope):
        for field in ("body", "orelse", "finalbody"):
            stmts = getattr(n, field, None)
            if isinstance(stmts, list) and stmts and isinstance(stmts[0], ast.stmt):
                block = [s for s in stmts if s.lineno >= start_line and s.end_lineno <= end_line]
                if block and block[0].lineno == start_line and block[-1].end_lineno == end_line:
                    body_owner, chosen = stmts, block
    if body_owner is None:
        raise RefactorError("the line range does not cover whole statements of one block")
    for s in chosen:
        for n in ast.walk(s):
            if isinstance(n, (ast.Return, ast.Yield, ast.YieldFrom, ast.Break, ast.Continue, ast.Global, ast.Nonlocal)):
                raise RefactorError(f"block contains {type(n).__name__.lower()}: control flow would change")
    before = [s for s in ast.walk(scope) if isinstance(s, ast.stmt) and s.end_lineno < start_line]
    bound_before = set(_names(before, (ast.Store,)))
    if isinstance(scope, (ast.FunctionDef, ast.AsyncFunctionDef)):
        a = scope.args
        bound_before |= {x.arg for x in a.posonlyargs + a.args + a.kwonlyargs} | ({a.vararg.arg} if a.vararg else set()) | \
                        ({a.kwarg.arg} if a.kwarg else set())
    elif scope is tree:
        bound_before = set()         # module level: earlier names are globals, visible from the new function anyway
    params = [n for n in _names(chosen, (ast.Load,)) if n in bound_before]
    after = [s for s in ast.walk(scope) if isinstance(s, ast.stmt) and s.lineno > end_line]
    read_after = set(_names(after, (ast.Load,)))
    rets = [n for n in _names(chosen, (ast.Store,)) if n in read_after]
    ls = _lines(src)
    block_lines = ls[start_line - 1:end_line]
    ind = _indent_of(block_lines[0])
    body = "".join("    " + (bl[len(ind):] if bl.startswith(ind) else bl.lstrip()) if bl.strip() else bl for bl in block_lines)
    func = f"def {name}({', '.join(params)}):\n{body}"
    if rets:
        func += f"    return {', '.join(rets)}\n"
    call = f"{name}({', '.join(params)})"
    call_line = f"{ind}{', '.join(rets)} = {call}\n" if rets else f"{ind}{call}\n"
    top = scope
    if scope is not tree:                     # climb to the module-level statement that contains the block
        top = next(s for s in tree.body if s.lineno <= start_line <= s.end_lineno)
    insert_at = (top.lineno - 1 - len(getattr(top, "decorator_list", []))) if scope is not tree else start_line - 1
    new = ls[:start_line - 1] + [call_line] + ls[end_line:]
    new[insert_at:insert_at] = [func, "\n", "\n"]
    return "".join(new)


def inline_function(src: str, func_name: str, call_line: int) -> str:
    """Replace the call of ``func_name`` on ``call_line`` by the function's returned expression (functions whose body is
    a single ``return``; positional and keyword arguments, defaults honoured)."""
    tree = ast.parse(src)
    defs = [n for n in ast.walk(tree) if isinstance(n, ast.FunctionDef) and n.name == func_name]
    if len(defs) != 1:
        raise RefactorError(f"expected exactly one definition of {func_name!r}")
    fn = defs[0]
    body = [s for s in fn.body if not (isinstance(s, ast.Expr) and isinstance(s.value, ast.Constant) and isinstance(s.value.value, str))]
    if len(body) != 1 or not isinstance(body[0], ast.Return) or body[0].value is None or fn.args.vararg or fn.args.kwarg:
        raise RefactorError("only functions of the form `return <expression>` with plain parameters can be inlined")
    calls = [n for n in ast.walk(tree) if isinstance(n, ast.Call) and isinstance(n.func, ast.Name) and n.func.id == func_name
             and n.lineno <= call_line <= n.end_lineno]
    if not calls:
        raise RefactorError(f"no call of {func_name!r} on line {call_line}")
    call = calls[0]
    params = [a.arg for a in fn.args.posonlyargs + fn.args.args]
    binding: dict[str, str] = {}
    defaults = fn.args.defaults
    for p, d in zip(params[len(params) - len(defaults):], defaults):
        binding[p] = ast.get_source_segment(src, d)
    for p, a in zip(params, call.args):
        seg = ast.get_source_segment(src, a)
        binding[p] = f"({seg})" if _needs_parens(a) else seg
    for kw in call.keywords:
        if kw.arg is None or kw.arg not in params:
            raise RefactorError("unsupported keyword argument")
        seg = ast.get_source_segment(src, kw.value)
        binding[kw.arg] = f"({seg})" if _needs_parens(kw.value) else seg
    if set(params) - set(binding):
        raise RefactorError(f"arguments missing for {sorted(set(params) - set(binding))}")
    ret = body[0].value
    expr_src = ast.get_source_segment(src, ret)
    # substitute parameter names inside the returned expression, back to front
    sub = ast.parse(expr_src, mode="eval")
    names = sorted((n for n in ast.walk(sub) if isinstance(n, ast.Name) and n.id in binding),
                   key=lambda n: (n.lineno, n.col_offset), reverse=True)
    text = expr_src
    for n in names:
        text = _replace_span(text, n, binding[n.id])
    if _needs_parens(ret):
        text = f"({text})"
    return _replace_span(src, call, text)
