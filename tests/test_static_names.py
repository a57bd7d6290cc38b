"""Every name a function of the package loads is defined somewhere it can see.

Most of the cuda backend's host code never runs on a machine without a GPU, so a misspelt or out-of-scope variable
there would only surface on the GPU box.  This walks the syntax trees with Python's scoping rules (function locals
and parameters, enclosing functions, module globals, builtins; class bodies are not visible from methods) and fails
on loads that resolve nowhere.
"""

from __future__ import annotations

import ast
import builtins
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
FILES = sorted(p for p in list((ROOT / "moeflow_b200").rglob("*.py")) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]
               if "__pycache__" not in p.parts)


def _bound_in(node: ast.AST) -> set[str]:
    """Names bound directly in this scope (not inside nested function or class scopes; comprehensions count as part
    of the scope, which only makes the check more permissive)."""
    out: set[str] = set()

    def visit(n: ast.AST, top: bool) -> None:
        if not top and isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
            out.add(n.name)
            return  # its body is another scope
        if not top and isinstance(n, ast.Lambda):
            return
        if isinstance(n, ast.Name) and isinstance(n.ctx, (ast.Store, ast.Del)):
            out.add(n.id)
        elif isinstance(n, (ast.Import, ast.ImportFrom)):
            for a in n.names:
                out.add((a.asname or a.name).split(".")[0])
        elif isinstance(n, ast.ExceptHandler) and n.name:
            out.add(n.name)
        elif isinstance(n, (ast.Global, ast.Nonlocal)):
            out.update(n.names)
        elif isinstance(n, ast.MatchAs) and n.name:
            out.add(n.name)
        for c in ast.iter_child_nodes(n):
            visit(c, False)

    visit(node, True)
    return out


def _params(fn: ast.FunctionDef | ast.AsyncFunctionDef | ast.Lambda) -> set[str]:
    a = fn.args
    names = [x.arg for x in a.posonlyargs + a.args + a.kwonlyargs]
    if a.vararg:
        names.append(a.vararg.arg)
    if a.kwarg:
        names.append(a.kwarg.arg)
    return set(names)


def undefined_names(source: str) -> list[tuple[int, str]]:
    tree = ast.parse(source)
    module_names = _bound_in(tree) | set(dir(builtins)) | {"__file__", "__name__", "__doc__", "__spec__", "__package__"}
    problems: list[tuple[int, str]] = []

    def check(scope: ast.AST, visible: set[str]) -> None:
        """`scope` is a function, lambda, class or the module; `visible` holds every name its code can load."""

        def walk(n: ast.AST, top: bool) -> None:
            if not top and isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef, ast.Lambda)):
                # decorators, defaults and annotations are evaluated in the enclosing scope
                outer = list(n.args.defaults) + [d for d in n.args.kw_defaults if d is not None]
                if not isinstance(n, ast.Lambda):
                    outer += list(n.decorator_list)
                for d in outer:
                    walk(d, False)
                inner = visible | _params(n) | _bound_in(n)  # a lambda binds comprehension targets in its body
                check(n, inner)
                return
            if not top and isinstance(n, ast.ClassDef):
                for d in list(n.decorator_list) + list(n.bases) + [k.value for k in n.keywords]:
                    walk(d, False)
                # the class body sees its own names; the methods inside do not (they get `visible` only)
                body_names = visible | _bound_in(n)
                for stmt in n.body:
                    if isinstance(stmt, (ast.FunctionDef, ast.AsyncFunctionDef)):
                        walk(stmt, False)
                    else:
                        saved = set(visible)
                        visible.update(body_names)
                        walk(stmt, False)
                        visible.clear()
                        visible.update(saved)
                return
            if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Load) and n.id not in visible:
                problems.append((n.lineno, n.id))
            for c in ast.iter_child_nodes(n):
                if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)) and top and c is n.args:
                    continue  # parameter annotations/defaults were handled by the enclosing scope
                if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)) and top and (c in n.decorator_list or c is n.returns):
                    continue
                walk(c, False)

        walk(scope, True)

    check(tree, set(module_names))
    return problems


def test_the_checker_sees_an_out_of_scope_name_and_accepts_closures():
    bad = "class A:\n    def __init__(self, w):\n        self.w = w\n    def later(self):\n        return w is None\n"
    assert undefined_names(bad) == [(5, "w")]
    good = ("import os\nX = 1\n"
            "def f(a, *rest, k=2, **kw):\n    b = [i for i in range(a)]\n    def g():\n        return b, X, os, rest, kw, k\n"
            "    try:\n        pass\n    except ValueError as e:\n        print(e)\n    return g, (lambda q: q + a)\n"
            "class C:\n    y = X\n    z = y\n    def m(self):\n        return C, X\n")
    assert undefined_names(good) == []


@pytest.mark.parametrize("path", FILES, ids=lambda p: str(p.relative_to(ROOT)))
def test_no_function_loads_a_name_it_cannot_see(path):
    assert undefined_names(path.read_text()) == []
