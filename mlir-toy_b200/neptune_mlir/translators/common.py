"""Shared helpers for HTile translators (B200 target).

Same entry-point shapes as the reference's module of this name
(src/neptune_mlir/translators/common.py:200-241): ``parse_mlir_module`` turns a ``.mlir`` path into a
module object after an optional pass pipeline, ``translate_file_with`` feeds it to a translator
class.  The reference shells out to ``mlir-opt`` and parses with ``mlir.ir``; here the stand-alone
C++ front end (``neptune_mlir.htile_native`` over libhtile_front.so) does that work, or, where that
library has not been built, the Python reader in ``neptune_mlir.htile_text`` with the rewrites in
``neptune_mlir.passes``; ``plugin`` / ``pass_plugin`` (paths to the dialect plugin there) are
accepted and unused.
"""

from __future__ import annotations

import ast
from typing import Type

from .. import htile_text as ht
from ..passes import PASS_PIPELINE, PassError, run_pipeline
from ..plugin import find_library_path

DEFAULT_LIBRARY = find_library_path()
DEFAULT_LIBRARY = None if DEFAULT_LIBRARY is None else DEFAULT_LIBRARY.as_posix()
HTILE_DOT_TRANSPOSE_TO_LOAD_ORDER_PIPELINE = PASS_PIPELINE


# ---------------------------------------------------------------------------
# AST helpers
# ---------------------------------------------------------------------------

def name(identifier: str) -> ast.Name:
    return ast.Name(id=identifier, ctx=ast.Load())


def const(value) -> ast.expr:
    if isinstance(value, tuple):
        return ast.Tuple(elts=[const(v) for v in value], ctx=ast.Load())
    return ast.Constant(value=value)


def call(func: ast.expr, *args: ast.expr, **kwargs: ast.expr) -> ast.Call:
    return ast.Call(func=func, args=list(args),
                    keywords=[ast.keyword(arg=k, value=v) for k, v in kwargs.items()])


def attr(value: ast.expr, attribute: str) -> ast.Attribute:
    return ast.Attribute(value=value, attr=attribute, ctx=ast.Load())


def function_def(fn_name: str, params: list[str], body: list[ast.stmt], doc: str | None = None) -> ast.FunctionDef:
    stmts: list[ast.stmt] = []
    if doc:
        stmts.append(ast.Expr(value=ast.Constant(value=doc)))
    stmts += body or [ast.Pass()]
    return ast.FunctionDef(
        name=fn_name,
        args=ast.arguments(posonlyargs=[], args=[ast.arg(arg=p, annotation=None) for p in params], vararg=None,
                           kwonlyargs=[], kw_defaults=[], kwarg=None, defaults=[]),
        body=stmts, decorator_list=[], returns=None, lineno=0, col_offset=0)


# ---------------------------------------------------------------------------
# MLIR helpers
# ---------------------------------------------------------------------------

def dot_transpose_attrs(op: ht.Op) -> list[str]:
    # presence decides, as in the reference (common.py:179-184): a unit attribute has no value to test
    return [n for n in ("transpose_a", "transpose_b") if op.attributes.get(n) is not None]


def reject_dot_transpose_attrs(op: ht.Op, backend: str) -> None:
    """Same contract and message as the reference (common.py:187-197)."""
    found = dot_transpose_attrs(op)
    if not found:
        return
    raise NotImplementedError(
        f"{backend} translation requires htile.dot transpose attributes "
        f"to be fissioned before emission; found {', '.join(found)}. "
        "Run the htile-dot-transpose-to-load-order pass, or inspect "
        "why that pass did not rewrite this dot.")


def parse_mlir_module(path: str, plugin: str | None = None, pass_pipeline: str | None = None,
                      pass_plugin: str | None = None) -> ht.Module:
    """Read *path* and run *pass_pipeline* (mlir-opt pipeline syntax) over it.

    Errors surface the way the reference's do (common.py:218-224): a RuntimeError carrying the
    diagnostic, here the reader's or the pass's own message.
    """
    del plugin, pass_plugin
    try:
        if front_end() == "native":
            from .. import htile_native

            return htile_native.parse_file(path, pass_pipeline)
        module = ht.parse_file(path)
        return run_pipeline(module, pass_pipeline)
    except (ht.HTileSyntaxError, PassError) as exc:
        raise RuntimeError(f"HTile front end failed on {path}: {exc}") from exc


def front_end() -> str:
    """Which reader parses and rewrites programs: the C++ front end ("native") or the Python one ("python").

    ``$NEPTUNE_HTILE_FRONT`` chooses; unset, the C++ library is used when it has been built.  Both
    produce the same object model (checked over the program corpus by the tests).
    """
    import os

    choice = os.environ.get("NEPTUNE_HTILE_FRONT", "").strip().lower()
    if choice in ("native", "python"):
        return choice
    if choice:
        raise ValueError(f"NEPTUNE_HTILE_FRONT must be 'native' or 'python', got {choice!r}")
    from .. import htile_native

    return "native" if htile_native.available() else "python"


def translate_file_with(path: str, translator_cls: Type, plugin: str | None = None,
                        pass_pipeline: str | None = None, pass_plugin: str | None = None) -> ast.Module:
    module = parse_mlir_module(path, plugin, pass_pipeline, pass_plugin)
    return translator_cls().translate(module)
