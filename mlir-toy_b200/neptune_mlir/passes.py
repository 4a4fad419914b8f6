"""Rewrites on the HTile object model.

``dot_transpose_to_load_order`` reproduces the observable result of the reference's only pass,
``htile-dot-transpose-to-load-order`` (lib/HTile/HTilePasses.cpp:52-141), whose post-conditions the
reference asserts at tests/test_translators.py:250-257:

1. every ``transpose_a`` / ``transpose_b`` unit attribute on an ``htile.dot`` becomes an explicit
   ``htile.permute ... permutation [1, 0]`` on that operand (rank-2 operands only);
2. a permute whose input is produced by an ``htile.load`` is folded into a new load that carries
   the permuted result type and a ``dimension_order`` array (composed with an existing one);
   the old load is dropped when nothing else uses it.

For the B200 target the folded form is also the cheap one: a K tile loaded row-major and used as
``B^T`` is simply a K-major tcgen05 operand, so no data movement is implied.
"""

from __future__ import annotations

from .htile_text import Block, Func, Module, Op, TensorType, Value

DIMENSION_ORDER = "dimension_order"  # lib/HTile/HTilePasses.cpp:20


class PassError(RuntimeError):
    pass


def _all_ops(module: Module):
    return list(module.walk())


def _replace_all_uses(module: Module, old: Value, new: Value) -> None:
    for op in module.walk():
        op.operands = [new if v is old else v for v in op.operands]


def _has_uses(module: Module, value: Value) -> bool:
    return any(any(v is value for v in op.operands) for op in module.walk())


def _insert_before(anchor: Op, new_op: Op) -> None:
    block: Block = anchor.parent
    block.operations.insert(block.operations.index(anchor), new_op)
    new_op.parent = block


def _erase(op: Op) -> None:
    op.parent.operations.remove(op)


def _permuted(ty: TensorType, perm) -> TensorType:
    return ty.with_shape(ty.shape[p] for p in perm)


def _fission(dot: Op, fresh) -> None:
    for attr, idx in (("transpose_a", 0), ("transpose_b", 1)):
        if not dot.attributes.get(attr):
            continue
        src = dot.operands[idx]
        if not isinstance(src.type, TensorType) or len(src.type.shape) != 2:
            side = "lhs" if idx == 0 else "rhs"
            raise PassError(f"htile.dot: {attr} fission expects a rank-2 {side}")  # HTilePasses.cpp:96-97,108-109
        permute = Op("htile.permute", operands=[src], attributes={"permutation": [1, 0]})
        permute.results = [Value(fresh(), _permuted(src.type, (1, 0)), permute, 0)]
        _insert_before(dot, permute)
        dot.operands[idx] = permute.result
        del dot.attributes[attr]


def _fold_into_load(module: Module, permute: Op, fresh) -> None:
    load = permute.operands[0].owner
    if not isinstance(load, Op) or load.name != "htile.load":
        return
    perm = list(permute.attributes["permutation"])
    existing = list(load.attributes.get(DIMENSION_ORDER, range(len(perm))))
    fused = Op("htile.load", operands=list(load.operands), attributes=dict(load.attributes))
    fused.attributes[DIMENSION_ORDER] = [existing[p] for p in perm]      # HTilePasses.cpp:31-45
    fused.results = [Value(fresh(), permute.result.type, fused, 0)]
    _insert_before(permute, fused)
    _replace_all_uses(module, permute.result, fused.result)
    _erase(permute)
    if not _has_uses(module, load.result):
        _erase(load)


def dot_transpose_to_load_order(module: Module) -> Module:
    """Apply the rewrite in place and return the module."""
    counter = [0]

    def fresh() -> str:
        counter[0] += 1
        return f"_t2lo{counter[0]}"

    for op in _all_ops(module):
        if op.name == "htile.dot" and (op.attributes.get("transpose_a") or op.attributes.get("transpose_b")):
            _fission(op, fresh)
    for op in _all_ops(module):
        if op.name == "htile.permute":
            _fold_into_load(module, op, fresh)
    return module


PASS_PIPELINE = "builtin.module(htile-dot-transpose-to-load-order,cse,canonicalize)"  # common.py:16-18


def run_pipeline(module: Module, pipeline: str | None) -> Module:
    """Run a pass pipeline given in mlir-opt syntax; only the reference's own pipeline is known."""
    if pipeline is None:
        return module
    inner = pipeline.strip()
    if inner.startswith("builtin.module(") and inner.endswith(")"):
        inner = inner[len("builtin.module("):-1]
    for name in filter(None, (p.strip() for p in inner.split(","))):
        if name == "htile-dot-transpose-to-load-order":
            dot_transpose_to_load_order(module)
        elif name in ("cse", "canonicalize"):
            continue  # no effect on what the B200 recogniser reads
        else:
            raise PassError(f"unknown pass '{name}'")
    return module


__all__ = ["dot_transpose_to_load_order", "run_pipeline", "PassError", "PASS_PIPELINE", "DIMENSION_ORDER",
           "Func"]
