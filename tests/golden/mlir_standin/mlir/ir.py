"""Stand-in for the handful of ``mlir.ir`` names the reference's Python translators touch.

Test infrastructure only.  The reference's translators (src/neptune_mlir/translators/common.py:10,
triton.py:12) import the LLVM project's ``mlir.ir`` bindings, which are not installed anywhere this
build runs, so those translators cannot even be imported.  This module offers the same names with
the same behaviour for the accessors they use -- ``operation.name``, ``operands``, ``results``,
``attributes.get``, ``regions[i].blocks[j].{operations,arguments}``, ``Value.type/.owner``, the two
shaped types with ``shape``/``element_type``, and the attribute classes used as casts -- on top of
the object model of ``neptune_mlir.htile_text``.  With it the UNMODIFIED reference translator emits
its kernels for HTile programs of other shapes and element types than its one test program, which
are then run (Triton interpreter, CPU) to pin this build's oracle: ``make_reference_translations.py``.
The stand-in itself is checked by reproducing the reference's golden translation byte for byte.
"""

from __future__ import annotations

import struct


# ---- types ------------------------------------------------------------------------------------
class Type:
    def __init__(self, text: str):
        self._text = text

    def __str__(self) -> str:
        return self._text

    def __eq__(self, other) -> bool:
        return isinstance(other, Type) and str(other) == self._text

    def __hash__(self) -> int:
        return hash(self._text)


class _Shaped(Type):
    def __init__(self, text: str, shape, element_type: Type):
        super().__init__(text)
        self.shape = list(shape)
        self.element_type = element_type


class RankedTensorType(_Shaped):
    pass


class MemRefType(_Shaped):
    pass


# ---- attributes -------------------------------------------------------------------------------
class Attribute:
    """Constructing a subclass from an attribute of that kind is a checked cast, as in ``mlir.ir``."""

    _kinds: tuple = ()

    def __init__(self, value):
        if isinstance(value, Attribute):
            if not isinstance(value, type(self)):
                raise ValueError(f"cannot cast {type(value).__name__} to {type(self).__name__}")
            value = value._value
        self._value = value

    def __str__(self) -> str:
        return str(self._value)


class IntegerAttr(Attribute):
    @property
    def value(self) -> int:
        return int(self._value)


class FloatAttr(Attribute):
    @property
    def value(self) -> float:
        return float(self._value)


class StringAttr(Attribute):
    @property
    def value(self) -> str:
        return str(self._value)


class UnitAttr(Attribute):
    pass


class DenseI64ArrayAttr(Attribute):
    def __iter__(self):
        return iter(self._value)

    def __len__(self) -> int:
        return len(self._value)


class _AttrDict(dict):
    """``op.attributes``: ``get`` plus ``in`` and indexing, which is all the translators use."""


# ---- SSA objects ------------------------------------------------------------------------------
class Value:
    def __init__(self, type_: Type, owner=None):
        self.type = type_
        self.owner = owner

    def __str__(self) -> str:
        return f"Value({self.type})"


class Block:
    def __init__(self):
        self.arguments: list[Value] = []
        self.operations: list["Operation"] = []


class Region:
    def __init__(self, block: Block):
        self.blocks = [block]


class Operation:
    def __init__(self, name: str):
        self.name = name
        self.operands: list[Value] = []
        self.results: list[Value] = []
        self.attributes = _AttrDict()
        self.regions: list[Region] = []

    @property
    def operation(self) -> "Operation":
        return self


class OpView:
    """Never instantiated here: every op is a plain ``Operation`` (as for unregistered dialects)."""


class _Body:
    def __init__(self, operations):
        self.operations = operations


class Module:
    def __init__(self, operations):
        self.body = _Body(list(operations))

    @staticmethod
    def parse(text: str) -> "Module":
        raise NotImplementedError("the stand-in is built from neptune_mlir.htile_text objects (from_htile)")


class Context:
    allow_unregistered_dialects = False

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


# ---- construction from the HTile text reader's object model --------------------------------------
def _round_f32(x: float) -> float:
    return struct.unpack("f", struct.pack("f", x))[0]


def _convert_type(t) -> Type:
    from neptune_mlir import htile_text as ht

    if isinstance(t, ht.TensorType):
        return RankedTensorType(str(t), t.shape, Type(str(t.element_type)))
    if isinstance(t, ht.MemRefType):
        return MemRefType(str(t), t.shape, Type(str(t.element_type)))
    return Type(str(t))


def _convert_attr(key: str, value, op):
    if key == "value" and op.name == "arith.constant":
        ty = str(op.results[0].type)
        if ty.startswith("f") or ty.startswith("bf"):
            v = float(value)
            return FloatAttr(_round_f32(v) if ty in ("f32", "f16", "bf16") else v)
        return IntegerAttr(int(value))
    if value is True:
        return UnitAttr(True)
    if isinstance(value, bool):
        return IntegerAttr(int(value))
    if isinstance(value, int):
        return IntegerAttr(value)
    if isinstance(value, float):
        return FloatAttr(value)
    if isinstance(value, str):
        return StringAttr(value)
    if isinstance(value, (list, tuple)):
        return DenseI64ArrayAttr([int(v) for v in value])
    raise NotImplementedError(f"attribute {key} = {value!r}")


def from_htile(module) -> Module:
    """Wrap a ``neptune_mlir.htile_text.Module`` (already canonical: see make_reference_translations.py)."""
    values: dict[int, Value] = {}

    def val(v, owner=None) -> Value:
        got = values.get(id(v))
        if got is None:
            got = values[id(v)] = Value(_convert_type(v.type), owner)
        return got

    def block(b) -> Block:
        out = Block()
        out.arguments = [val(a, out) for a in b.arguments]
        for o in b.operations:
            out.operations.append(op(o))
        return out

    def op(o) -> Operation:
        out = Operation(o.name)
        out.operands = [val(v) for v in o.operands]
        out.results = [val(r, out) for r in o.results]
        for k, v in o.attributes.items():
            out.attributes[k] = _convert_attr(k, v, o)
        out.regions = [Region(block(r)) for r in o.regions]
        return out

    funcs = []
    for fn in module.functions:
        f = Operation("func.func")
        f.attributes["sym_name"] = StringAttr(fn.name)
        entry = block(fn.body)
        f.regions = [Region(entry)]
        funcs.append(f)
    return Module(funcs)
