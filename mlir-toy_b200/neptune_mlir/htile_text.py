"""A stand-alone reader (and printer) for the textual form of HTile programs.

The reference hands a ``.mlir`` file to ``mlir-opt`` with the HTile dialect plugin loaded and parses
the generic-form output with the upstream ``mlir.ir`` bindings
(src/neptune_mlir/translators/common.py:200-229).  Neither tool is needed here: this module reads
the custom assembly of the eleven HTile ops (include/HTile/HTileOps.td:21-217), the
``#htile.encoding`` attribute (include/HTile/HTileAttrs.td:5-29) and the upstream ops that HTile
programs use around them (func, arith, math, scf.for, gpu.launch, linalg.broadcast, tensor.empty)
into a small SSA object model.  It is a strict subset reader: anything it does not know raises
``HTileSyntaxError`` instead of being skipped.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Any

__all__ = [
    "HTileSyntaxError", "MemRefType", "TensorType", "ScalarType", "Value", "Op", "Block", "Func",
    "Module", "parse_module", "parse_file", "print_module", "parse_type",
]


class HTileSyntaxError(ValueError):
    """The text is not in the subset of MLIR that this reader understands."""


# ---------------------------------------------------------------------------------------------
# types
# ---------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class ScalarType:
    name: str  # f16, bf16, f32, f64, i1, i8 ... i64, index

    def __str__(self) -> str:
        return self.name


@dataclass(frozen=True)
class MemRefType:
    shape: tuple[int, ...]
    element_type: ScalarType

    def __str__(self) -> str:
        return "memref<" + "x".join([*map(str, self.shape), str(self.element_type)]) + ">"


@dataclass(frozen=True)
class TensorType:
    shape: tuple[int, ...]
    element_type: ScalarType
    placement: str | None = None  # "shared" / "local" (the #htile.encoding placement) or None

    def __str__(self) -> str:
        body = "x".join([*map(str, self.shape), str(self.element_type)])
        if self.placement is not None:
            body += f", #htile.encoding<placement = {self.placement}>"
        return f"tensor<{body}>"

    def with_shape(self, shape) -> "TensorType":
        return TensorType(tuple(shape), self.element_type, self.placement)


_SCALAR_RE = re.compile(r"(bf16|f16|f32|f64|index|i1|i8|i16|i32|i64)\b")


# ---------------------------------------------------------------------------------------------
# SSA object model
# ---------------------------------------------------------------------------------------------

class Value:
    """An SSA value: a block argument (owner is a Block) or an op result (owner is an Op)."""

    __slots__ = ("name", "type", "owner", "index")

    def __init__(self, name: str, type_: Any, owner: Any = None, index: int = 0):
        self.name, self.type, self.owner, self.index = name, type_, owner, index

    def __repr__(self) -> str:
        return f"Value(%{self.name}: {self.type})"


@dataclass(eq=False)
class Op:
    name: str
    operands: list[Value] = field(default_factory=list)
    results: list[Value] = field(default_factory=list)
    attributes: dict[str, Any] = field(default_factory=dict)
    regions: list["Block"] = field(default_factory=list)
    parent: "Block | None" = None

    @property
    def result(self) -> Value:
        if len(self.results) != 1:
            raise ValueError(f"{self.name} has {len(self.results)} results")
        return self.results[0]


@dataclass(eq=False)
class Block:
    arguments: list[Value] = field(default_factory=list)
    operations: list[Op] = field(default_factory=list)
    parent_op: Op | None = None

    def walk(self):
        for op in list(self.operations):
            yield op
            for region in op.regions:
                yield from region.walk()


@dataclass(eq=False)
class Func:
    name: str
    arguments: list[Value]
    attributes: dict[str, Any]
    body: Block


@dataclass(eq=False)
class Module:
    functions: list[Func]

    def walk(self):
        for fn in self.functions:
            yield from fn.body.walk()


# ---------------------------------------------------------------------------------------------
# parser
# ---------------------------------------------------------------------------------------------

_WS_RE = re.compile(r"(?:\s+|//[^\n]*)*")
_SSA_RE = re.compile(r"%([A-Za-z0-9_.$-]+)")
_IDENT_RE = re.compile(r"[A-Za-z_][A-Za-z0-9_.$]*")
_NUM_RE = re.compile(r"[-+]?(?:0x[0-9a-fA-F]+|\d+\.\d*(?:[eE][-+]?\d+)?|\d+[eE][-+]?\d+|\d+)")
_STR_RE = re.compile(r'"((?:[^"\\]|\\.)*)"')

_ELEMENTWISE_BINARY = {
    "arith.addf", "arith.subf", "arith.mulf", "arith.divf", "arith.maximumf", "arith.minimumf",
    "arith.addi", "arith.subi", "arith.muli", "arith.divsi", "arith.remsi", "arith.maxsi", "arith.minsi",
    "arith.andi", "arith.ori",
}
_ELEMENTWISE_UNARY = {"math.exp2", "math.exp", "math.log2", "math.log", "math.sqrt", "math.rsqrt",
                      "math.tanh", "arith.negf"}
_CASTS = {"arith.truncf", "arith.extf", "arith.sitofp", "arith.fptosi", "arith.index_cast"}


class _Parser:
    def __init__(self, text: str):
        self.text = text
        self.pos = 0
        self.aliases: dict[str, str] = {}
        self.scopes: list[dict[str, Value]] = []

    # -- low-level cursor helpers --
    def error(self, msg: str) -> HTileSyntaxError:
        line = self.text.count("\n", 0, self.pos) + 1
        snippet = self.text[self.pos:self.pos + 40].split("\n")[0]
        return HTileSyntaxError(f"line {line}: {msg} (at {snippet!r})")

    def ws(self) -> None:
        self.pos = _WS_RE.match(self.text, self.pos).end()

    def peek(self, s: str) -> bool:
        self.ws()
        return self.text.startswith(s, self.pos)

    def accept(self, s: str) -> bool:
        if self.peek(s):
            self.pos += len(s)
            return True
        return False

    def expect(self, s: str) -> None:
        if not self.accept(s):
            raise self.error(f"expected {s!r}")

    def match(self, regex: re.Pattern) -> re.Match | None:
        self.ws()
        m = regex.match(self.text, self.pos)
        if m:
            self.pos = m.end()
        return m

    def keyword(self, word: str) -> bool:
        self.ws()
        m = _IDENT_RE.match(self.text, self.pos)
        if m and m.group(0) == word:
            self.pos = m.end()
            return True
        return False

    def ident(self) -> str:
        m = self.match(_IDENT_RE)
        if not m:
            raise self.error("expected identifier")
        return m.group(0)

    # -- SSA scopes --
    def define(self, value: Value) -> Value:
        self.scopes[-1][value.name] = value
        return value

    def lookup(self, name: str) -> Value:
        for scope in reversed(self.scopes):
            if name in scope:
                return scope[name]
        raise self.error(f"use of undefined value %{name}")

    def ssa_name(self) -> str:
        m = self.match(_SSA_RE)
        if not m:
            raise self.error("expected SSA value")
        return m.group(1)

    def ssa_use(self) -> Value:
        return self.lookup(self.ssa_name())

    def ssa_use_list(self, close: str) -> list[Value]:
        vals: list[Value] = []
        if self.accept(close):
            return vals
        while True:
            vals.append(self.ssa_use())
            if self.accept(close):
                return vals
            self.expect(",")

    # -- types and attributes --
    def type(self):
        self.ws()
        for kind in ("memref", "tensor"):
            if self.text.startswith(kind + "<", self.pos):
                start = self.pos + len(kind) + 1
                depth, i = 1, start
                while depth:
                    if i >= len(self.text):
                        raise self.error("unterminated type")
                    depth += {"<": 1, ">": -1}.get(self.text[i], 0)
                    i += 1
                body = self.text[start:i - 1]
                self.pos = i
                return self._shaped(kind, body)
        m = self.match(_SCALAR_RE)
        if not m:
            raise self.error("expected type")
        return ScalarType(m.group(1))

    def _shaped(self, kind: str, body: str):
        dims_part, _, enc = body.partition(",")
        m = re.fullmatch(r"((?:\d+x)*)([A-Za-z][A-Za-z0-9]*)", dims_part.strip())
        if not m:
            raise self.error(f"dynamic or malformed shape in {kind}<{body}>")
        shape = tuple(int(p) for p in m.group(1).split("x") if p)
        parts = [m.group(2)]
        if not _SCALAR_RE.fullmatch(parts[-1]):
            raise self.error(f"unknown element type {parts[-1]!r}")
        elem = ScalarType(parts[-1].strip())
        if kind == "memref":
            if enc.strip():
                raise self.error("memref layouts / memory spaces are not supported")
            return MemRefType(shape, elem)
        placement = None
        enc = enc.strip()
        if enc:
            if enc.startswith("#") and enc[1:] in self.aliases:
                enc = self.aliases[enc[1:]]
            m = re.fullmatch(r"#htile\.encoding<\s*placement\s*=\s*(\w+)\s*>", enc)
            if not m or m.group(1) not in ("shared", "local"):
                raise self.error(f"unknown tensor encoding {enc!r}")
            placement = m.group(1)
        return TensorType(shape, elem, placement)

    def attr_value(self):
        self.ws()
        if self.accept("array<"):
            self.ident()  # i64 / i1
            vals = []
            if self.accept(":"):
                while True:
                    vals.append(self.attr_value())
                    if not self.accept(","):
                        break
            self.expect(">")
            return vals
        if self.accept("["):
            vals = []
            if not self.accept("]"):
                while True:
                    vals.append(self.attr_value())
                    if self.accept("]"):
                        break
                    self.expect(",")
            return vals
        m = self.match(_STR_RE)
        if m:
            return m.group(1)
        if self.keyword("true"):
            return True
        if self.keyword("false"):
            return False
        if self.keyword("unit"):
            return True
        m = self.match(_NUM_RE)
        if m:
            txt = m.group(0)
            val: Any = int(txt, 0) if re.fullmatch(r"[-+]?(0x[0-9a-fA-F]+|\d+)", txt) else float(txt)
            if self.accept(":"):
                self.type()
            return val
        raise self.error("unsupported attribute value")

    def attr_dict(self) -> dict[str, Any]:
        attrs: dict[str, Any] = {}
        if not self.accept("{"):
            return attrs
        if self.accept("}"):
            return attrs
        while True:
            self.ws()
            m = self.match(re.compile(r"[A-Za-z_][A-Za-z0-9_.$]*"))
            if not m:
                raise self.error("expected attribute name")
            key = m.group(0)
            attrs[key] = self.attr_value() if self.accept("=") else True  # bare name = unit attribute
            if self.accept("}"):
                return attrs
            self.expect(",")

    # -- module / function --
    def module(self) -> Module:
        funcs: list[Func] = []
        self.scopes.append({})
        while True:
            self.ws()
            if self.pos >= len(self.text):
                break
            m = re.compile(r"#([A-Za-z_][A-Za-z0-9_]*)\s*=\s*([^\n]+)").match(self.text, self.pos)
            if m:
                self.aliases[m.group(1)] = m.group(2).strip()
                self.pos = m.end()
                continue
            if self.keyword("module"):
                self.attr_dict_keyword()
                self.expect("{")
                while not self.accept("}"):
                    funcs.append(self.func())
                continue
            funcs.append(self.func())
        return Module(funcs)

    def attr_dict_keyword(self) -> dict[str, Any]:
        return self.attr_dict() if self.keyword("attributes") else {}

    def func(self) -> Func:
        if not self.keyword("func.func"):
            raise self.error("expected func.func")
        self.keyword("private") or self.keyword("public")
        self.expect("@")
        name = self.ident()
        self.expect("(")
        body = Block()
        self.scopes.append({})
        if not self.accept(")"):
            while True:
                an = self.ssa_name()
                self.expect(":")
                body.arguments.append(self.define(Value(an, self.type(), body, len(body.arguments))))
                if self.accept(")"):
                    break
                self.expect(",")
        if self.accept("->"):
            raise self.error("functions with results are not supported")
        attrs = self.attr_dict_keyword()
        self.expect("{")
        self.block_body(body, "}")
        self.scopes.pop()
        return Func(name, body.arguments, attrs, body)

    def block_body(self, block: Block, close: str) -> None:
        while not self.accept(close):
            op = self.operation()
            op.parent = block
            block.operations.append(op)

    # -- operations --
    def operation(self) -> Op:
        self.ws()
        result_names: list[str] = []
        if self.peek("%"):
            while True:
                nm = self.ssa_name()
                if self.accept(":"):                   # %a:3 packs are not used by HTile programs
                    raise self.error("result packs (%x:N) are not supported; name each result")
                result_names.append(nm)
                if not self.accept(","):
                    break
            self.expect("=")
        name = self.ident()
        op = Op(name)
        types = self.op_body(op)
        if len(types) != len(result_names):
            raise self.error(f"{name}: {len(result_names)} result names for {len(types)} results")
        for i, (nm, ty) in enumerate(zip(result_names, types)):
            op.results.append(self.define(Value(nm, ty, op, i)))
        return op

    def op_body(self, op: Op) -> list:
        """Parse everything after the op name; returns the result types."""
        n = op.name
        if n in ("return", "func.return", "gpu.terminator"):
            return []
        if n == "arith.constant":
            self.ws()
            op.attributes["value"] = self.attr_value_no_type()
            self.expect(":")
            return [self.type()]
        if n in _ELEMENTWISE_BINARY:
            op.operands = [self.ssa_use()]
            self.expect(",")
            op.operands.append(self.ssa_use())
            op.attributes.update(self.attr_dict())
            self.expect(":")
            return [self.type()]
        if n in _ELEMENTWISE_UNARY:
            op.operands = [self.ssa_use()]
            op.attributes.update(self.attr_dict())
            self.expect(":")
            return [self.type()]
        if n in _CASTS:
            op.operands = [self.ssa_use()]
            self.expect(":")
            self.type()
            if not self.keyword("to"):
                raise self.error("expected 'to'")
            return [self.type()]
        if n in ("arith.cmpi", "arith.cmpf"):
            op.attributes["predicate"] = self.ident()
            self.expect(",")
            op.operands = [self.ssa_use()]
            self.expect(",")
            op.operands.append(self.ssa_use())
            self.expect(":")
            ty = self.type()
            i1 = ScalarType("i1")
            return [TensorType(ty.shape, i1, ty.placement) if isinstance(ty, TensorType) else i1]
        if n == "arith.select":
            op.operands = [self.ssa_use()]
            for _ in range(2):
                self.expect(",")
                op.operands.append(self.ssa_use())
            self.expect(":")
            ty = self.type()
            if self.accept(","):
                ty = self.type()
            return [ty]
        if n == "tensor.empty":
            self.expect("(")
            self.expect(")")
            self.expect(":")
            return [self.type()]
        if n == "linalg.broadcast":
            if not self.keyword("ins"):
                raise self.error("expected 'ins'")
            self.expect("(")
            op.operands = [self.ssa_use()]
            self.expect(":")
            self.type()
            self.expect(")")
            if not self.keyword("outs"):
                raise self.error("expected 'outs'")
            self.expect("(")
            op.operands.append(self.ssa_use())
            self.expect(":")
            out_ty = self.type()
            self.expect(")")
            if not self.keyword("dimensions"):
                raise self.error("expected 'dimensions'")
            self.expect("=")
            op.attributes["dimensions"] = self.attr_value()
            return [out_ty]
        if n == "htile.hello":
            op.attributes.update(self.attr_dict())
            return []
        if n in ("htile.load", "htile.gather_nd"):
            op.operands = [self.ssa_use()]
            self.expect("[")
            op.operands += self.ssa_use_list("]")
            op.attributes.update(self.attr_dict())
            self.expect(":")
            self.type()
            while self.accept(","):
                self.type()
            self.expect("->")
            return [self.type()]
        if n == "htile.store":
            op.operands = [self.ssa_use()]
            self.expect(",")
            op.operands.append(self.ssa_use())
            self.expect("[")
            op.operands += self.ssa_use_list("]")
            op.attributes.update(self.attr_dict())
            self.expect(":")
            self.type()
            self.expect(",")
            self.type()
            return []
        if n == "htile.dot":
            op.operands = [self.ssa_use()]
            self.expect(",")
            op.operands.append(self.ssa_use())
            if self.accept(","):
                op.operands.append(self.ssa_use())
            op.attributes.update(self.attr_dict())
            policy = op.attributes.get("warp_policy")
            if policy is not None and policy not in ("square", "full_row", "full_col"):
                raise self.error(f"htile.dot: invalid warp_policy {policy!r}")  # HTileOps.td:11-19
            self.expect(":")
            for _ in op.operands:
                self.type()
                self.accept(",")
            self.expect("->")
            return [self.type()]
        if n == "htile.reduce":
            op.operands = [self.ssa_use()]
            if not self.keyword("axis"):
                raise self.error("expected 'axis'")
            op.attributes["axis"] = self.attr_value()
            if not self.keyword("kind"):
                raise self.error("expected 'kind'")
            op.attributes["kind"] = self.attr_value()
            op.attributes.update(self.attr_dict())
            return self._arrow_types()
        if n in ("htile.full", "htile.copy"):
            op.operands = [self.ssa_use()]
            op.attributes.update(self.attr_dict())
            return self._arrow_types()
        if n in ("htile.permute", "htile.unsqueeze"):
            op.operands = [self.ssa_use()]
            key = "permutation" if n == "htile.permute" else "mask"
            if not self.keyword(key):
                raise self.error(f"expected '{key}'")
            op.attributes[key] = self.attr_value()
            op.attributes.update(self.attr_dict())
            return self._arrow_types()
        if n == "htile.arange":
            op.operands = [self.ssa_use()]
            if not self.keyword("to"):
                raise self.error("expected 'to'")
            op.operands.append(self.ssa_use())
            op.attributes.update(self.attr_dict())
            self.expect(":")
            return [self.type()]
        if n == "scf.yield":
            if self.peek("%"):
                while True:
                    op.operands.append(self.ssa_use())
                    if not self.accept(","):
                        break
                self.expect(":")
                for i in range(len(op.operands)):
                    self.type()
                    if i + 1 < len(op.operands):
                        self.expect(",")
            return []
        if n == "scf.for":
            return self._scf_for(op)
        if n == "gpu.launch":
            return self._gpu_launch(op)
        raise self.error(f"unsupported operation '{n}'")

    def attr_value_no_type(self):
        m = self.match(_NUM_RE)
        if m:
            txt = m.group(0)
            return int(txt, 0) if re.fullmatch(r"[-+]?(0x[0-9a-fA-F]+|\d+)", txt) else float(txt)
        if self.keyword("true"):
            return True
        if self.keyword("false"):
            return False
        raise self.error("expected a numeric constant")

    def _arrow_types(self) -> list:
        self.expect(":")
        self.type()
        self.expect("->")
        return [self.type()]

    def _scf_for(self, op: Op) -> list:
        iv = self.ssa_name()
        self.expect("=")
        lb = self.ssa_use()
        if not self.keyword("to"):
            raise self.error("expected 'to'")
        ub = self.ssa_use()
        if not self.keyword("step"):
            raise self.error("expected 'step'")
        step = self.ssa_use()
        op.operands = [lb, ub, step]
        body = Block(parent_op=op)
        iter_names: list[str] = []
        if self.keyword("iter_args"):
            self.expect("(")
            while True:
                iter_names.append(self.ssa_name())
                self.expect("=")
                op.operands.append(self.ssa_use())
                if self.accept(")"):
                    break
                self.expect(",")
        types: list = []
        if self.accept("->"):
            self.expect("(")
            while True:
                types.append(self.type())
                if self.accept(")"):
                    break
                self.expect(",")
        if len(types) != len(iter_names):
            raise self.error("scf.for: iter_args and result types differ in number")
        self.scopes.append({})
        body.arguments.append(self.define(Value(iv, ScalarType("index"), body, 0)))
        for i, (nm, ty) in enumerate(zip(iter_names, types)):
            body.arguments.append(self.define(Value(nm, ty, body, i + 1)))
        self.expect("{")
        self.block_body(body, "}")
        self.scopes.pop()
        op.regions = [body]
        op.attributes.update(self.attr_dict())
        return types

    def _gpu_launch(self, op: Op) -> list:
        body = Block(parent_op=op)
        self.scopes.append({})
        index = ScalarType("index")
        size_values: list[Value] = []
        for word in ("blocks", "threads"):
            if not self.keyword(word):
                raise self.error(f"expected '{word}'")
            self.expect("(")
            ids = []
            while True:
                ids.append(self.ssa_name())
                if self.accept(")"):
                    break
                self.expect(",")
            if not self.keyword("in"):
                raise self.error("expected 'in'")
            self.expect("(")
            sizes = []
            while True:
                sizes.append(self.ssa_name())
                self.expect("=")
                op.operands.append(self.ssa_use())
                if self.accept(")"):
                    break
                self.expect(",")
            if len(ids) != 3 or len(sizes) != 3:
                raise self.error("gpu.launch needs three ids and three sizes per level")
            for nm in ids:
                body.arguments.append(self.define(Value(nm, index, body, len(body.arguments))))
            size_values += [Value(nm, index, body) for nm in sizes]
        # block arguments: 3 block ids, 3 thread ids, then the 6 sizes (as in the upstream op)
        for v in size_values:
            v.index = len(body.arguments)
            body.arguments.append(self.define(v))
        self.expect("{")
        self.block_body(body, "}")
        self.scopes.pop()
        op.regions = [body]
        return []


def parse_module(text: str) -> Module:
    """Parse HTile program text into a Module; raises HTileSyntaxError on anything unknown."""
    return _Parser(text).module()


def parse_file(path) -> Module:
    with open(path, "r", encoding="utf-8") as f:
        return parse_module(f.read())


def parse_type(text: str):
    return _Parser(text).type()


# ---------------------------------------------------------------------------------------------
# printer (custom assembly, values renumbered %0, %1, ... in definition order)
# ---------------------------------------------------------------------------------------------

def _fmt_attr(v) -> str:
    if v is True:
        return "unit"
    if isinstance(v, str):
        return f'"{v}"'
    if isinstance(v, list):
        return "array<i64: " + ", ".join(str(int(x)) for x in v) + ">"
    return repr(v)


def _fmt_attr_dict(attrs: dict, skip=()) -> str:
    items = []
    for k, v in attrs.items():
        if k in skip:
            continue
        items.append(k if v is True else f"{k} = {_fmt_attr(v)}")
    return " {" + ", ".join(items) + "}" if items else ""


def print_module(module: Module) -> str:
    """Render a Module back to custom assembly (used by the pass tests and for debugging)."""
    names: dict[int, str] = {}
    counter = [0]
    lines: list[str] = ["module {"]

    def nm(v: Value) -> str:
        return "%" + names[id(v)]

    def fresh(v: Value, fixed: str | None = None) -> str:
        if fixed is None:
            fixed = str(counter[0])
            counter[0] += 1
        names[id(v)] = fixed
        return "%" + fixed

    def emit_block(block: Block, indent: str) -> None:
        for op in block.operations:
            emit_op(op, indent)

    def emit_op(op: Op, ind: str) -> None:
        n, a = op.name, op.attributes
        ops = [nm(v) for v in op.operands]
        if n == "arith.constant":
            lines.append(f"{ind}{fresh(op.result)} = arith.constant {a['value']!r} : {op.result.type}")
            return
        if n == "scf.for":
            body = op.regions[0]
            res = ", ".join(fresh(r) for r in op.results)
            iv = fresh(body.arguments[0])
            iters = ", ".join(f"{fresh(arg)} = {nm(init)}" for arg, init in zip(body.arguments[1:], op.operands[3:]))
            head = f"{ind}{res + ' = ' if res else ''}scf.for {iv} = {ops[0]} to {ops[1]} step {ops[2]}"
            if iters:
                head += f" iter_args({iters}) -> (" + ", ".join(str(r.type) for r in op.results) + ")"
            lines.append(head + " {")
            emit_block(body, ind + "  ")
            lines.append(f"{ind}}}" + _fmt_attr_dict(a))
            return
        if n == "gpu.launch":
            body = op.regions[0]
            ids = [fresh(v) for v in body.arguments[:6]]
            szs = [fresh(v) for v in body.arguments[6:]]
            lines.append(
                f"{ind}gpu.launch blocks({', '.join(ids[:3])}) in ("
                + ", ".join(f"{s} = {o}" for s, o in zip(szs[:3], ops[:3])) + ") threads("
                + ", ".join(ids[3:]) + ") in (" + ", ".join(f"{s} = {o}" for s, o in zip(szs[3:], ops[3:])) + ") {")
            emit_block(body, ind + "  ")
            lines.append(f"{ind}}}")
            return
        res = ", ".join(fresh(r) for r in op.results)
        lhs = f"{ind}{res} = " if res else ind
        tys = [str(v.type) for v in op.operands]
        if n in ("htile.load", "htile.gather_nd"):
            lines.append(f"{lhs}{n} {ops[0]}[{', '.join(ops[1:])}]{_fmt_attr_dict(a)} : {tys[0]} -> {op.result.type}")
        elif n == "htile.store":
            lines.append(f"{lhs}{n} {ops[0]}, {ops[1]}[{', '.join(ops[2:])}]{_fmt_attr_dict(a)} : {tys[0]}, {tys[1]}")
        elif n == "htile.dot":
            lines.append(f"{lhs}{n} {', '.join(ops)}{_fmt_attr_dict(a)} : {', '.join(tys)} -> {op.result.type}")
        elif n == "htile.reduce":
            lines.append(f"{lhs}{n} {ops[0]} axis {a['axis']} kind \"{a['kind']}\"{_fmt_attr_dict(a, ('axis', 'kind'))}"
                         f" : {tys[0]} -> {op.result.type}")
        elif n in ("htile.permute", "htile.unsqueeze"):
            key = "permutation" if n == "htile.permute" else "mask"
            items = ", ".join(("true" if x else "false") if isinstance(x, bool) else str(x) for x in a[key])
            lines.append(f"{lhs}{n} {ops[0]} {key} [{items}]{_fmt_attr_dict(a, (key,))} : {tys[0]} -> {op.result.type}")
        elif n in ("htile.full", "htile.copy"):
            lines.append(f"{lhs}{n} {ops[0]}{_fmt_attr_dict(a)} : {tys[0]} -> {op.result.type}")
        elif n == "htile.arange":
            lines.append(f"{lhs}{n} {ops[0]} to {ops[1]} : {op.result.type}")
        elif n == "tensor.empty":
            lines.append(f"{lhs}tensor.empty() : {op.result.type}")
        elif n == "linalg.broadcast":
            lines.append(f"{lhs}linalg.broadcast ins({ops[0]} : {tys[0]}) outs({ops[1]} : {tys[1]}) "
                         f"dimensions = {a['dimensions']}")
        elif n in _CASTS:
            lines.append(f"{lhs}{n} {ops[0]} : {tys[0]} to {op.result.type}")
        elif n in ("arith.cmpi", "arith.cmpf"):
            lines.append(f"{lhs}{n} {a['predicate']}, {ops[0]}, {ops[1]} : {tys[0]}")
        elif n == "scf.yield":
            lines.append(f"{lhs}scf.yield {', '.join(ops)}" + (" : " + ", ".join(tys) if ops else ""))
        elif n in ("return", "func.return", "gpu.terminator", "htile.hello"):
            lines.append(f"{lhs}{n}{_fmt_attr_dict(a)}")
        else:  # elementwise arith / math / select
            ty = op.result.type if op.results else ""
            lines.append(f"{lhs}{n} {', '.join(ops)}{_fmt_attr_dict(a)} : {ty}")

    for fn in module.functions:
        counter[0] = 0
        args = ", ".join(f"{fresh(arg, f'arg{i}')}: {arg.type}" for i, arg in enumerate(fn.arguments))
        attrs = " attributes" + _fmt_attr_dict(fn.attributes) if fn.attributes else ""
        lines.append(f"  func.func @{fn.name}({args}){attrs} {{")
        emit_block(fn.body, "    ")
        lines.append("  }")
    lines.append("}")
    return "\n".join(lines) + "\n"
