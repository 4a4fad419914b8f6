"""Lowering of a Level-1 ("scheduled tile IR") attention program to HTile text.

Level 1 is the reference project's target-independent tile form (docs/tile-ir-level1.md:8-14 of the
reference): plain tensors, ``scf.forall`` for the grid of disjoint output tiles, ``affine.for`` (or
``scf.for``) with ``iter_args`` for the streamed reduction, ``tensor.extract_slice`` /
``tensor.parallel_insert_slice`` for tiles, and ``linalg`` / ``arith`` / ``math`` tile bodies; no GPU
hierarchy, no placements.  Its canonical example is tests/data/flash_attention_l1.mlir:1-161 of the
reference.  The reference has no pass from that level to its HTile dialect (the HTile program
tests/data/flash_attention_htile.mlir was written by hand); this module is that step, so that tile sizes
and shapes come from the scheduled program instead of hand-edited constants:

    scf.forall (%b, %h, %i) in (B, H, GM)      -> gpu.launch blocks (GM, H, B), threads (tile rows, 1, 1)
    tensor.extract_slice (rank-reducing)       -> htile.load  ... -> tensor<.., #shared>
    linalg.fill of a tensor.empty              -> htile.full  (dropped when it only seeds a matmul: htile.dot
                                                  without an accumulator starts from zero)
    affine.for / scf.for + iter_args           -> scf.for with index constants, htile.pipeline_stages kept
    affine.apply (d) -> (d * c)                -> arith.muli
    linalg.matmul (indexing maps n,k on B)     -> htile.dot {transpose_b}        (plain maps: htile.dot)
    linalg.map { mulf by a scalar }            -> htile.full + arith.mulf
    linalg.reduce { maximumf | addf } dims [1] -> htile.reduce axis 1 kind "max" | "sum"
    linalg.broadcast, arith.*, math.exp2, arith.truncf on tiles carry over, results placed #local
    tensor.parallel_insert_slice               -> htile.store

Placement policy (the one decision Level 1 leaves open, docs/tile-ir-level1.md:120-131): tiles read from a
function argument are ``#shared``, every computed tile is ``#local`` -- what the reference's hand-written HTile
program does.  The reader below accepts the subset of upstream MLIR assembly that such programs use and raises
``L1SyntaxError`` / ``NotImplementedError`` on anything else.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field


class L1SyntaxError(ValueError):
    pass


# ---------------------------------------------------------------------------------------------- tokens
_TOKEN = re.compile(r"""
    (?P<ws>\s+|//[^\n]*)
  | (?P<type>(?:tensor|memref)<[^<>]*>)
  | (?P<ssa>%[A-Za-z0-9_$.\-]+)
  | (?P<sym>@[A-Za-z0-9_$.]+)
  | (?P<num>-?(?:\d+\.\d*(?:[eE][-+]?\d+)?|\d+[eE][-+]?\d+|\d+))
  | (?P<arrow>->)
  | (?P<word>[A-Za-z_][A-Za-z0-9_.]*)
  | (?P<punct>[(){}\[\]<>,:=*+])
""", re.X)


def _tokenize(text: str) -> list[tuple[str, str]]:
    out, pos = [], 0
    while pos < len(text):
        if text.startswith("affine_map<", pos):            # one token, up to the matching '>' ("->" is not a bracket)
            depth, i = 0, pos + len("affine_map")
            while i < len(text):
                if text.startswith("->", i):
                    i += 2
                    continue
                if text[i] == "<":
                    depth += 1
                elif text[i] == ">":
                    depth -= 1
                    if depth == 0:
                        break
                i += 1
            out.append(("map", text[pos:i + 1]))
            pos = i + 1
            continue
        m = _TOKEN.match(text, pos)
        if not m:
            line = text.count("\n", 0, pos) + 1
            raise L1SyntaxError(f"line {line}: unexpected character {text[pos]!r}")
        if m.lastgroup != "ws":
            out.append((m.lastgroup, m.group()))
        pos = m.end()
    return out


@dataclass
class Op:
    name: str
    results: list[str] = field(default_factory=list)
    operands: list = field(default_factory=list)          # SSA names or literals
    types: list[str] = field(default_factory=list)        # as written
    attrs: dict = field(default_factory=dict)
    regions: list[list["Op"]] = field(default_factory=list)


@dataclass
class Func:
    name: str
    args: list[tuple[str, str]]
    result_type: str
    body: list[Op]


def _shape(ty: str) -> tuple[tuple[int, ...], str]:
    m = re.fullmatch(r"(?:tensor|memref)<([^<>]*)>", ty)
    if not m:
        raise L1SyntaxError(f"not a shaped type: {ty}")
    parts = m.group(1).split("x")
    return tuple(int(p) for p in parts[:-1]), parts[-1].strip()


class _Parser:
    def __init__(self, text: str):
        self.toks = _tokenize(text)
        self.i = 0

    # -- primitives
    def peek(self, value: str | None = None, kind: str | None = None, ahead: int = 0) -> bool:
        if self.i + ahead >= len(self.toks):
            return False
        k, v = self.toks[self.i + ahead]
        return (value is None or v == value) and (kind is None or k == kind)

    def next(self) -> tuple[str, str]:
        if self.i >= len(self.toks):
            raise L1SyntaxError("unexpected end of input")
        tok = self.toks[self.i]
        self.i += 1
        return tok

    def expect(self, value: str) -> None:
        k, v = self.next()
        if v != value:
            raise L1SyntaxError(f"expected {value!r}, found {v!r}")

    def accept(self, value: str) -> bool:
        if self.peek(value):
            self.i += 1
            return True
        return False

    def kind(self, kind: str) -> str:
        k, v = self.next()
        if k != kind:
            raise L1SyntaxError(f"expected a {kind}, found {v!r}")
        return v

    def operand(self):
        k, v = self.next()
        if k == "ssa":
            return v
        if k == "num":
            return float(v) if any(c in v for c in ".eE") else int(v)
        raise L1SyntaxError(f"expected an operand, found {v!r}")

    def list_of(self, open_: str, close: str, item) -> list:
        self.expect(open_)
        items = []
        while not self.peek(close):
            items.append(item())
            if not self.accept(","):
                break
        self.expect(close)
        return items

    def type_(self) -> str:
        k, v = self.next()
        if k in ("type", "word"):
            return v
        raise L1SyntaxError(f"expected a type, found {v!r}")

    def attr_dict(self) -> dict:
        attrs = {}
        self.expect("{")
        while not self.peek("}"):
            key = self.kind("word")
            self.expect("=")
            val = self.operand()
            if self.accept(":"):
                self.type_()
            attrs[key] = val
            if not self.accept(","):
                break
        self.expect("}")
        return attrs

    # -- structure
    def module(self) -> Func:
        if self.accept("module"):
            self.expect("{")
            fn = self.func()
            self.expect("}")
        else:
            fn = self.func()
        if self.i != len(self.toks):
            raise L1SyntaxError(f"trailing input at {self.toks[self.i][1]!r}")
        return fn

    def func(self) -> Func:
        self.expect("func.func")
        name = self.kind("sym")[1:]
        args = self.list_of("(", ")", lambda: (self.kind("ssa"), (self.expect(":"), self.type_())[1]))
        self.expect("->")
        rtype = self.type_()
        self.expect("{")
        body = self.block(("return", "func.return"))
        self.expect("}")
        return Func(name, args, rtype, body)

    def block(self, terminators: tuple[str, ...]) -> list[Op]:
        ops = []
        while True:
            op = self.operation()
            ops.append(op)
            if op.name in terminators:
                return ops

    def operation(self) -> Op:
        results = []
        if self.peek(kind="ssa"):
            results.append(self.kind("ssa"))
            while self.accept(","):
                results.append(self.kind("ssa"))
            self.expect("=")
        name = self.kind("word")
        op = Op(name, results)
        handler = getattr(self, "_op_" + name.replace(".", "_"), None)
        if handler is None:
            raise NotImplementedError(f"Level-1 reader: operation '{name}' is not supported")
        handler(op)
        return op

    # -- operations
    def _op_return(self, op):
        op.operands = [self.operand()]
        self.expect(":")
        op.types = [self.type_()]

    _op_func_return = _op_return

    def _op_arith_constant(self, op):
        op.attrs["value"] = self.operand()
        self.expect(":")
        op.types = [self.type_()]

    def _op_tensor_empty(self, op):
        self.expect("(")
        self.expect(")")
        self.expect(":")
        op.types = [self.type_()]

    def _binary(self, op):
        op.operands = [self.operand()]
        self.expect(",")
        op.operands.append(self.operand())
        self.expect(":")
        op.types = [self.type_()]

    _op_arith_muli = _op_arith_addi = _op_arith_maximumf = _op_arith_subf = _op_arith_mulf = _binary
    _op_arith_addf = _op_arith_divf = _binary

    def _op_math_exp2(self, op):
        op.operands = [self.operand()]
        self.expect(":")
        op.types = [self.type_()]

    def _op_arith_truncf(self, op):
        op.operands = [self.operand()]
        self.expect(":")
        src = self.type_()
        self.expect("to")
        op.types = [src, self.type_()]

    def _ins_outs(self, op):
        self.expect("ins")
        self.expect("(")
        ins = [self.operand()]
        while self.accept(","):
            ins.append(self.operand())
        self.expect(":")
        in_types = [self.type_()]
        while self.accept(","):
            in_types.append(self.type_())
        self.expect(")")
        self.expect("outs")
        self.expect("(")
        out = self.operand()
        self.expect(":")
        out_type = self.type_()
        self.expect(")")
        op.operands = ins + [out]
        op.types = in_types + [out_type]

    def _op_linalg_fill(self, op):
        self._ins_outs(op)
        self.expect("->")
        self.type_()

    def _op_linalg_matmul(self, op):
        if self.accept("indexing_maps"):
            self.expect("=")
            op.attrs["indexing_maps"] = self.list_of("[", "]", lambda: self.kind("map"))
        self._ins_outs(op)
        self.expect("->")
        self.type_()

    def _op_linalg_broadcast(self, op):
        self._ins_outs(op)
        self.expect("dimensions")
        self.expect("=")
        op.attrs["dimensions"] = self.list_of("[", "]", self.operand)

    def _op_linalg_reduce(self, op):
        self.expect("{")
        op.attrs["combiner"] = self.kind("word")
        self.expect("}")
        self._ins_outs(op)
        self.expect("dimensions")
        self.expect("=")
        op.attrs["dimensions"] = self.list_of("[", "]", self.operand)

    def _op_linalg_map(self, op):
        self._ins_outs(op)
        params = self.list_of("(", ")", lambda: (self.kind("ssa"), (self.expect(":"), self.type_())[1]))
        op.attrs["params"] = params
        self.expect("{")
        op.regions = [self.block(("linalg.yield",))]
        self.expect("}")

    def _op_linalg_yield(self, op):
        op.operands = [self.operand()]
        self.expect(":")
        op.types = [self.type_()]

    def _op_tensor_extract_slice(self, op):
        op.operands = [self.kind("ssa")]
        op.attrs["offsets"] = self.list_of("[", "]", self.operand)
        op.attrs["sizes"] = self.list_of("[", "]", self.operand)
        op.attrs["strides"] = self.list_of("[", "]", self.operand)
        self.expect(":")
        src = self.type_()
        self.expect("to")
        op.types = [src, self.type_()]

    def _op_tensor_parallel_insert_slice(self, op):
        op.operands = [self.kind("ssa")]
        self.expect("into")
        op.operands.append(self.kind("ssa"))
        op.attrs["offsets"] = self.list_of("[", "]", self.operand)
        op.attrs["sizes"] = self.list_of("[", "]", self.operand)
        op.attrs["strides"] = self.list_of("[", "]", self.operand)
        self.expect(":")
        src = self.type_()
        self.expect("into")
        op.types = [src, self.type_()]

    def _op_affine_apply(self, op):
        op.attrs["map"] = self.kind("map")
        op.operands = self.list_of("(", ")", self.operand)

    def _loop(self, op, yield_name: str):
        op.attrs["iv"] = self.kind("ssa")
        self.expect("=")
        op.attrs["lb"] = self.operand()
        self.expect("to")
        op.attrs["ub"] = self.operand()
        op.attrs["step"] = self.operand() if self.accept("step") else 1
        self.expect("iter_args")
        pairs = self.list_of("(", ")", lambda: (self.kind("ssa"), (self.expect("="), self.operand())[1]))
        op.attrs["iter_args"] = [p[0] for p in pairs]
        op.operands = [p[1] for p in pairs]
        self.expect("->")
        op.types = self.list_of("(", ")", self.type_) if self.peek("(") else [self.type_()]
        self.expect("{")
        op.regions = [self.block((yield_name,))]
        self.expect("}")
        if self.peek("{"):
            op.attrs["loop_attrs"] = self.attr_dict()

    def _op_affine_for(self, op):
        self._loop(op, "affine.yield")

    def _op_scf_for(self, op):
        self._loop(op, "scf.yield")

    def _yield(self, op):
        op.operands = [self.operand()]
        while self.accept(","):
            op.operands.append(self.operand())
        self.expect(":")
        op.types = [self.type_()]
        while self.accept(","):
            op.types.append(self.type_())

    _op_affine_yield = _op_scf_yield = _yield

    def _op_scf_forall(self, op):
        op.attrs["ivs"] = self.list_of("(", ")", lambda: self.kind("ssa"))
        self.expect("in")
        op.attrs["bounds"] = self.list_of("(", ")", self.operand)
        self.expect("shared_outs")
        pairs = self.list_of("(", ")", lambda: (self.kind("ssa"), (self.expect("="), self.operand())[1]))
        op.attrs["outs"] = [p[0] for p in pairs]
        op.operands = [p[1] for p in pairs]
        self.expect("->")
        op.types = [self.type_()]
        self.expect("{")
        op.regions = [self.block(("scf.forall.in_parallel",))]
        self.expect("}")

    def _op_scf_forall_in_parallel(self, op):
        self.expect("{")
        op.regions = [[self.operation()]]
        self.expect("}")


def parse(text: str) -> Func:
    """Read one Level-1 function (optionally wrapped in ``module { }``)."""
    return _Parser(text).module()


# ---------------------------------------------------------------------------------------------- lowering
class _Emitter:
    def __init__(self, fn: Func):
        self.fn = fn
        self.lines: list[str] = []
        self.names: dict[str, str] = {}          # L1 SSA name -> HTile SSA name
        self.types: dict[str, str] = {}          # HTile SSA name -> type text
        self.defs: dict[str, Op] = {}            # L1 SSA name -> defining op
        self.consts: dict = {}                   # (value, type) -> HTile SSA name of a hoisted constant
        self.const_lines: list[str] = []
        self.counter = 0

    def fresh(self, hint: str) -> str:
        self.counter += 1
        return f"%{hint}_{self.counter}"

    def const(self, value, ty: str) -> str:
        key = (value, ty)
        if key not in self.consts:
            name = f"%c{len(self.consts)}"
            text = repr(float(value)) if ty == "f32" else str(int(value))
            self.const_lines.append(f"    {name} = arith.constant {text} : {ty}")
            self.consts[key] = name
        return self.consts[key]

    def index(self, v) -> str:
        """An index operand: an SSA value already lowered, or a literal hoisted as a constant."""
        return self.names[v] if isinstance(v, str) else self.const(v, "index")

    @staticmethod
    def tile(ty: str, placement: str) -> str:
        shape, elem = _shape(ty)
        return f"tensor<{'x'.join(map(str, shape))}x{elem}, #{placement}>"

    def emit(self, indent: int, text: str) -> None:
        self.lines.append("  " * indent + text)

    def bind(self, l1_name: str, ht_name: str, ty: str) -> str:
        self.names[l1_name] = ht_name
        self.types[ht_name] = ty
        return ht_name


def lower_to_htile(source: str | Func) -> str:
    """HTile text for a Level-1 attention-style program (text or a parsed function)."""
    fn = parse(source) if isinstance(source, str) else source
    e = _Emitter(fn)
    need = _need(fn.name)

    # ---- function level: constants, the output's tensor.empty, one scf.forall, return of its result
    foralls = [op for op in fn.body if op.name == "scf.forall"]
    need(len(foralls) == 1, "exactly one scf.forall (the grid of output tiles)")
    forall = foralls[0]
    scalars: dict[str, tuple] = {}
    for op in fn.body:
        if op.name == "arith.constant":
            scalars[op.results[0]] = (op.attrs["value"], op.types[0])
        elif op.name == "tensor.empty":
            e.defs[op.results[0]] = op
        elif op.name not in ("scf.forall", "return", "func.return"):
            raise NotImplementedError(f"@{fn.name}: '{op.name}' outside the scf.forall is not supported")
    ret = fn.body[-1]
    need(ret.operands == forall.results, "the function returns the scf.forall result")
    need(len(forall.operands) == 1 and forall.operands[0] in e.defs, "shared_outs starts from a tensor.empty")
    out_type = forall.types[0]
    need(out_type == fn.result_type, "the forall produces the function's result type")

    # memref arguments: the tensors, then the result as an output argument
    def memref(ty: str) -> str:
        shape, elem = _shape(ty)
        return f"memref<{'x'.join(map(str, shape))}x{elem}>"

    args = []
    for name, ty in fn.args:
        e.bind(name, name, memref(ty))
        args.append(f"{name}: {memref(ty)}")
    out_name = "%out"
    e.bind(forall.attrs["outs"][0], out_name, memref(out_type))
    args.append(f"{out_name}: {memref(out_type)}")

    for name, (value, ty) in scalars.items():
        e.bind(name, e.const(value, ty), ty)

    ivs, bounds = forall.attrs["ivs"], forall.attrs["bounds"]
    need(len(ivs) == 3 and all(isinstance(b, int) for b in bounds), "scf.forall over three static extents (batch, head, row block)")
    # the innermost forall index walks output row blocks: it becomes the x block id, as in the reference's HTile program
    e.bind(ivs[2], "%bx", "index")
    e.bind(ivs[1], "%by", "index")
    e.bind(ivs[0], "%bz", "index")

    body = forall.regions[0]
    insert = body[-1].regions[0][0]
    need(insert.name == "tensor.parallel_insert_slice", "the forall publishes its tile with tensor.parallel_insert_slice")
    tile_rows = insert.attrs["sizes"][-2]
    _lower_block(e, body[:-1], 3, scalars)
    # ---- publish the tile
    need(insert.operands[1] == forall.attrs["outs"][0], "the tile is inserted into the shared output")
    offs = ", ".join(e.index(o) for o in insert.attrs["offsets"])
    val = e.names[insert.operands[0]]
    e.emit(3, f"htile.store {val}, {out_name}[{offs}] : {e.types[val]}, {memref(out_type)}")
    e.emit(3, "gpu.terminator")

    one = e.const(1, "index")
    gx, gy, gz = (e.const(b, "index") for b in (bounds[2], bounds[1], bounds[0]))
    tx = e.const(tile_rows, "index")
    head = [
        "#shared = #htile.encoding<placement = shared>",
        "#local = #htile.encoding<placement = local>",
        "",
        "module {",
        f"  func.func @{fn.name}({', '.join(args)}) {{",
        *e.const_lines,
        f"    gpu.launch blocks(%bx, %by, %bz) in (%gx = {gx}, %gy = {gy}, %gz = {gz})",
        f"               threads(%tx, %ty, %tz) in (%sx = {tx}, %sy = {one}, %sz = {one}) {{",
    ]
    tail = ["    }", "    return", "  }", "}"]
    return "\n".join(head + e.lines + tail) + "\n"


def _need(fn_name: str):
    def need(cond: bool, what: str) -> None:
        if not cond:
            raise NotImplementedError(f"@{fn_name}: Level-1 lowering expects {what}")
    return need


_ELEMENTWISE = {"arith.maximumf", "arith.subf", "arith.mulf", "arith.addf", "arith.divf"}


def _lower_block(e: _Emitter, ops: list[Op], ind: int, scalars: dict) -> None:
    need = _need(e.fn.name)
    for op in ops:
        r = op.results[0] if op.results else None
        if op.name == "tensor.empty":
            e.defs[r] = op
        elif op.name == "arith.constant":
            scalars[r] = (op.attrs["value"], op.types[0])
            e.bind(r, e.const(op.attrs["value"], op.types[0]), op.types[0])
        elif op.name in ("arith.muli", "arith.addi"):
            a, b = (e.index(o) for o in op.operands)
            e.emit(ind, f"{e.bind(r, e.fresh('i'), 'index')} = {op.name} {a}, {b} : index")
        elif op.name == "affine.apply":
            m = re.fullmatch(r"affine_map<\((\w+)\)\s*->\s*\(\1\s*\*\s*(\d+)\)>", op.attrs["map"])
            need(m is not None and len(op.operands) == 1, f"affine.apply of (d) -> (d * c), got {op.attrs['map']}")
            e.emit(ind, f"{e.bind(r, e.fresh('i'), 'index')} = arith.muli {e.index(op.operands[0])}, {e.const(int(m.group(2)), 'index')} : index")
        elif op.name == "tensor.extract_slice":
            src = op.operands[0]
            need(src in e.names and e.types[e.names[src]].startswith("memref"), "tiles are sliced from function arguments")
            src_shape, _ = _shape(op.types[0])
            dst_shape, _ = _shape(op.types[1])
            sizes = op.attrs["sizes"]
            need(all(s == 1 for s in op.attrs["strides"]) and tuple(sizes[len(sizes) - len(dst_shape):]) == dst_shape
                 and all(s == 1 for s in sizes[:len(sizes) - len(dst_shape)]), "unit-stride, rank-reducing tile slices")
            ty = e.tile(op.types[1], "shared")
            offs = ", ".join(e.index(o) for o in op.attrs["offsets"])
            e.emit(ind, f"{e.bind(r, e.fresh('tile'), ty)} = htile.load {e.names[src]}[{offs}] : {e.types[e.names[src]]} -> {ty}")
        elif op.name == "linalg.fill":
            e.defs[r] = op                                    # materialised on first use as a value (see _value)
        elif op.name == "linalg.matmul":
            a, b, acc = op.operands
            need(acc in e.defs and e.defs[acc].name == "linalg.fill" and _fill_value(e, e.defs[acc], scalars) == 0.0,
                 "matmul accumulating into a zero fill")
            maps = op.attrs.get("indexing_maps")
            transpose_b = False
            if maps is not None:
                norm = [re.sub(r"\s+", "", m) for m in maps]
                need(len(norm) == 3 and norm[0].endswith("->(m,k)>") and norm[2].endswith("->(m,n)>"), "matmul maps (m,k), B, (m,n)")
                transpose_b = norm[1].endswith("->(n,k)>")
                need(transpose_b or norm[1].endswith("->(k,n)>"), "B indexed (k,n) or (n,k)")
            ty = e.tile(op.types[2], "local")
            attrs = "{transpose_b, warp_policy = \"full_row\"}" if transpose_b else "{warp_policy = \"full_row\"}"
            va, vb = _value(e, a, ind, scalars), _value(e, b, ind, scalars)
            e.emit(ind, f"{e.bind(r, e.fresh('dot'), ty)} = htile.dot {va}, {vb} {attrs} : {e.types[va]}, {e.types[vb]} -> {ty}")
        elif op.name == "linalg.map":
            inner = op.regions[0]
            need(len(inner) == 2 and inner[0].name == "arith.mulf" and inner[1].operands == inner[0].results,
                 "linalg.map whose body multiplies by a scalar")
            param = op.attrs["params"][0][0]
            other = [o for o in inner[0].operands if o != param]
            need(len(other) == 1 and other[0] in scalars, "the multiplier is a scalar constant")
            ty = e.tile(op.types[0], "local")
            c = e.fresh("scale")
            e.types[c] = ty
            e.emit(ind, f"{c} = htile.full {e.const(*scalars[other[0]])} : f32 -> {ty}")
            x = _value(e, op.operands[0], ind, scalars)
            e.emit(ind, f"{e.bind(r, e.fresh('t'), ty)} = arith.mulf {x}, {c} : {ty}")
        elif op.name == "linalg.reduce":
            kinds = {"arith.maximumf": "max", "arith.addf": "sum"}
            need(op.attrs["combiner"] in kinds and len(op.attrs["dimensions"]) == 1, "row maximum or row sum over one axis")
            seed = op.operands[1]
            need(seed in e.defs and e.defs[seed].name == "linalg.fill", "reduction seeded by a fill")
            ty = e.tile(op.types[1], "local")
            x = _value(e, op.operands[0], ind, scalars)
            e.emit(ind, f"{e.bind(r, e.fresh('red'), ty)} = htile.reduce {x} axis {op.attrs['dimensions'][0]} kind \"{kinds[op.attrs['combiner']]}\" : {e.types[x]} -> {ty}")
        elif op.name == "linalg.broadcast":
            ty = e.tile(op.types[1], "local")
            x = _value(e, op.operands[0], ind, scalars)
            empty = e.fresh("e")
            e.emit(ind, f"{empty} = tensor.empty() : {ty}")
            dims = ", ".join(str(d) for d in op.attrs["dimensions"])
            e.emit(ind, f"{e.bind(r, e.fresh('bc'), ty)} = linalg.broadcast ins({x} : {e.types[x]}) outs({empty} : {ty}) dimensions = [{dims}]")
        elif op.name in _ELEMENTWISE:
            ty = e.tile(op.types[0], "local")
            a, b = (_value(e, o, ind, scalars) for o in op.operands)
            e.emit(ind, f"{e.bind(r, e.fresh('t'), ty)} = {op.name} {a}, {b} : {ty}")
        elif op.name == "math.exp2":
            ty = e.tile(op.types[0], "local")
            e.emit(ind, f"{e.bind(r, e.fresh('t'), ty)} = math.exp2 {_value(e, op.operands[0], ind, scalars)} : {ty}")
        elif op.name == "arith.truncf":
            src, dst = e.tile(op.types[0], "local"), e.tile(op.types[1], "local")
            e.emit(ind, f"{e.bind(r, e.fresh('t'), dst)} = arith.truncf {_value(e, op.operands[0], ind, scalars)} : {src} to {dst}")
        elif op.name in ("affine.for", "scf.for"):
            lb, ub, step = (e.index(op.attrs[k]) for k in ("lb", "ub", "step"))
            inits = [_value(e, o, ind, scalars) for o in op.operands]
            tys = [e.tile(t, "local") for t in op.types]
            iv = e.bind(op.attrs["iv"], e.fresh("j"), "index")
            iters = []
            for name, init, ty in zip(op.attrs["iter_args"], inits, tys):
                iters.append(f"{e.bind(name, e.fresh('it'), ty)} = {init}")
            outs = [e.bind(res, e.fresh("out"), ty) for res, ty in zip(op.results, tys)]
            e.emit(ind, f"{', '.join(outs)} = scf.for {iv} = {lb} to {ub} step {step}")
            e.emit(ind + 2, f"iter_args({', '.join(iters)})")
            e.emit(ind + 2, f"-> ({', '.join(tys)}) {{")
            inner = op.regions[0]
            _lower_block(e, inner[:-1], ind + 1, scalars)
            ys = [_value(e, o, ind + 1, scalars) for o in inner[-1].operands]
            e.emit(ind + 1, f"scf.yield {', '.join(ys)} : {', '.join(tys)}")
            stages = op.attrs.get("loop_attrs", {}).get("pipeline_stages")
            e.emit(ind, "}" + (f" {{htile.pipeline_stages = {stages} : i32}}" if stages is not None else ""))
        else:
            raise NotImplementedError(f"@{e.fn.name}: Level-1 lowering has no rule for '{op.name}'")


def _fill_value(e: _Emitter, fill: Op, scalars: dict):
    src = fill.operands[0]
    return scalars[src][0] if src in scalars else None


def _value(e: _Emitter, name: str, ind: int, scalars: dict) -> str:
    """The HTile value for an L1 value used as a tile operand; a linalg.fill becomes an htile.full at first use."""
    if name in e.names:
        return e.names[name]
    op = e.defs.get(name)
    if op is not None and op.name == "linalg.fill":
        value = _fill_value(e, op, scalars)
        if value is None:
            raise NotImplementedError(f"@{e.fn.name}: linalg.fill of a non-constant")
        ty = e.tile(op.types[1], "local")
        e.emit(ind, f"{e.bind(name, e.fresh('full'), ty)} = htile.full {e.const(value, 'f32')} : f32 -> {ty}")
        return e.names[name]
    raise NotImplementedError(f"@{e.fn.name}: value {name} has no HTile counterpart")


def lower_file(path) -> str:
    from pathlib import Path

    return lower_to_htile(Path(path).read_text())


def translate_file(path, plugin: str | None = None):
    """Level-1 file -> HTile text -> the B200 translator's ``ast.Module`` (the same pipeline as
    ``neptune_mlir.translators.b200.translate_file`` with the lowering in front)."""
    import os
    import tempfile

    from .translators import b200

    with tempfile.NamedTemporaryFile("w", suffix=".mlir", delete=False) as f:
        f.write(lower_file(path))
    try:
        return b200.translate_file(f.name, plugin)
    finally:
        os.unlink(f.name)


def main() -> None:
    """``python -m neptune_mlir.l1 file.mlir [--translate]``: print the HTile text (or the emitted Python module)."""
    import argparse
    import ast

    ap = argparse.ArgumentParser(description="Lower a Level-1 tile program to HTile")
    ap.add_argument("path")
    ap.add_argument("--translate", action="store_true", help="also run the B200 translator and print its module")
    args = ap.parse_args()
    print(ast.unparse(translate_file(args.path)) if args.translate else lower_file(args.path), end="")


if __name__ == "__main__":
    main()
