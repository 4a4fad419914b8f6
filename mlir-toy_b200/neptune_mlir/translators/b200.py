#!/usr/bin/env python3
"""HTile MLIR -> B200 (sm_100a) kernel-library translator.

Usage:
    python -m neptune_mlir.translators.b200 <input.mlir> [--plugin <libnb200.so>]

Same surface as the reference's translators (src/neptune_mlir/translators/triton.py:36,63,479,490):
``Translator().translate(module) -> ast.Module``, ``translate_file(path, plugin=None)``, ``main()``.
The emitted module defines one Python function per ``func.func``, named by its symbol and taking
the memref arguments positionally as torch CUDA tensors, outputs written in place.

Where the reference's translators lower op by op into a tile DSL, this target maps a whole
function onto one hand-written kernel family.  It therefore *recognises* programs:

* the FlashAttention recurrence of tests/data/flash_attention_htile.mlir (any B, H, S, D, tile sizes,
  f16 / bf16 / f32, optional causal mask written with htile.arange + arith.cmpi + arith.select);
  the function's expression graph is compared with the recurrence, and shapes, scale constant and
  causality are read off it;
* split-K flash-decoding with its log-sum-exp combine spelled in HTile ops (two ``gpu.launch`` regions:
  the per-split online softmax of the grouped query heads, then the merge of the partials;
  ``neptune_mlir.programs.decode_splitk_htile`` writes it): both regions are compared with the operator's
  equations and B, Hq, Hkv, L, D, the split count and the scale are read off them;
* operator declarations: a ``func.func`` with attribute ``htile.operator`` naming one of
  ``decode_splitk``, ``selective_scan``, ``ssd_chunk_scan`` and an empty body; the memref
  argument types carry the problem sizes.  The dialect has no scan op
  (include/HTile/HTileOps.td:21-217), so these operators cannot be spelled op by op.

Anything else raises ``NotImplementedError`` -- nothing is skipped silently (the reference emits a
``'# TODO'`` string for unknown ops, triton.py:170-172).
"""

from __future__ import annotations

import ast
import math

from .. import htile_text as ht
from .common import (
    DEFAULT_LIBRARY,
    HTILE_DOT_TRANSPOSE_TO_LOAD_ORDER_PIPELINE,
    attr,
    call,
    const,
    function_def,
    name,
    reject_dot_transpose_attrs,
    translate_file_with,
)

_COMMUTATIVE = {"arith.addf", "arith.mulf", "arith.maximumf", "arith.addi", "arith.muli"}
_FLOAT_DTYPES = ("f16", "bf16", "f32")


def _unsupported(msg: str) -> NotImplementedError:
    return NotImplementedError(f"B200 translation: {msg}")


class _Graph:
    """Canonical expression trees of SSA values (commutative operands sorted, placements ignored)."""

    def __init__(self, func: ht.Func):
        self.func = func
        # block ids of the first gpu.launch are ("bid", i); those of launch k > 0 are ("bid", i, k)
        self._launch_no = {id(op): k for k, op in enumerate(o for o in func.body.operations if o.name == "gpu.launch")}
        self._memo: dict[int, tuple] = {}

    def of(self, v: ht.Value) -> tuple:
        key = id(v)
        if key not in self._memo:
            self._memo[key] = self._build(v)
        return self._memo[key]

    def _build(self, v: ht.Value) -> tuple:
        owner = v.owner
        if isinstance(owner, ht.Block):
            parent = owner.parent_op
            if parent is None:
                return ("arg", v.index)
            if parent.name == "gpu.launch":
                kinds = ("bid", "bid", "bid", "tid", "tid", "tid")
                which = self._launch_no.get(id(parent), 0)
                if v.index >= 6:
                    return ("launch_size", v.index - 6)
                return (kinds[v.index], v.index % 3) if which == 0 else (kinds[v.index], v.index % 3, which)
            if parent.name == "scf.for":
                return ("iv", id(parent)) if v.index == 0 else ("iter", id(parent), v.index - 1)
            raise _unsupported(f"block argument of {parent.name}")
        op: ht.Op = owner
        n = op.name
        if n == "arith.constant":
            return ("const", op.attributes["value"])
        if n in ("htile.copy", "htile.full"):
            return self.of(op.operands[0])
        if n == "linalg.broadcast":
            inner = self.of(op.operands[0])
            src_ty = op.operands[0].type
            if isinstance(src_ty, ht.TensorType) and src_ty.element_type.name == "index":
                return ("bcast", tuple(op.attributes["dimensions"]), inner)
            return inner
        if n == "tensor.empty":
            return ("empty",)
        if n == "scf.for":
            return ("for", id(op), v.index)
        if n == "htile.load":
            order = tuple(op.attributes.get("dimension_order", range(len(v.type.shape))))
            return ("load", self.of(op.operands[0]), tuple(self.of(o) for o in op.operands[1:]), order,
                    tuple(v.type.shape))
        if n == "htile.dot":
            if len(op.operands) != 2:
                raise _unsupported("htile.dot with an accumulator operand")
            return ("dot", self.of(op.operands[0]), self.of(op.operands[1]),
                    bool(op.attributes.get("transpose_a")), bool(op.attributes.get("transpose_b")))
        if n == "htile.reduce":
            return ("reduce", op.attributes["kind"], op.attributes["axis"], self.of(op.operands[0]))
        if n == "htile.arange":
            return ("arange", self.of(op.operands[0]), self.of(op.operands[1]))
        if n == "htile.unsqueeze":
            return ("unsqueeze", tuple(bool(b) for b in op.attributes["mask"]), self.of(op.operands[0]))
        if n == "arith.truncf":
            return ("truncf", v.type.element_type.name, self.of(op.operands[0]))
        if n in ("arith.cmpi", "arith.cmpf"):
            return (n, op.attributes["predicate"], self.of(op.operands[0]), self.of(op.operands[1]))
        if n.startswith("arith.") or n.startswith("math."):
            args = [self.of(o) for o in op.operands]
            if n in _COMMUTATIVE:
                args.sort(key=repr)
            return (n, *args)
        raise _unsupported(f"operation '{n}' is not part of any program this target recognises")


def _mul(a, b):
    return ("arith.muli", *sorted([a, b], key=repr))


def _c(fn_name: str, *args):
    if fn_name in _COMMUTATIVE:
        args = tuple(sorted(args, key=repr))
    return (fn_name, *args)


def _const_int(expr, what: str) -> int:
    if expr[0] != "const" or not isinstance(expr[1], int):
        raise _unsupported(f"{what} must be an integer constant")
    return expr[1]


class Translator:
    """Recognise each func.func of an HTile module and emit its call into the kernel library."""

    RUNTIME_ALIAS = "nb200"

    def __init__(self):
        self._emitted: list[str] = []

    # --- module entry ---

    def translate(self, module: ht.Module) -> ast.Module:
        body: list[ast.stmt] = [
            ast.ImportFrom(module="neptune_mlir", names=[ast.alias(name="runtime", asname=self.RUNTIME_ALIAS)],
                           level=0),
        ]
        for fn in module.functions:
            body.append(self._func(fn))
        mod = ast.Module(body=body, type_ignores=[])
        ast.fix_missing_locations(mod)
        return mod

    def _func(self, fn: ht.Func) -> ast.FunctionDef:
        params = [f"ptr_{i}" for i in range(len(fn.arguments))]
        for arg in fn.arguments:
            if not isinstance(arg.type, ht.MemRefType):
                raise _unsupported(f"@{fn.name}: only memref arguments are supported, got {arg.type}")
        operator = fn.attributes.get("htile.operator")
        if operator is not None:
            stmt = self._declared_operator(fn, operator, params)
        elif sum(1 for op in fn.body.operations if op.name == "gpu.launch") == 2:
            stmt = self._decode_program(fn, params)
        else:
            stmt = self._attention(fn, params)
        return function_def(fn.name, params, [stmt])

    def _runtime_call(self, fn_name: str, params: list[str], **kwargs) -> ast.stmt:
        return ast.Expr(value=call(attr(name(self.RUNTIME_ALIAS), fn_name), *[name(p) for p in params],
                                   **{k: const(v) for k, v in kwargs.items()}))

    # --- declared operators (decode, scans) ---

    def _declared_operator(self, fn: ht.Func, operator: str, params: list[str]) -> ast.stmt:
        live = [op for op in fn.body.operations if op.name not in ("return", "func.return")]
        if live:
            raise _unsupported(f"@{fn.name}: an operator declaration must have an empty body")
        types = [a.type for a in fn.arguments]
        shapes = [t.shape for t in types]
        dts = [t.element_type.name for t in types]

        def need(cond: bool, what: str) -> None:
            if not cond:
                raise _unsupported(f"@{fn.name} ({operator}): {what}")

        if operator == "decode_splitk":
            need(len(types) == 5, "expects (q, k, v, partials, out)")
            q, k, v, part, out = shapes
            need(len(q) == 3 and len(k) == 4 and k == v and out == q, "q/out [B,Hq,D], k/v [B,Hkv,L,D]")
            B, Hq, D = q
            Hkv, L = k[1], k[2]
            need(k[0] == B and k[3] == D and Hq % Hkv == 0, "inconsistent extents")
            need(len(part) == 4 and part[:2] == (B, Hq) and part[3] == D + 2 and dts[3] == "f32",
                 "partials must be memref<BxHqxSx(D+2)xf32>")
            need(dts[0] in ("f16", "bf16") and dts[0] == dts[1] == dts[2] == dts[4], "q/k/v/out share f16 or bf16")
            # n_splits = 0 leaves the count to the library (it fills the GPU's CTA slots a whole number of times);
            # the partials memref then only bounds it
            n_splits = int(fn.attributes.get("n_splits", part[2]))
            need(n_splits in (0, part[2]), "n_splits attribute disagrees with partials")
            scale = float(fn.attributes.get("scale", 1.0 / math.sqrt(D)))
            return self._runtime_call("decode_splitk", params, B=B, Hq=Hq, Hkv=Hkv, L=L, D=D, n_splits=n_splits,
                                      dtype=dts[0], scale_log2=scale * math.log2(math.e))
        if operator == "decode_paged":
            need(len(types) == 7, "expects (q, k_pages, v_pages, block_table, seq_lens, partials, out)")
            q, kp, vp, table, lens, part, out = shapes
            need(len(q) == 3 and out == q and len(kp) == 4 and kp == vp, "q/out [B,Hq,D], pools [pages,Hkv,page,D]")
            B, Hq, D = q
            Hkv, page = kp[1], kp[2]
            need(kp[3] == D and Hq % Hkv == 0, "inconsistent extents")
            need(len(table) == 2 and table[0] == B and lens == (B,) and dts[3] == dts[4] == "i32",
                 "block_table memref<Bxmax_pagesxi32>, seq_lens memref<Bxi32>")
            need(len(part) == 4 and part[:2] == (B, Hq) and part[3] == D + 2 and dts[5] == "f32",
                 "partials must be memref<BxHqxSx(D+2)xf32>")
            need(dts[0] in ("f16", "bf16") and dts[0] == dts[1] == dts[2] == dts[6], "q/pools/out share f16 or bf16")
            n_splits = part[2]
            need(int(fn.attributes.get("n_splits", n_splits)) == n_splits, "n_splits attribute disagrees with partials")
            scale = float(fn.attributes.get("scale", 1.0 / math.sqrt(D)))
            return self._runtime_call("decode_paged", params, B=B, Hq=Hq, Hkv=Hkv, max_pages=table[1], page_size=page,
                                      D=D, n_splits=n_splits, dtype=dts[0], scale_log2=scale * math.log2(math.e))
        if operator == "selective_scan":
            need(len(types) == 8, "expects (u, delta, A, B, C, D, z, out)")
            u, dl, A, Bm, Cm, Dk, z, out = shapes
            need(len(u) == 3 and u == dl == z == out, "u/delta/z/out [B,D,L]")
            B, Dm, L = u
            need(len(A) == 2 and A[0] == Dm and Bm == Cm == (B, A[1], L) and Dk == (Dm,), "A [D,N], B/C [B,N,L], D [D]")
            need(dts[2] == dts[5] == "f32", "A and D are f32")
            need(dts[0] in ("f16", "bf16") and all(dts[i] == dts[0] for i in (1, 3, 4, 6, 7)), "one 16-bit storage dtype")
            return self._runtime_call("selective_scan", params, B=B, Dm=Dm, L=L, N=A[1], dtype=dts[0])
        if operator == "ssd_chunk_scan":
            need(len(types) == 7, "expects (x, dt, A, B, C, workspace, y)")
            x, dt, A, Bm, Cm, ws, y = shapes
            need(len(x) == 4 and x == y, "x/y [B,L,H,P]")
            B, L, H, P = x
            need(dt == (B, L, H) and A == (H,) and len(Bm) == 4 and Bm == Cm and Bm[:2] == (B, L), "dt/A/B/C extents")
            G, N = Bm[2], Bm[3]
            need(dts[1] == dts[2] == "f32" and dts[0] in ("f16", "bf16") and dts[3] == dts[4] == dts[6] == dts[0],
                 "dt/A f32, x/B/C/y one 16-bit dtype")
            chunk = int(fn.attributes.get("chunk", 256))
            return self._runtime_call("ssd_chunk_scan", params, B=B, L=L, H=H, P=P, N=N, G=G, chunk=chunk, dtype=dts[0])
        raise _unsupported(f"@{fn.name}: unknown htile.operator '{operator}'")

    # --- split-K decode and its combine, spelled in HTile ops ---

    def _decode_program(self, fn: ht.Func, params: list[str]) -> ast.stmt:
        def need(cond: bool, what: str) -> None:
            if not cond:
                raise _unsupported(f"@{fn.name}: not the split-K decode program this target implements ({what})")

        for op in fn.body.walk():
            if op.name == "htile.dot":
                reject_dot_transpose_attrs(op, "B200")
        launches = [op for op in fn.body.operations if op.name == "gpu.launch"]
        others = [op for op in fn.body.operations if op.name not in ("gpu.launch", "arith.constant", "return", "func.return")]
        need(len(launches) == 2 and not others and len(fn.arguments) == 5, "five memrefs, constants and two gpu.launch regions")
        g = _Graph(fn)
        q_ty, k_ty, v_ty, p_ty, o_ty = (a.type for a in fn.arguments)
        need(len(q_ty.shape) == 3 and len(k_ty.shape) == 4 and k_ty.shape == v_ty.shape and o_ty.shape == q_ty.shape,
             "q/out [B,Hq,D], k/v [B,Hkv,L,D]")
        B, Hq, D = q_ty.shape
        Hkv, L = k_ty.shape[1], k_ty.shape[2]
        dtype = q_ty.element_type.name
        need(k_ty.shape[0] == B and k_ty.shape[3] == D and Hq % Hkv == 0, "consistent extents")
        need(dtype in ("f16", "bf16") and all(t.element_type.name == dtype for t in (k_ty, v_ty, o_ty)), "q/k/v/out share f16 or bf16")
        need(len(p_ty.shape) == 4 and p_ty.shape[:2] == (B, Hq) and p_ty.shape[3] == D + 2 and p_ty.element_type.name == "f32",
             "partials memref<BxHqxSx(D+2)xf32>")
        S = p_ty.shape[2]
        need(L % S == 0, "equal splits")
        G, T = Hq // Hkv, L // S
        c0 = ("const", 0)

        # ---- first region: one block per (split, kv head, sequence)
        first, second = launches
        body = first.regions[0]
        stores = [op for op in body.operations if op.name == "htile.store"]
        fors = [op for op in body.operations if op.name == "scf.for"]
        need(len(stores) == 3 and len(fors) == 1, "one kv loop and three stores (o, m, l) in the first region")
        need([_const_int(g.of(o), "grid size") for o in first.operands[:3]] == [S, Hkv, B], "grid (splits, kv heads, batch)")
        loop = fors[0]
        lid = id(loop)
        h0, t0 = _mul(("bid", 1), ("const", G)), _mul(("bid", 0), ("const", T))
        by_col = {}
        for st in stores:
            need(g.of(st.operands[1]) == ("arg", 3), "the first region stores into partials")
            offs = tuple(g.of(o) for o in st.operands[2:])
            need(len(offs) == 4 and offs[:3] == (("bid", 2), h0, ("bid", 0)) and offs[3][0] == "const",
                 "partials written at [bz, by*G, bx, column]")
            by_col[offs[3][1]] = g.of(st.operands[0])
        need(set(by_col) == {0, D, D + 1}, "columns 0 (o), D (m) and D+1 (l)")

        def carried(expr, mask):
            need(expr[0] == "unsqueeze" and expr[1] == mask and expr[2][:2] == ("for", lid), "stores of the loop's results")
            return expr[2][2]

        k_acc = carried(by_col[0], (False, True, False))
        k_m, k_l = carried(by_col[D], (False, True, True)), carried(by_col[D + 1], (False, True, True))
        need({k_acc, k_m, k_l} == {0, 1, 2}, "o, m, l are the three carried tiles")
        lb, ub, step = (_const_int(g.of(o), "loop bound") for o in loop.operands[:3])
        need(lb == 0 and step == 1 and ub > 0 and len(loop.results) == 3, "for j = 0 to N step 1 with three carried tiles")
        inits = [g.of(o) for o in loop.operands[3:]]
        need(inits[k_acc] == ("const", 0.0) and inits[k_l] == ("const", 0.0), "o and l start at zero")
        need(inits[k_m][0] == "const" and inits[k_m][1] < -1e30, "running maximum starts at -FLT_MAX")
        yld = loop.regions[0].operations[-1]
        need(yld.name == "scf.yield" and len(yld.operands) == 3, "loop ends in scf.yield of three tiles")
        y = [g.of(o) for o in yld.operands]
        it_acc, it_l, it_m = ("iter", lid, k_acc), ("iter", lid, k_l), ("iter", lid, k_m)
        m_new = y[k_m]
        need(m_new[0] == "arith.maximumf" and it_m in m_new[1:], "m' = max(m, rowmax S)")
        red = m_new[1] if m_new[2] == it_m else m_new[2]
        need(red[:3] == ("reduce", "max", 1), "row maximum over axis 1")
        Sx = red[3]
        need(Sx[0] == "arith.mulf", "scores scaled by a constant")
        scale_c = next((a for a in Sx[1:] if a[0] == "const"), None)
        qk = next((a for a in Sx[1:] if a[0] == "dot"), None)
        need(scale_c is not None and qk is not None and isinstance(scale_c[1], float), "S = dot(Q, K) * c")
        q_load, k_load = qk[1], qk[2]
        need(q_load[0] == "load" and k_load[0] == "load" and not qk[3] and not qk[4], "dot of two loaded tiles")
        need(q_load[1] == ("arg", 0) and q_load[2] == (("bid", 2), h0, c0) and q_load[4] == (G, D) and q_load[3] == (0, 1),
             "Q tile [G, D]: the query heads of the kv head's group")
        need(k_load[3] == (1, 0), "K tile read through dimension_order [1, 0] (K^T)")
        tile_n = k_load[4][1]
        need(ub * tile_n == T, "the loop covers the split's rows")
        rows = _c("arith.addi", t0, _mul(("iv", lid), ("const", tile_n)))
        kv_offsets = (("bid", 2), ("bid", 1), rows, c0)
        need(k_load[1] == ("arg", 1) and k_load[2] == kv_offsets and k_load[4] == (D, tile_n), "K tile [BN, D] at [bz, by, bx*T + j*BN, 0]")
        P = _c("math.exp2", _c("arith.subf", Sx, m_new))
        alpha = _c("math.exp2", _c("arith.subf", it_m, m_new))
        need(y[k_l] == _c("arith.addf", _c("arith.mulf", it_l, alpha), ("reduce", "sum", 1, P)), "l' = l * 2^(m - m') + rowsum 2^(S - m')")
        acc_new = y[k_acc]
        need(acc_new[0] == "arith.addf", "o' = o * 2^(m - m') + P V")
        pv = next((a for a in acc_new[1:] if a[0] == "dot"), None)
        rest = next((a for a in acc_new[1:] if a[0] != "dot"), None)
        need(pv is not None and rest == _c("arith.mulf", it_acc, alpha), "o rescaled by 2^(m - m')")
        need(pv[1] == P and not pv[3] and not pv[4] and pv[2][0] == "arith.extf", "P (fp32) times V extended to fp32")
        v_load = pv[2][1]
        need(v_load[0] == "load" and v_load[1] == ("arg", 2) and v_load[2] == kv_offsets and v_load[4] == (tile_n, D)
             and v_load[3] == (0, 1), "V tile [BN, D] at the K tile's offsets")

        # ---- second region: one block per (query head, sequence) merges the splits
        body2 = second.regions[0]
        stores2 = [op for op in body2.operations if op.name == "htile.store"]
        need(len(stores2) == 1 and not [op for op in body2.operations if op.name == "scf.for"], "one store and no loop in the second region")
        need([_const_int(g.of(o), "grid size") for o in second.operands[:3]] == [Hq, B, 1], "grid (query heads, batch, 1)")
        st = stores2[0]
        cx, cy = ("bid", 0, 1), ("bid", 1, 1)
        need(g.of(st.operands[1]) == ("arg", 4) and tuple(g.of(o) for o in st.operands[2:]) == (cy, cx, c0)
             and tuple(st.operands[0].type.shape) == (1, D), "out[b, h, :] written as a [1, D] tile")

        def part(col, shape):
            return ("load", ("arg", 3), (cy, cx, c0, ("const", col)), tuple(range(len(shape))), shape)

        o_l, m_l, l_l = part(0, (S, D)), part(D, (S, 1)), part(D + 1, (S, 1))
        w = _c("math.exp2", _c("arith.subf", m_l, ("reduce", "max", 0, m_l)))
        num = ("reduce", "sum", 0, _c("arith.mulf", o_l, ("reduce", "sum", 1, w)))
        den = ("reduce", "sum", 0, _c("arith.mulf", w, l_l))
        want = ("truncf", dtype, _c("arith.divf", ("unsqueeze", (True, False), num), den))
        need(g.of(st.operands[0]) == want, "out = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s, rounded to the storage dtype")
        return self._runtime_call("decode_splitk", params, B=B, Hq=Hq, Hkv=Hkv, L=L, D=D, n_splits=S, dtype=dtype,
                                  scale_log2=scale_c[1])

    # --- the FlashAttention recurrence ---

    def _attention(self, fn: ht.Func, params: list[str]) -> ast.stmt:
        def need(cond: bool, what: str) -> None:
            if not cond:
                raise _unsupported(f"@{fn.name}: not the attention recurrence this target implements ({what})")

        for op in fn.body.walk():
            if op.name == "htile.dot":
                reject_dot_transpose_attrs(op, "B200")
        need(len(fn.arguments) == 4, "expected four memrefs q, k, v, out")
        launches = [op for op in fn.body.operations if op.name == "gpu.launch"]
        others = [op for op in fn.body.operations if op.name not in ("gpu.launch", "arith.constant", "return", "func.return")]
        need(len(launches) == 1 and not others, "one gpu.launch preceded by constants")
        launch = launches[0]
        g = _Graph(fn)
        body = launch.regions[0]
        stores = [op for op in body.operations if op.name == "htile.store"]
        fors = [op for op in body.operations if op.name == "scf.for"]
        need(len(stores) == 1 and len(fors) == 1, "one KV loop and one store")
        store, loop = stores[0], fors[0]
        lid = id(loop)

        # ---- output: O = trunc(acc / l) stored at [bz, by, bx*BM, 0] ----
        out_arg = g.of(store.operands[1])
        need(out_arg[0] == "arg", "store destination is a function argument")
        out_ty: ht.MemRefType = fn.arguments[out_arg[1]].type
        dtype = out_ty.element_type.name
        need(dtype in _FLOAT_DTYPES and len(out_ty.shape) == 4, "4-D float output")
        B, H, Sq, D = out_ty.shape
        val = g.of(store.operands[0])
        if dtype != "f32":
            need(val[0] == "truncf" and val[1] == dtype, "output rounded to the storage dtype")
            val = val[2]
        need(val[0] == "arith.divf" and val[1][:2] == ("for", lid) and val[2][:2] == ("for", lid), "acc / l")
        k_acc, k_l = val[1][2], val[2][2]
        tile_m = store.operands[0].type.shape[0]
        need(tuple(store.operands[0].type.shape) == (tile_m, D), "output tile [BM, D]")
        i_base = _mul(("bid", 0), ("const", tile_m))
        q_offsets = (("bid", 2), ("bid", 1), i_base, ("const", 0))
        need(tuple(g.of(o) for o in store.operands[2:]) == q_offsets, "store offsets [bz, by, bx*BM, 0]")
        grid = [_const_int(g.of(o), "grid size") for o in launch.operands[:3]]
        need(grid == [Sq // tile_m, H, B] and Sq % tile_m == 0, f"grid (Sq/BM, H, B), got {grid}")

        # ---- loop bounds and carried values ----
        lb, ub, step = (_const_int(g.of(o), "loop bound") for o in loop.operands[:3])
        need(lb == 0 and step == 1 and ub > 0 and len(loop.results) == 3, "for j = 0 to N step 1 with three carried tiles")
        k_m = ({0, 1, 2} - {k_acc, k_l}).pop()
        inits = [g.of(o) for o in loop.operands[3:]]
        need(inits[k_acc] == ("const", 0.0) and inits[k_l] == ("const", 0.0), "acc and l start at zero")
        need(inits[k_m][0] == "const" and inits[k_m][1] < -1e30, "running maximum starts at -FLT_MAX")
        neg_init = inits[k_m]
        yld = loop.regions[0].operations[-1]
        need(yld.name == "scf.yield" and len(yld.operands) == 3, "loop ends in scf.yield of three tiles")
        y = [g.of(o) for o in yld.operands]
        it_acc, it_l, it_m = ("iter", lid, k_acc), ("iter", lid, k_l), ("iter", lid, k_m)

        # ---- m' = max(m, rowmax S) ----
        m_new = y[k_m]
        need(m_new[0] == "arith.maximumf" and it_m in m_new[1:], "m' = max(m, rowmax S)")
        red = m_new[1] if m_new[2] == it_m else m_new[2]
        need(red[:3] == ("reduce", "max", 1), "row maximum over axis 1")
        S = red[3]

        # ---- S = (Q K^T) * c, optionally causally masked ----
        causal = False
        if S[0] == "arith.select":
            mask, S, fill = S[1], S[2], S[3]
            need(fill == neg_init, "masked scores take the running maximum's initial value")
            need(mask[0] == "arith.cmpi" and mask[1] in ("sge", "sle"), "mask is an integer comparison")
            rows, cols = (mask[2], mask[3]) if mask[1] == "sge" else (mask[3], mask[2])
            need(rows[0] == "bcast" and rows[1] == (1,) and cols[0] == "bcast" and cols[1] == (0,), "row >= col mask")
            need(rows[2][0] == "arange" and rows[2][1] == i_base, "row indices start at the query tile")
            need(cols[2][0] == "arange" and cols[2][1][0] == "arith.muli", "column indices start at the kv tile")
            causal = True
        need(S[0] == "arith.mulf", "scores scaled by a constant")
        scale_c = next((a for a in S[1:] if a[0] == "const"), None)
        qk = next((a for a in S[1:] if a[0] == "dot"), None)
        need(scale_c is not None and qk is not None and isinstance(scale_c[1], float), "S = dot(Q, K) * c")
        q_load, k_load = qk[1], qk[2]
        need(q_load[0] == "load" and k_load[0] == "load" and not qk[3] and not qk[4], "dot of two loaded tiles")
        need(k_load[3] == (1, 0), "K tile read through dimension_order [1, 0] (K^T)")
        tile_n = k_load[4][1]
        j_base = _mul(("iv", lid), ("const", tile_n))
        kv_offsets = (("bid", 2), ("bid", 1), j_base, ("const", 0))
        need(q_load[1][0] == "arg" and q_load[2] == q_offsets and q_load[4] == (tile_m, D), "Q tile [BM, D] at the query offsets")
        need(k_load[1][0] == "arg" and k_load[2] == kv_offsets and k_load[4] == (D, tile_n), "K tile [BN, D] at [bz, by, j*BN, 0]")
        if causal:
            need(cols[2][1] == j_base, "column indices start at j*BN")
        Skv = ub * tile_n
        k_ty: ht.MemRefType = fn.arguments[k_load[1][1]].type
        need(k_ty.shape == (B, H, Skv, D), "K extent equals trip count x kv tile")
        need(not causal or Skv == Sq, "causal programs are square (Skv == Sq)")

        # ---- P, l', acc' ----
        S_used = red[3]
        P = _c("math.exp2", _c("arith.subf", S_used, m_new))
        alpha = _c("math.exp2", _c("arith.subf", it_m, m_new))
        need(y[k_l] == _c("arith.addf", _c("arith.mulf", it_l, alpha), ("reduce", "sum", 1, P)),
             "l' = l * 2^(m - m') + rowsum 2^(S - m')")
        acc_new = y[k_acc]
        need(acc_new[0] == "arith.addf", "acc' = acc * 2^(m - m') + P V")
        pv = next((a for a in acc_new[1:] if a[0] == "dot"), None)
        rest = next((a for a in acc_new[1:] if a[0] != "dot"), None)
        need(pv is not None and rest == _c("arith.mulf", it_acc, alpha), "acc rescaled by 2^(m - m')")
        P_in = ("truncf", dtype, P) if dtype != "f32" else P
        v_load = pv[2]
        need(pv[1] == P_in and not pv[3] and not pv[4], "PV product uses P rounded to the storage dtype")
        need(v_load[0] == "load" and v_load[1][0] == "arg" and v_load[2] == kv_offsets and v_load[4] == (tile_n, D)
             and v_load[3] == (0, 1), "V tile [BN, D] at [bz, by, j*BN, 0]")
        args_used = [q_load[1][1], k_load[1][1], v_load[1][1], out_arg[1]]
        need(sorted(args_used) == [0, 1, 2, 3], "q, k, v, out are the four distinct arguments")
        for i in args_used[:3]:
            need(fn.arguments[i].type.element_type.name == dtype, "q, k, v, out share one dtype")
        need(fn.arguments[args_used[0]].type.shape == (B, H, Sq, D), "Q extent")
        need(fn.arguments[args_used[2]].type.shape == (B, H, Skv, D), "V extent")

        ordered = [params[i] for i in args_used]
        return self._runtime_call("attn_fwd", ordered, shape=(B, H, Sq, D), kv_len=Skv, dtype=dtype,
                                  scale_log2=scale_c[1], causal=causal)


# ---------------------------------------------------------------------------
# Entry point
# ---------------------------------------------------------------------------


def translate_file(path: str, plugin: str | None = None) -> ast.Module:
    """Read *path*, run the dot-transpose pass pipeline, and return a Python ast.Module."""
    return translate_file_with(
        path,
        Translator,
        plugin,
        pass_pipeline=HTILE_DOT_TRANSPOSE_TO_LOAD_ORDER_PIPELINE,
        pass_plugin=plugin,
    )


def main():
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("mlir_file")
    ap.add_argument("--plugin", default=DEFAULT_LIBRARY,
                    help="path to libnb200.so (informational; the emitted module locates it at run time)")
    args = ap.parse_args()

    py_module = translate_file(args.mlir_file, args.plugin)
    print(ast.unparse(py_module))


if __name__ == "__main__":
    main()
