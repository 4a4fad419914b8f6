"""Writers of HTile program text for the operator families the B200 target implements.

The attention writer produces the FlashAttention recurrence in the value-based HTile style of the
reference's example (tests/data/flash_attention_htile.mlir), parametrised by shape, dtype, tile
sizes and causality, so that programs for other problem sizes need no hand editing.  The causal
variant masks scores with htile.arange + arith.cmpi + arith.select (ops the dialect defines,
include/HTile/HTileOps.td:90-101, but no reference translator handles).  The decode / scan writers
emit operator declarations: a func.func with an ``htile.operator`` attribute and an empty body.
"""

from __future__ import annotations

import math
import struct


def _f32(x: float) -> float:
    return struct.unpack("f", struct.pack("f", x))[0]


def attention_htile(name: str, B: int, H: int, S: int, D: int, dtype: str = "f16", causal: bool = False,
                    tile_m: int = 128, tile_n: int = 64, stages: int = 2) -> str:
    """HTile text of softmax(Q K^T / sqrt(D)) V with an exp2-domain online softmax."""
    assert S % tile_m == 0 and S % tile_n == 0
    mem = f"memref<{B}x{H}x{S}x{D}x{dtype}>"
    scale = _f32(math.log2(math.e) / math.sqrt(D))

    def t(shape, elem, place):
        return f"tensor<{'x'.join(map(str, shape))}x{elem}, #{place}>"

    sc, row, acc = t((tile_m, tile_n), "f32", "local"), t((tile_m,), "f32", "local"), t((tile_m, D), "f32", "local")
    p_ty = t((tile_m, tile_n), dtype, "local")
    o_ty = t((tile_m, D), dtype, "local")
    L: list[str] = []
    a = L.append
    a("#shared = #htile.encoding<placement = shared>")
    a("#local = #htile.encoding<placement = local>")
    a("")
    a("module {")
    a(f"  func.func @{name}(%q: {mem}, %k: {mem}, %v: {mem}, %out: {mem}) {{")
    a("    %c0 = arith.constant 0 : index")
    a("    %c1 = arith.constant 1 : index")
    a(f"    %grid_m = arith.constant {S // tile_m} : index")
    a(f"    %heads = arith.constant {H} : index")
    a(f"    %batch = arith.constant {B} : index")
    a(f"    %kv_steps = arith.constant {S // tile_n} : index")
    a(f"    %bm = arith.constant {tile_m} : index")
    a(f"    %bn = arith.constant {tile_n} : index")
    a("    %zero = arith.constant 0.0 : f32")
    a("    %lowest = arith.constant -3.40282347E+38 : f32")
    a(f"    %c = arith.constant {scale!r} : f32")
    a("    gpu.launch blocks(%bx, %by, %bz) in (%gx = %grid_m, %gy = %heads, %gz = %batch)")
    a("               threads(%tx, %ty, %tz) in (%sx = %bm, %sy = %c1, %sz = %c1) {")
    a("      %i0 = arith.muli %bx, %bm : index")
    a(f"      %q_tile = htile.load %q[%bz, %by, %i0, %c0] : {mem} -> {t((tile_m, D), dtype, 'shared')}")
    a(f"      %m_init = htile.full %lowest : f32 -> {row}")
    a(f"      %l_init = htile.full %zero : f32 -> {row}")
    a(f"      %acc_init = htile.full %zero : f32 -> {acc}")
    if causal:
        a("      %i1 = arith.addi %i0, %bm : index")
        a(f"      %rows = htile.arange %i0 to %i1 : {t((tile_m,), 'index', 'local')}")
        a(f"      %rows_e = tensor.empty() : {t((tile_m, tile_n), 'index', 'local')}")
        a(f"      %rows_b = linalg.broadcast ins(%rows : {t((tile_m,), 'index', 'local')}) "
          f"outs(%rows_e : {t((tile_m, tile_n), 'index', 'local')}) dimensions = [1]")
        a(f"      %fill = htile.full %lowest : f32 -> {sc}")
    a("      %l_out, %acc_out, %m_out = scf.for %j = %c0 to %kv_steps step %c1")
    a("          iter_args(%l = %l_init, %acc = %acc_init, %m = %m_init)")
    a(f"          -> ({row}, {acc}, {row}) {{")
    a("        %j0 = arith.muli %j, %bn : index")
    a(f"        %k_tile = htile.load %k[%bz, %by, %j0, %c0] : {mem} -> {t((tile_n, D), dtype, 'shared')}")
    a(f"        %qk = htile.dot %q_tile, %k_tile {{transpose_b, warp_policy = \"full_row\"}} : "
      f"{t((tile_m, D), dtype, 'shared')}, {t((tile_n, D), dtype, 'shared')} -> {sc}")
    a(f"        %c_tile = htile.full %c : f32 -> {sc}")
    a(f"        %s_raw = arith.mulf %qk, %c_tile : {sc}")
    score = "%s_raw"
    if causal:
        a("        %j1 = arith.addi %j0, %bn : index")
        a(f"        %cols = htile.arange %j0 to %j1 : {t((tile_n,), 'index', 'local')}")
        a(f"        %cols_e = tensor.empty() : {t((tile_m, tile_n), 'index', 'local')}")
        a(f"        %cols_b = linalg.broadcast ins(%cols : {t((tile_n,), 'index', 'local')}) "
          f"outs(%cols_e : {t((tile_m, tile_n), 'index', 'local')}) dimensions = [0]")
        a(f"        %visible = arith.cmpi sge, %rows_b, %cols_b : {t((tile_m, tile_n), 'index', 'local')}")
        a(f"        %s = arith.select %visible, %s_raw, %fill : {t((tile_m, tile_n), 'i1', 'local')}, {sc}")
        score = "%s"
    a(f"        %s_max = htile.reduce {score} axis 1 kind \"max\" : {sc} -> {row}")
    a(f"        %m_new = arith.maximumf %m, %s_max : {row}")
    a(f"        %m_new_e = tensor.empty() : {sc}")
    a(f"        %m_new_b = linalg.broadcast ins(%m_new : {row}) outs(%m_new_e : {sc}) dimensions = [1]")
    a(f"        %shifted = arith.subf {score}, %m_new_b : {sc}")
    a(f"        %p = math.exp2 %shifted : {sc}")
    a(f"        %p_sum = htile.reduce %p axis 1 kind \"sum\" : {sc} -> {row}")
    a(f"        %dm = arith.subf %m, %m_new : {row}")
    a(f"        %alpha = math.exp2 %dm : {row}")
    a(f"        %l_scaled = arith.mulf %l, %alpha : {row}")
    a(f"        %l_new = arith.addf %l_scaled, %p_sum : {row}")
    p_val = "%p"
    if dtype != "f32":
        a(f"        %p_lo = arith.truncf %p : {sc} to {p_ty}")
        p_val = "%p_lo"
    a(f"        %v_tile = htile.load %v[%bz, %by, %j0, %c0] : {mem} -> {t((tile_n, D), dtype, 'shared')}")
    a(f"        %pv = htile.dot {p_val}, %v_tile {{warp_policy = \"full_row\"}} : "
      f"{p_ty if dtype != 'f32' else sc}, {t((tile_n, D), dtype, 'shared')} -> {acc}")
    a(f"        %alpha_e = tensor.empty() : {acc}")
    a(f"        %alpha_b = linalg.broadcast ins(%alpha : {row}) outs(%alpha_e : {acc}) dimensions = [1]")
    a(f"        %acc_scaled = arith.mulf %acc, %alpha_b : {acc}")
    a(f"        %acc_new = arith.addf %acc_scaled, %pv : {acc}")
    a(f"        scf.yield %l_new, %acc_new, %m_new : {row}, {acc}, {row}")
    a(f"      }} {{htile.pipeline_stages = {stages} : i32}}")
    a(f"      %l_e = tensor.empty() : {acc}")
    a(f"      %l_b = linalg.broadcast ins(%l_out : {row}) outs(%l_e : {acc}) dimensions = [1]")
    a(f"      %o = arith.divf %acc_out, %l_b : {acc}")
    o_val = "%o"
    if dtype != "f32":
        a(f"      %o_lo = arith.truncf %o : {acc} to {o_ty}")
        o_val = "%o_lo"
    a(f"      htile.store {o_val}, %out[%bz, %by, %i0, %c0] : {o_ty if dtype != 'f32' else acc}, {mem}")
    a("      gpu.terminator")
    a("    }")
    a("    return")
    a("  }")
    a("}")
    return "\n".join(L) + "\n"


def attention_l1(name: str, B: int, H: int, S: int, D: int, dtype: str = "f16", tile_m: int = 128, tile_n: int = 64,
                 stages: int = 2) -> str:
    """Level-1 (scheduled tile IR) text of non-causal attention: tensors, scf.forall over (batch, head, row
    block), affine.for over the kv blocks carrying (l, acc, m), linalg / arith / math tile bodies -- the form of the
    reference's tests/data/flash_attention_l1.mlir, which ``neptune_mlir.l1.lower_to_htile`` lowers to HTile."""
    assert S % tile_m == 0 and S % tile_n == 0
    full = f"tensor<{B}x{H}x{S}x{D}x{dtype}>"
    scale = math.log2(math.e) / math.sqrt(D)

    def t(*shape, elem="f32"):
        return f"tensor<{'x'.join(map(str, shape))}x{elem}>"

    q_t, kv_t = t(tile_m, D, elem=dtype), t(tile_n, D, elem=dtype)
    s_t, row, acc = t(tile_m, tile_n), t(tile_m), t(tile_m, D)
    trunc_p = f"%p_lo = arith.truncf %p : {s_t} to {t(tile_m, tile_n, elem=dtype)}" if dtype != "f32" else None
    p_in, p_ty = ("%p_lo", t(tile_m, tile_n, elem=dtype)) if dtype != "f32" else ("%p", s_t)
    L = [
        "module {",
        f"  func.func @{name}(%q: {full}, %k: {full}, %v: {full}) -> {full} {{",
        "    %zero = arith.constant 0.0 : f32",
        "    %lowest = arith.constant -3.40282347E+38 : f32",
        f"    %scale = arith.constant {scale!r} : f32",
        f"    %bm = arith.constant {tile_m} : index",
        f"    %o_init = tensor.empty() : {full}",
        f"    %o = scf.forall (%b, %h, %blk) in ({B}, {H}, {S // tile_m}) shared_outs(%o_it = %o_init) -> {full} {{",
        "      %i0 = arith.muli %blk, %bm : index",
        f"      %q_tile = tensor.extract_slice %q[%b, %h, %i0, 0] [1, 1, {tile_m}, {D}] [1, 1, 1, 1] : {full} to {q_t}",
        f"      %acc_e = tensor.empty() : {acc}",
        f"      %acc0 = linalg.fill ins(%zero : f32) outs(%acc_e : {acc}) -> {acc}",
        f"      %row_e = tensor.empty() : {row}",
        f"      %m0 = linalg.fill ins(%lowest : f32) outs(%row_e : {row}) -> {row}",
        f"      %l0 = linalg.fill ins(%zero : f32) outs(%row_e : {row}) -> {row}",
        f"      %l_out, %acc_out, %m_out = affine.for %j = 0 to {S // tile_n} iter_args(%l = %l0, %acc = %acc0, %m = %m0) -> ({row}, {acc}, {row}) {{",
        f"        %j0 = affine.apply affine_map<(d) -> (d * {tile_n})>(%j)",
        f"        %k_tile = tensor.extract_slice %k[%b, %h, %j0, 0] [1, 1, {tile_n}, {D}] [1, 1, 1, 1] : {full} to {kv_t}",
        f"        %s_e = tensor.empty() : {s_t}",
        f"        %s0 = linalg.fill ins(%zero : f32) outs(%s_e : {s_t}) -> {s_t}",
        "        %qk = linalg.matmul indexing_maps = [affine_map<(m, n, k) -> (m, k)>, affine_map<(m, n, k) -> (n, k)>, affine_map<(m, n, k) -> (m, n)>]",
        f"            ins(%q_tile, %k_tile : {q_t}, {kv_t}) outs(%s0 : {s_t}) -> {s_t}",
        f"        %s = linalg.map ins(%qk : {s_t}) outs(%s_e : {s_t}) (%x: f32, %unused: f32) {{",
        "          %y = arith.mulf %x, %scale : f32",
        "          linalg.yield %y : f32",
        "        }",
        f"        %max_seed = linalg.fill ins(%lowest : f32) outs(%row_e : {row}) -> {row}",
        f"        %s_max = linalg.reduce {{ arith.maximumf }} ins(%s : {s_t}) outs(%max_seed : {row}) dimensions = [1]",
        f"        %m_new = arith.maximumf %m, %s_max : {row}",
        f"        %m_new_b = linalg.broadcast ins(%m_new : {row}) outs(%s_e : {s_t}) dimensions = [1]",
        f"        %shifted = arith.subf %s, %m_new_b : {s_t}",
        f"        %p = math.exp2 %shifted : {s_t}",
        f"        %sum_seed = linalg.fill ins(%zero : f32) outs(%row_e : {row}) -> {row}",
        f"        %p_sum = linalg.reduce {{ arith.addf }} ins(%p : {s_t}) outs(%sum_seed : {row}) dimensions = [1]",
        f"        %dm = arith.subf %m, %m_new : {row}",
        f"        %alpha = math.exp2 %dm : {row}",
        f"        %l_scaled = arith.mulf %l, %alpha : {row}",
        f"        %l_new = arith.addf %l_scaled, %p_sum : {row}",
        *([f"        {trunc_p}"] if trunc_p else []),
        f"        %v_tile = tensor.extract_slice %v[%b, %h, %j0, 0] [1, 1, {tile_n}, {D}] [1, 1, 1, 1] : {full} to {kv_t}",
        f"        %pv0 = linalg.fill ins(%zero : f32) outs(%acc_e : {acc}) -> {acc}",
        f"        %pv = linalg.matmul ins({p_in}, %v_tile : {p_ty}, {kv_t}) outs(%pv0 : {acc}) -> {acc}",
        f"        %alpha_b = linalg.broadcast ins(%alpha : {row}) outs(%acc_e : {acc}) dimensions = [1]",
        f"        %acc_scaled = arith.mulf %acc, %alpha_b : {acc}",
        f"        %acc_new = arith.addf %acc_scaled, %pv : {acc}",
        f"        affine.yield %l_new, %acc_new, %m_new : {row}, {acc}, {row}",
        f"      }} {{pipeline_stages = {stages} : i32}}",
        f"      %l_b = linalg.broadcast ins(%l_out : {row}) outs(%acc_e : {acc}) dimensions = [1]",
        f"      %norm = arith.divf %acc_out, %l_b : {acc}",
        *([f"      %o_tile = arith.truncf %norm : {acc} to {t(tile_m, D, elem=dtype)}"] if dtype != "f32" else []),
        "      scf.forall.in_parallel {",
        f"        tensor.parallel_insert_slice {'%o_tile' if dtype != 'f32' else '%norm'} into %o_it[%b, %h, %i0, 0] [1, 1, {tile_m}, {D}] [1, 1, 1, 1] : {t(tile_m, D, elem=dtype)} into {full}",
        "      }",
        "    }",
        f"    return %o : {full}",
        "  }",
        "}",
    ]
    return "\n".join(L) + "\n"


def decode_splitk_htile(name: str, B: int, Hq: int, Hkv: int, L: int, D: int, n_splits: int, dtype: str = "bf16",
                        tile_n: int = 64) -> str:
    """Split-K flash-decoding with grouped-query attention and its log-sum-exp combine, spelled in HTile ops.

    Two ``gpu.launch`` regions in one function.  The first has one block per (split, kv head, sequence): the G
    query heads that share the kv head form a G x D tile, the split's rows are streamed in tiles of ``tile_n``
    with the same exp2-domain online softmax as the attention program (scores from the 16-bit tiles, everything
    after in fp32, V extended rather than P rounded), and the un-normalised output, the running maximum and the
    sum go to ``partials[b, h, split, 0:D | D | D+1]``.  The second has one block per (query head, sequence): it
    reads the head's [splits, D + 2] partials and writes ``sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s``.
    Splits are equal here (L a multiple of n_splits * tile_n); the operator declaration
    (``decode_splitk_decl``) covers ragged splits and a split count chosen by the library."""
    assert Hq % Hkv == 0 and L % n_splits == 0 and (L // n_splits) % tile_n == 0
    G, T, S = Hq // Hkv, L // n_splits, n_splits
    q_mem, kv_mem = f"memref<{B}x{Hq}x{D}x{dtype}>", f"memref<{B}x{Hkv}x{L}x{D}x{dtype}>"
    p_mem = f"memref<{B}x{Hq}x{S}x{D + 2}xf32>"
    scale = _f32(math.log2(math.e) / math.sqrt(D))

    def t(shape, elem="f32", place="local"):
        return f"tensor<{'x'.join(map(str, shape))}x{elem}, #{place}>"

    sc, row, acc = t((G, tile_n)), t((G,)), t((G, D))
    kv_t = t((tile_n, D), dtype, "shared")
    L_: list[str] = []
    a = L_.append
    a("#shared = #htile.encoding<placement = shared>")
    a("#local = #htile.encoding<placement = local>")
    a("")
    a("module {")
    a(f"  func.func @{name}(%q: {q_mem}, %k: {kv_mem}, %v: {kv_mem}, %partials: {p_mem}, %out: {q_mem}) {{")
    a("    %c0 = arith.constant 0 : index")
    a("    %c1 = arith.constant 1 : index")
    a(f"    %splits = arith.constant {S} : index")
    a(f"    %kv_heads = arith.constant {Hkv} : index")
    a(f"    %q_heads = arith.constant {Hq} : index")
    a(f"    %batch = arith.constant {B} : index")
    a(f"    %group = arith.constant {G} : index")
    a(f"    %split_rows = arith.constant {T} : index")
    a(f"    %kv_steps = arith.constant {T // tile_n} : index")
    a(f"    %bn = arith.constant {tile_n} : index")
    a(f"    %col_m = arith.constant {D} : index")
    a(f"    %col_l = arith.constant {D + 1} : index")
    a("    %threads = arith.constant 256 : index")
    a("    %zero = arith.constant 0.0 : f32")
    a("    %lowest = arith.constant -3.40282347E+38 : f32")
    a(f"    %c = arith.constant {scale!r} : f32")
    a("    gpu.launch blocks(%bx, %by, %bz) in (%gx = %splits, %gy = %kv_heads, %gz = %batch)")
    a("               threads(%tx, %ty, %tz) in (%sx = %threads, %sy = %c1, %sz = %c1) {")
    a("      %h0 = arith.muli %by, %group : index")
    a("      %t0 = arith.muli %bx, %split_rows : index")
    a(f"      %q_tile = htile.load %q[%bz, %h0, %c0] : {q_mem} -> {t((G, D), dtype, 'shared')}")
    a(f"      %m_init = htile.full %lowest : f32 -> {row}")
    a(f"      %l_init = htile.full %zero : f32 -> {row}")
    a(f"      %acc_init = htile.full %zero : f32 -> {acc}")
    a("      %l_out, %acc_out, %m_out = scf.for %j = %c0 to %kv_steps step %c1")
    a("          iter_args(%l = %l_init, %acc = %acc_init, %m = %m_init)")
    a(f"          -> ({row}, {acc}, {row}) {{")
    a("        %j0 = arith.muli %j, %bn : index")
    a("        %r0 = arith.addi %t0, %j0 : index")
    a(f"        %k_tile = htile.load %k[%bz, %by, %r0, %c0] : {kv_mem} -> {kv_t}")
    a(f"        %qk = htile.dot %q_tile, %k_tile {{transpose_b, warp_policy = \"full_row\"}} : {t((G, D), dtype, 'shared')}, {kv_t} -> {sc}")
    a(f"        %c_tile = htile.full %c : f32 -> {sc}")
    a(f"        %s = arith.mulf %qk, %c_tile : {sc}")
    a(f"        %s_max = htile.reduce %s axis 1 kind \"max\" : {sc} -> {row}")
    a(f"        %m_new = arith.maximumf %m, %s_max : {row}")
    a(f"        %m_new_e = tensor.empty() : {sc}")
    a(f"        %m_new_b = linalg.broadcast ins(%m_new : {row}) outs(%m_new_e : {sc}) dimensions = [1]")
    a(f"        %shifted = arith.subf %s, %m_new_b : {sc}")
    a(f"        %p = math.exp2 %shifted : {sc}")
    a(f"        %p_sum = htile.reduce %p axis 1 kind \"sum\" : {sc} -> {row}")
    a(f"        %dm = arith.subf %m, %m_new : {row}")
    a(f"        %alpha = math.exp2 %dm : {row}")
    a(f"        %l_scaled = arith.mulf %l, %alpha : {row}")
    a(f"        %l_new = arith.addf %l_scaled, %p_sum : {row}")
    a(f"        %v_tile = htile.load %v[%bz, %by, %r0, %c0] : {kv_mem} -> {kv_t}")
    a(f"        %v_f = arith.extf %v_tile : {kv_t} to {t((tile_n, D))}")
    a(f"        %pv = htile.dot %p, %v_f {{warp_policy = \"full_row\"}} : {sc}, {t((tile_n, D))} -> {acc}")
    a(f"        %alpha_e = tensor.empty() : {acc}")
    a(f"        %alpha_b = linalg.broadcast ins(%alpha : {row}) outs(%alpha_e : {acc}) dimensions = [1]")
    a(f"        %acc_scaled = arith.mulf %acc, %alpha_b : {acc}")
    a(f"        %acc_new = arith.addf %acc_scaled, %pv : {acc}")
    a(f"        scf.yield %l_new, %acc_new, %m_new : {row}, {acc}, {row}")
    a("      }")
    a(f"      %o3 = htile.unsqueeze %acc_out mask [false, true, false] : {acc} -> {t((G, 1, D))}")
    a(f"      htile.store %o3, %partials[%bz, %h0, %bx, %c0] : {t((G, 1, D))}, {p_mem}")
    a(f"      %m3 = htile.unsqueeze %m_out mask [false, true, true] : {row} -> {t((G, 1, 1))}")
    a(f"      htile.store %m3, %partials[%bz, %h0, %bx, %col_m] : {t((G, 1, 1))}, {p_mem}")
    a(f"      %l3 = htile.unsqueeze %l_out mask [false, true, true] : {row} -> {t((G, 1, 1))}")
    a(f"      htile.store %l3, %partials[%bz, %h0, %bx, %col_l] : {t((G, 1, 1))}, {p_mem}")
    a("      gpu.terminator")
    a("    }")
    col, one, vec = t((S, 1), place="shared"), t((1,)), t((D,))
    a("    gpu.launch blocks(%cx, %cy, %cz) in (%hx = %q_heads, %hy = %batch, %hz = %c1)")
    a("               threads(%ux, %uy, %uz) in (%wx = %threads, %wy = %c1, %wz = %c1) {")
    a(f"      %o_sh = htile.load %partials[%cy, %cx, %c0, %c0] : {p_mem} -> {t((S, D), place='shared')}")
    a(f"      %ms_sh = htile.load %partials[%cy, %cx, %c0, %col_m] : {p_mem} -> {col}")
    a(f"      %ls_sh = htile.load %partials[%cy, %cx, %c0, %col_l] : {p_mem} -> {col}")
    a(f"      %o = htile.copy %o_sh : {t((S, D), place='shared')} -> {t((S, D))}")
    a(f"      %ms = htile.copy %ms_sh : {col} -> {t((S, 1))}")
    a(f"      %ls = htile.copy %ls_sh : {col} -> {t((S, 1))}")
    a(f"      %big = htile.reduce %ms axis 0 kind \"max\" : {t((S, 1))} -> {one}")
    a(f"      %big_e = tensor.empty() : {t((S, 1))}")
    a(f"      %big_b = linalg.broadcast ins(%big : {one}) outs(%big_e : {t((S, 1))}) dimensions = [0]")
    a(f"      %dms = arith.subf %ms, %big_b : {t((S, 1))}")
    a(f"      %w = math.exp2 %dms : {t((S, 1))}")
    a(f"      %wl = arith.mulf %w, %ls : {t((S, 1))}")
    a(f"      %den = htile.reduce %wl axis 0 kind \"sum\" : {t((S, 1))} -> {one}")
    a(f"      %w1 = htile.reduce %w axis 1 kind \"sum\" : {t((S, 1))} -> {t((S,))}")
    a(f"      %w_e = tensor.empty() : {t((S, D))}")
    a(f"      %w_b = linalg.broadcast ins(%w1 : {t((S,))}) outs(%w_e : {t((S, D))}) dimensions = [1]")
    a(f"      %wo = arith.mulf %o, %w_b : {t((S, D))}")
    a(f"      %num = htile.reduce %wo axis 0 kind \"sum\" : {t((S, D))} -> {vec}")
    a(f"      %num2 = htile.unsqueeze %num mask [true, false] : {vec} -> {t((1, D))}")
    a(f"      %den_e = tensor.empty() : {t((1, D))}")
    a(f"      %den_b = linalg.broadcast ins(%den : {one}) outs(%den_e : {t((1, D))}) dimensions = [1]")
    a(f"      %res = arith.divf %num2, %den_b : {t((1, D))}")
    a(f"      %res_lo = arith.truncf %res : {t((1, D))} to {t((1, D), dtype)}")
    a(f"      htile.store %res_lo, %out[%cy, %cx, %c0] : {t((1, D), dtype)}, {q_mem}")
    a("      gpu.terminator")
    a("    }")
    a("    return")
    a("  }")
    a("}")
    return "\n".join(L_) + "\n"


def _decl(name: str, args: list[tuple[str, str]], attrs: dict) -> str:
    sig = ", ".join(f"%{n}: {ty}" for n, ty in args)
    parts = []
    for k, v in attrs.items():
        if isinstance(v, str):
            parts.append(f'{k} = "{v}"')
        elif isinstance(v, float):
            parts.append(f"{k} = {v!r} : f32")
        else:
            parts.append(f"{k} = {v} : i64")
    return ("module {\n"
            f"  func.func @{name}({sig}) attributes {{{', '.join(parts)}}} {{\n"
            "    return\n  }\n}\n")


def decode_splitk_decl(name: str, B: int, Hq: int, Hkv: int, L: int, D: int, n_splits: int, dtype: str = "bf16",
                       auto_splits: bool = False) -> str:
    """Declaration of split-K flash-decoding: (q, k, v, partials, out).

    With ``auto_splits`` the partials memref is still sized for ``n_splits`` but the attribute says 0: the library
    picks the count (at most ``n_splits``) that fills the GPU it runs on."""
    attr_splits = 0 if auto_splits else n_splits
    return _decl(name, [
        ("q", f"memref<{B}x{Hq}x{D}x{dtype}>"),
        ("k", f"memref<{B}x{Hkv}x{L}x{D}x{dtype}>"),
        ("v", f"memref<{B}x{Hkv}x{L}x{D}x{dtype}>"),
        ("partials", f"memref<{B}x{Hq}x{n_splits}x{D + 2}xf32>"),
        ("out", f"memref<{B}x{Hq}x{D}x{dtype}>"),
    ], {"htile.operator": "decode_splitk", "n_splits": attr_splits, "scale": _f32(1.0 / math.sqrt(D))})


def decode_paged_decl(name: str, B: int, Hq: int, Hkv: int, num_pages: int, max_pages: int, D: int, n_splits: int,
                      page_size: int = 64, dtype: str = "bf16") -> str:
    """Declaration of split-K decode over a paged KV cache: (q, k_pages, v_pages, block_table, seq_lens, partials, out)."""
    pool = f"memref<{num_pages}x{Hkv}x{page_size}x{D}x{dtype}>"
    return _decl(name, [
        ("q", f"memref<{B}x{Hq}x{D}x{dtype}>"),
        ("k_pages", pool),
        ("v_pages", pool),
        ("block_table", f"memref<{B}x{max_pages}xi32>"),
        ("seq_lens", f"memref<{B}xi32>"),
        ("partials", f"memref<{B}x{Hq}x{n_splits}x{D + 2}xf32>"),
        ("out", f"memref<{B}x{Hq}x{D}x{dtype}>"),
    ], {"htile.operator": "decode_paged", "n_splits": n_splits, "scale": _f32(1.0 / math.sqrt(D))})


def selective_scan_decl(name: str, B: int, Dm: int, L: int, N: int = 16, dtype: str = "bf16") -> str:
    """Declaration of the Mamba-1 selective scan: (u, delta, A, B, C, D, z, out)."""
    seq = f"memref<{B}x{Dm}x{L}x{dtype}>"
    bc = f"memref<{B}x{N}x{L}x{dtype}>"
    return _decl(name, [("u", seq), ("delta", seq), ("A", f"memref<{Dm}x{N}xf32>"), ("B", bc), ("C", bc),
                        ("D", f"memref<{Dm}xf32>"), ("z", seq), ("out", seq)],
                 {"htile.operator": "selective_scan"})


def ssd_chunk_scan_decl(name: str, B: int, L: int, H: int, P: int, N: int, G: int, chunk: int,
                        workspace_bytes: int, dtype: str = "bf16") -> str:
    """Declaration of the Mamba-2 SSD chunked scan: (x, dt, A, B, C, workspace, y)."""
    xy = f"memref<{B}x{L}x{H}x{P}x{dtype}>"
    bc = f"memref<{B}x{L}x{G}x{N}x{dtype}>"
    return _decl(name, [("x", xy), ("dt", f"memref<{B}x{L}x{H}xf32>"), ("A", f"memref<{H}xf32>"), ("B", bc),
                        ("C", bc), ("workspace", f"memref<{workspace_bytes}xi8>"), ("y", xy)],
                 {"htile.operator": "ssd_chunk_scan", "chunk": chunk})
