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
