"""HTile text reader, the dot-transpose rewrite and the B200 translator (no GPU needed).

Modelled on the reference's tests/test_translators.py: golden-text equality of the emitted module
(:154-181), the pass's textual post-conditions (:235-257) and the negative test for unfissioned
transposes (:260-263).
"""

import ast
import os
from pathlib import Path

import pytest

from neptune_mlir import htile_text as ht
from neptune_mlir import passes, programs
from neptune_mlir.translators import b200
from neptune_mlir.translators.common import parse_mlir_module, translate_file_with

ROOT = Path(__file__).resolve().parents[1]
DATA = ROOT / "tests" / "data"
GOLDEN = ROOT / "tests" / "golden"
# the reference project's own program, when its tree is available ($NEPTUNE_REFERENCE_ROOT, else a sibling "reference" directory)
REFERENCE_ROOT = Path(os.environ.get("NEPTUNE_REFERENCE_ROOT", ROOT.parent / "reference"))
REFERENCE_PROGRAM = REFERENCE_ROOT / "tests" / "data" / "flash_attention_htile.mlir"

STEMS = sorted(p.stem for p in DATA.glob("*.mlir"))


@pytest.mark.parametrize("stem", STEMS)
def test_b200_translator_matches_golden(stem):
    actual = ast.unparse(b200.translate_file(str(DATA / f"{stem}.mlir"))) + "\n"
    assert actual == (GOLDEN / f"{stem}_b200.py").read_text()


@pytest.mark.parametrize("stem", STEMS)
def test_printer_round_trip(stem):
    module = parse_mlir_module(str(DATA / f"{stem}.mlir"), pass_pipeline=passes.PASS_PIPELINE)
    again = ht.parse_module(ht.print_module(module))
    assert ast.unparse(b200.Translator().translate(again)) == ast.unparse(b200.Translator().translate(module))


def test_dot_transpose_to_load_order_pass():
    """Same post-conditions as the reference asserts on mlir-opt's output."""
    module = parse_mlir_module(str(DATA / "attention_f16_1x32x4096x128.mlir"), pass_pipeline=passes.PASS_PIPELINE)
    text = ht.print_module(module)
    assert "transpose_b" not in text
    assert "htile.permute" not in text
    assert "dimension_order = array<i64: 1, 0>" in text
    dots = [l.strip() for l in text.splitlines() if "htile.dot" in l]
    assert len(dots) == 2
    # the QK^T dot now reads a K tile typed 128x64 (D x BN), as in tests/test_translators.py:252-257
    assert ('{warp_policy = "full_row"} : '
            "tensor<128x128xf16, #htile.encoding<placement = shared>>, "
            "tensor<128x64xf16, #htile.encoding<placement = shared>>") in dots[0]
    loads = [op for op in module.walk() if op.name == "htile.load"]
    assert len(loads) == 3  # the original K load was erased


def test_pass_composes_existing_dimension_order_and_rejects_rank3():
    text = """
    #shared = #htile.encoding<placement = shared>
    func.func @f(%a: memref<4x8x16xf16>) {
      %c0 = arith.constant 0 : index
      %t = htile.load %a[%c0, %c0, %c0] {dimension_order = array<i64: 1, 0>} : memref<4x8x16xf16> -> tensor<16x8xf16, #shared>
      %u = htile.permute %t permutation [1, 0] : tensor<16x8xf16, #shared> -> tensor<8x16xf16, #shared>
      %d = htile.dot %u, %t : tensor<8x16xf16, #shared>, tensor<16x8xf16, #shared> -> tensor<8x8xf32, #shared>
      return
    }
    """
    module = passes.dot_transpose_to_load_order(ht.parse_module(text))
    orders = [op.attributes["dimension_order"] for op in module.walk() if op.name == "htile.load"]
    assert [0, 1] in orders and [1, 0] in orders  # composed (1,0)o(1,0) = identity; original kept (still used)
    bad = text.replace("%d = htile.dot %u, %t :", "%d = htile.dot %u, %w {transpose_b} :").replace(
        "return", "").replace(
        "%d = htile.dot", "%w = htile.load %a[%c0, %c0, %c0] : memref<4x8x16xf16> -> tensor<4x8x16xf16, #shared>\n      %d = htile.dot")
    bad = bad.replace("tensor<8x16xf16, #shared>, tensor<16x8xf16, #shared> -> tensor<8x8xf32, #shared>",
                      "tensor<8x16xf16, #shared>, tensor<4x8x16xf16, #shared> -> tensor<8x8xf32, #shared>\n      return")
    with pytest.raises(passes.PassError, match="rank-2"):
        passes.dot_transpose_to_load_order(ht.parse_module(bad))


def test_b200_rejects_unfissioned_dot_transpose():
    with pytest.raises(NotImplementedError, match="htile-dot-transpose-to-load-order"):
        translate_file_with(str(DATA / "attention_f16_1x32x4096x128.mlir"), b200.Translator)


def test_unknown_operation_is_an_error_not_a_todo():
    text = programs.attention_htile("f", 1, 1, 128, 64, "f16").replace("math.exp2 %dm", "math.cos %dm")
    with pytest.raises(ht.HTileSyntaxError, match="unsupported operation 'math.cos'"):
        ht.parse_module(text)


@pytest.mark.parametrize("mutation, reason", [
    (("kind \"sum\"", "kind \"max\""), "rowsum"),
    (("%l_scaled = arith.mulf %l, %alpha", "%l_scaled = arith.addf %l, %alpha"), "l'"),
    (("arith.constant 0.0 : f32", "arith.constant 1.0 : f32"), "start at zero"),
    (("%gz = %batch", "%gz = %heads"), "grid"),
])
def test_b200_rejects_programs_that_are_not_the_recurrence(mutation, reason, tmp_path):
    text = programs.attention_htile("f", 2, 3, 256, 128, "bf16", causal=True).replace(*mutation)
    path = tmp_path / "m.mlir"
    path.write_text(text)
    with pytest.raises(NotImplementedError, match=reason):
        b200.translate_file(str(path))


def test_b200_reads_shapes_scale_and_causality(tmp_path):
    for kw in (dict(B=2, H=3, S=512, D=128, dtype="bf16", causal=True, tile_m=128, tile_n=128),
               dict(B=1, H=1, S=128, D=64, dtype="f32", causal=False, tile_m=64, tile_n=32)):
        path = tmp_path / "p.mlir"
        path.write_text(programs.attention_htile("attn", **kw))
        src = ast.unparse(b200.translate_file(str(path)))
        assert f"shape=({kw['B']}, {kw['H']}, {kw['S']}, {kw['D']})" in src
        assert f"causal={kw['causal']}" in src and f"dtype='{kw['dtype']}'" in src


def test_operator_declarations_check_their_signatures(tmp_path):
    good = programs.decode_splitk_decl("d", 2, 8, 2, 1024, 128, 4)
    path = tmp_path / "d.mlir"
    path.write_text(good)
    assert "n_splits=4" in ast.unparse(b200.translate_file(str(path)))
    path.write_text(good.replace("memref<2x8x4x130xf32>", "memref<2x8x4x128xf32>"))
    with pytest.raises(NotImplementedError, match="partials"):
        b200.translate_file(str(path))
    path.write_text(good.replace('"decode_splitk"', '"conv2d"'))
    with pytest.raises(NotImplementedError, match="unknown htile.operator"):
        b200.translate_file(str(path))


def test_paged_decode_declaration(tmp_path, monkeypatch):
    text = programs.decode_paged_decl("dp", 7, 8, 2, 117, 16, 128, 3)
    path = tmp_path / "dp.mlir"
    path.write_text(text)
    sources = []
    for front in ("native", "python"):
        monkeypatch.setenv("NEPTUNE_HTILE_FRONT", front)
        sources.append(ast.unparse(b200.translate_file(str(path))))
    assert sources[0] == sources[1]
    assert "nb200.decode_paged(ptr_0, ptr_1, ptr_2, ptr_3, ptr_4, ptr_5, ptr_6, B=7, Hq=8, Hkv=2, max_pages=16, " \
           "page_size=64, D=128, n_splits=3, dtype='bf16'" in sources[0]
    path.write_text(text.replace("memref<7x16xi32>", "memref<7x16xi64>"))
    with pytest.raises(NotImplementedError, match="block_table"):
        b200.translate_file(str(path))


def test_decode_program_spelled_in_htile_ops_is_recognised(tmp_path):
    """Split-K decode + combine written with load / dot / reduce / exp2 / unsqueeze / store (two gpu.launch regions)
    maps to the same call as the operator declaration; edits that change its meaning are refused."""
    good = programs.decode_splitk_htile("dec", 2, 8, 2, 1024, 128, 4)
    path = tmp_path / "dec.mlir"
    path.write_text(good)
    src = ast.unparse(b200.translate_file(str(path)))
    assert "nb200.decode_splitk(ptr_0, ptr_1, ptr_2, ptr_3, ptr_4, B=2, Hq=8, Hkv=2, L=1024, D=128, n_splits=4, " \
           "dtype='bf16', scale_log2=0.127517431974411)" in src
    decl = tmp_path / "decl.mlir"
    decl.write_text(programs.decode_splitk_decl("dec", 2, 8, 2, 1024, 128, 4))
    assert ast.unparse(b200.translate_file(str(decl))).replace("0.1275174286422308", "X") == src.replace("0.127517431974411", "X")
    for old, new, why in (
            ("%col_l = arith.constant 129 : index", "%col_l = arith.constant 128 : index", "columns 0"),      # l stored over m
            ("in (%gx = %splits, %gy = %kv_heads, %gz = %batch)", "in (%gx = %kv_heads, %gy = %splits, %gz = %batch)", "grid"),
            ('%den = htile.reduce %wl axis 0 kind "sum"', '%den = htile.reduce %wl axis 0 kind "max"', "out = sum_s"),
            ("%r0 = arith.addi %t0, %j0 : index", "%r0 = arith.addi %j0, %j0 : index", "K tile"),
            ("%l_new = arith.addf %l_scaled, %p_sum", "%l_new = arith.addf %l, %p_sum", "l' = l"),
    ):
        assert old in good
        path.write_text(good.replace(old, new))
        with pytest.raises(NotImplementedError, match=why):
            b200.translate_file(str(path))


def test_syntax_errors_surface_as_runtime_error(tmp_path):
    path = tmp_path / "bad.mlir"
    path.write_text("func.func @f(%a: memref<?x4xf16>) { return }")
    with pytest.raises(RuntimeError, match="HTile front end failed"):
        parse_mlir_module(str(path))


@pytest.mark.skipif(not REFERENCE_PROGRAM.exists(), reason="reference tree not present")
def test_reference_program_translates():
    src = ast.unparse(b200.translate_file(str(REFERENCE_PROGRAM)))
    assert "def flash_attention_htile(ptr_0, ptr_1, ptr_2, ptr_3):" in src
    assert "shape=(1, 32, 4096, 128), kv_len=4096, dtype='f16', scale_log2=0.12751743082459868, causal=False" in src


@pytest.mark.skipif(not REFERENCE_PROGRAM.exists(), reason="reference tree not present")
def test_unmodified_reference_translators_reproduce_their_own_goldens():
    """The strongest pin of the front end: the reference's Triton, TileLang and cuTile translators, imported
    unmodified and fed by this build's HTile reader (the C++ one and the Python twin) plus the dot-transpose pass
    through the ``mlir.ir`` stand-in, emit the reference's three golden texts byte for byte
    (tests/golden/flash_attention_{triton,tilelang,cutile}.py of the reference); and the emitted modules stored
    for the benchmark's reference arm are what those translators emit today.  Runs in a child process because the
    generator switches Triton to its interpreter."""
    import subprocess
    import sys

    script = Path(__file__).parent / "golden" / "make_reference_translations.py"
    ref_root = REFERENCE_PROGRAM.parents[2]
    res = subprocess.run([sys.executable, str(script), str(ref_root), "--check-only"], capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("byte for byte") == 6          # three goldens x two front ends
    assert res.stdout.count("is current") == 3


def test_cli_prints_module(capsys, monkeypatch):
    monkeypatch.setattr("sys.argv", ["neptune-b200", str(DATA / "selective_scan_bf16_8x4096x4096.mlir")])
    b200.main()
    assert "nb200.selective_scan(" in capsys.readouterr().out
