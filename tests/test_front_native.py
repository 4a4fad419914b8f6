"""The C++ HTile front end (libhtile_front.so) against the Python reader, over the program corpus."""

import ctypes
import re
from pathlib import Path

import pytest

from neptune_mlir import htile_native as hn
from neptune_mlir import htile_text as ht
from neptune_mlir import passes, programs

ROOT = Path(__file__).resolve().parents[1]
DATA = sorted((ROOT / "tests" / "data").glob("*.mlir"))
HEADER = ROOT / "include" / "htile_front.h"


def _built_programs():
    yield "attention_nc", programs.attention_htile("a", 2, 4, 512, 128, "f16", causal=False)
    yield "attention_causal", programs.attention_htile("b", 1, 4, 256, 64, "f32", causal=True)
    yield "decode", programs.decode_splitk_decl("d", 2, 8, 2, 1024, 128, 4)
    yield "decode_htile", programs.decode_splitk_htile("dh", 2, 8, 2, 1024, 128, 4)
    yield "decode_htile_f16", programs.decode_splitk_htile("dh16", 1, 16, 2, 2048, 128, 8, "f16", tile_n=128)
    yield "scan", programs.selective_scan_decl("s", 2, 64, 256, 16)
    yield "ssd", programs.ssd_chunk_scan_decl("m", 1, 512, 4, 64, 128, 1, 256, 16)


def test_library_exports_every_declared_symbol(native_lib):
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    declared = sorted(set(re.findall(r"\b(htf_\w+)\s*\(", text)))
    assert declared == sorted(hn.SYMBOLS)
    cdll = ctypes.CDLL(str(hn.find_front_path()))
    for name in declared:
        assert hasattr(cdll, name)
    assert hn.load().htf_version() >= 100


@pytest.mark.parametrize("path", DATA, ids=lambda p: p.stem)
def test_same_object_model_as_the_python_reader(native_lib, path):
    text = path.read_text()
    assert ht.print_module(hn.parse_module(text)) == ht.print_module(ht.parse_module(text))
    want = ht.print_module(passes.run_pipeline(ht.parse_module(text), passes.PASS_PIPELINE))
    assert ht.print_module(hn.parse_module(text, passes.PASS_PIPELINE)) == want
    with hn.NativeModule(text) as nm:  # the C++ printer writes what the Python printer writes
        assert nm.text() == ht.print_module(ht.parse_module(text))


def test_generated_programs_and_value_identity(native_lib):
    for name, text in _built_programs():
        nat, py = hn.parse_module(text), ht.parse_module(text)
        assert ht.print_module(nat) == ht.print_module(py), name
        # operands are the very objects that were defined (the translators key dictionaries on identity)
        defined = {id(v) for fn in nat.functions for v in fn.arguments}
        for op in nat.walk():
            for region in op.regions:
                defined.update(id(a) for a in region.arguments)
            assert all(id(v) in defined for v in op.operands), (name, op.name)
            defined.update(id(r) for r in op.results)
            assert all(r.owner is op for r in op.results)


def test_pass_post_conditions_of_the_reference(native_lib):
    """tests/test_translators.py:250-257 of the reference: no transpose attribute survives, the K load carries
    dimension_order [1, 0] and the transposed tile type."""
    text = (ROOT / "tests" / "data" / "attention_f16_1x32x4096x128.mlir").read_text()
    mod = hn.parse_module(text, passes.PASS_PIPELINE)
    dots = [op for op in mod.walk() if op.name == "htile.dot"]
    assert dots and all("transpose_a" not in d.attributes and "transpose_b" not in d.attributes for d in dots)
    loads = [op for op in mod.walk() if op.name == "htile.load" and op.attributes.get("dimension_order") == [1, 0]]
    assert len(loads) == 1 and loads[0].result.type.shape == (128, 64)
    assert not [op for op in mod.walk() if op.name == "htile.permute"]


@pytest.mark.parametrize("text, message", [
    ("func.func @f(%a: memref<4xf32>) {\n  %x = arith.addf %a, %nope : f32\n  return\n}", "undefined value %nope"),
    ("func.func @f() {\n  %x = foo.bar : f32\n  return\n}", "unsupported operation 'foo.bar'"),
    ("func.func @f(%a: memref<?x4xf32>) {\n  return\n}", "malformed shape"),
    ("func.func @f(%a: tensor<4xf32, #nope>) {\n  return\n}", "unknown tensor encoding"),
])
def test_syntax_errors_carry_line_and_reason(native_lib, text, message):
    with pytest.raises(ht.HTileSyntaxError, match=message) as native_err:
        hn.parse_module(text)
    with pytest.raises(ht.HTileSyntaxError, match=message) as python_err:
        ht.parse_module(text)
    assert str(native_err.value).split(":")[0] == str(python_err.value).split(":")[0]  # same line number


_HEAD = """#shared = #htile.encoding<placement = shared>
#local = #htile.encoding<placement = local>
func.func @f(%m: memref<1x4x256x64xf16>, %i: index) {
"""


@pytest.mark.parametrize("body, message", [
    ("%a = htile.load %m[%i, %i, %i, %i] : memref<1x4x256x64xf16> -> tensor<128x64xf16, #shared>\n"
     "%b = htile.load %m[%i, %i, %i, %i] : memref<1x4x256x64xf16> -> tensor<64x64xf16, #shared>\n"
     "%c = htile.dot %a, %b : tensor<128x64xf16, #shared>, tensor<64x64xf16, #shared> -> tensor<128x128xf32, #local>",
     "htile.dot: result must be 128x64"),
    ("%a = htile.load %m[%i, %i, %i] : memref<1x4x256x64xf16> -> tensor<128x64xf16, #shared>",
     "htile.load: expects one offset per memref dimension"),
    ("%a = htile.load %m[%i, %i, %i, %i] {dimension_order = array<i64: 1, 1>} : memref<1x4x256x64xf16> -> tensor<64x128xf16, #shared>",
     "dimension_order is not a permutation"),
    ("%a = htile.load %m[%i, %i, %i, %i] : memref<1x4x256x64xf16> -> tensor<128x64xf16, #shared>\n"
     '%r = htile.reduce %a axis 2 kind "max" : tensor<128x64xf16, #shared> -> tensor<128xf16, #local>',
     "htile.reduce: axis out of range"),
    ("%a = htile.load %m[%i, %i, %i, %i] : memref<1x4x256x64xf16> -> tensor<128x64xf16, #shared>\n"
     "%p = htile.permute %a permutation [1, 0] : tensor<128x64xf16, #shared> -> tensor<128x64xf16, #shared>",
     "htile.permute: result shape does not follow the permutation"),
])
def test_verifier_rejects_malformed_htile_ops(native_lib, body, message):
    text = _HEAD + body + "\n  return\n}\n"
    ht.parse_module(text)  # syntactically fine
    with pytest.raises(ht.HTileSyntaxError, match=re.escape(message)):
        hn.parse_module(text)


def test_unknown_pass_is_refused(native_lib):
    with pytest.raises(passes.PassError, match="unknown pass 'inline'"):
        hn.parse_module((ROOT / "tests" / "data" / "attention_f16_1x32x4096x128.mlir").read_text(),
                        "builtin.module(inline)")


def test_translators_use_the_native_front_end_by_default(native_lib, monkeypatch):
    from neptune_mlir.translators import b200, common
    import ast

    monkeypatch.delenv("NEPTUNE_HTILE_FRONT", raising=False)
    assert common.front_end() == "native"
    path = str(ROOT / "tests" / "data" / "attention_causal_bf16_8x32x4096x128.mlir")
    native_src = ast.unparse(b200.translate_file(path))
    monkeypatch.setenv("NEPTUNE_HTILE_FRONT", "python")
    assert common.front_end() == "python"
    assert ast.unparse(b200.translate_file(path)) == native_src
    monkeypatch.setenv("NEPTUNE_HTILE_FRONT", "fortran")
    with pytest.raises(ValueError):
        common.front_end()
