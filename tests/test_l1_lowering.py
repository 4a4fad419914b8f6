"""Level-1 (scheduled tile IR) -> HTile lowering (neptune_mlir.l1)."""

import ast
import os
from collections import Counter
from pathlib import Path

import pytest

from neptune_mlir import htile_native, htile_text, l1, passes, programs
from neptune_mlir.translators import b200

# the reference project's tree, when it is available ($NEPTUNE_REFERENCE_ROOT, else a sibling "reference" directory)
REFERENCE_ROOT = Path(os.environ.get("NEPTUNE_REFERENCE_ROOT", Path(__file__).resolve().parents[2] / "reference"))
REFERENCE_L1 = REFERENCE_ROOT / "tests" / "data" / "flash_attention_l1.mlir"
REFERENCE_HTILE = REFERENCE_ROOT / "tests" / "data" / "flash_attention_htile.mlir"


def _translate_text(tmp_path, text, name="p.mlir"):
    path = tmp_path / name
    path.write_text(text)
    return ast.unparse(b200.translate_file(str(path)))


def _htile_ops(text):
    module = htile_text.parse_module(text)
    return Counter(op.name for op in module.walk() if op.name.startswith("htile.") or op.name in ("scf.for", "gpu.launch"))


@pytest.mark.skipif(not REFERENCE_L1.exists(), reason="reference tree not present")
def test_reference_l1_program_lowers_to_the_program_the_target_accepts(tmp_path):
    """The reference's own Level-1 file lowers to HTile that (a) both front ends read and verify, (b) uses the same
    HTile operations as the reference's hand-written HTile program for the same schedule, and (c) the B200
    translator recognises with the reference's shape and the file's own scale constant."""
    text = l1.lower_file(REFERENCE_L1)
    htile_native.parse_module(text, passes.PASS_PIPELINE)          # C++ front end: reads, verifies, rewrites
    assert _htile_ops(text) == _htile_ops(REFERENCE_HTILE.read_text())
    src = _translate_text(tmp_path, text)
    assert "def flash_attention(ptr_0, ptr_1, ptr_2, ptr_3):" in src
    assert "shape=(1, 32, 4096, 128), kv_len=4096, dtype='f16', scale_log2=0.12751743082459868, causal=False" in src
    # and through the one-call entry point
    assert ast.unparse(l1.translate_file(str(REFERENCE_L1))) == src


@pytest.mark.parametrize("B,H,S,D,dtype,tm,tn", [(2, 4, 512, 128, "f16", 128, 64), (1, 4, 256, 64, "f32", 128, 64),
                                                 (8, 32, 4096, 128, "bf16", 128, 128)])
def test_generated_l1_programs_lower_and_translate(tmp_path, B, H, S, D, dtype, tm, tn):
    text = l1.lower_to_htile(programs.attention_l1("attn_l1", B, H, S, D, dtype, tile_m=tm, tile_n=tn))
    module = htile_text.parse_module(text)                         # the Python reader accepts it too
    passes.dot_transpose_to_load_order(module)
    ops = _htile_ops(text)
    assert ops["htile.load"] == 3 and ops["htile.dot"] == 2 and ops["htile.reduce"] == 2 and ops["htile.store"] == 1
    src = _translate_text(tmp_path, text)
    assert f"shape=({B}, {H}, {S}, {D}), kv_len={S}, dtype='{dtype}'" in src and "causal=False" in src
    # the same schedule written directly in HTile translates to the same call (up to the f32 rounding of the scale)
    direct = _translate_text(tmp_path, programs.attention_htile("attn_l1", B, H, S, D, dtype, tile_m=tm, tile_n=tn), "d.mlir")
    strip = lambda s: s[:s.index("scale_log2=")]                   # noqa: E731
    assert strip(src) == strip(direct)


def test_placements_and_structure_of_the_lowered_text():
    text = l1.lower_to_htile(programs.attention_l1("a", 1, 2, 256, 128, "f16"))
    assert "gpu.launch blocks(%bx, %by, %bz)" in text and "htile.pipeline_stages = 2 : i32" in text
    loads = [ln for ln in text.splitlines() if "htile.load" in ln]
    assert len(loads) == 3 and all("#shared>" in ln for ln in loads)
    dots = [ln for ln in text.splitlines() if "htile.dot" in ln]
    assert "transpose_b" in dots[0] and "transpose_b" not in dots[1]
    assert "linalg.matmul" not in text and "tensor.extract_slice" not in text and "affine." not in text


def test_unsupported_level1_input_is_refused():
    good = programs.attention_l1("a", 1, 2, 256, 128, "f16")
    with pytest.raises(NotImplementedError, match="not supported"):
        l1.lower_to_htile(good.replace("math.exp2 %shifted", "math.tanh %shifted"))
    with pytest.raises(NotImplementedError, match="d \\* c"):
        l1.lower_to_htile(good.replace("(d) -> (d * 64)", "(d) -> (d + 64)"))
    with pytest.raises(l1.L1SyntaxError):
        l1.lower_to_htile(good.replace("scf.forall (%b, %h, %blk) in", "scf.forall (%b, %h, %blk) of"))
    with pytest.raises(NotImplementedError, match="exactly one scf.forall"):
        l1.lower_to_htile("module { func.func @f(%q: tensor<4xf16>) -> tensor<4xf16> { return %q : tensor<4xf16> } }")


def test_cli_prints_htile(tmp_path, capsys, monkeypatch):
    path = tmp_path / "p.mlir"
    path.write_text(programs.attention_l1("a", 1, 2, 256, 128, "f16"))
    monkeypatch.setattr("sys.argv", ["neptune-l1", str(path)])
    l1.main()
    assert "htile.store" in capsys.readouterr().out
