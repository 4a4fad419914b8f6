#!/usr/bin/env python3
"""Regenerate the HTile programs under tests/data/ and their expected translations under tests/golden/.

    python tests/data/make_programs.py

The programs come from neptune_mlir.programs (one per benchmark configuration plus the reference's
own problem shape); the goldens are what neptune_mlir.translators.b200 emits for them, checked
byte for byte by tests/test_frontend.py in the manner of the reference's golden-text tests
(tests/test_translators.py:154-165).
"""

import ast
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "mlir-toy_b200"))

from neptune_mlir import programs  # noqa: E402
from neptune_mlir.translators import b200  # noqa: E402

DATA = Path(__file__).resolve().parent
GOLDEN = ROOT / "tests" / "golden"

from neptune_mlir import native  # noqa: E402

# workspace of the SSD configuration, as the library sizes it (status words plus room for the states that are
# handed from segment to segment when a sequence is cut; see include/nb200.h)
SSD_WS = native.lib().nb200_ssd_workspace_bytes(4, 8192, 64, 64, 128, 1, 256)

PROGRAMS = {
    "attention_f16_1x32x4096x128": programs.attention_htile("attention_f16", 1, 32, 4096, 128, "f16", causal=False),
    "attention_causal_f32_1x4x256x64": programs.attention_htile("attention_causal_f32", 1, 4, 256, 64, "f32", causal=True),
    "attention_causal_bf16_8x32x4096x128": programs.attention_htile("attention_causal_bf16", 8, 32, 4096, 128, "bf16", causal=True),
    "decode_splitk_bf16_64x32x8x32768x128": programs.decode_splitk_decl("decode_splitk_bf16", 64, 32, 8, 32768, 128, 16),
    "decode_splitk_htile_bf16_64x32x8x32768x128": programs.decode_splitk_htile("decode_splitk_htile_bf16", 64, 32, 8, 32768, 128, 16),
    "selective_scan_bf16_8x4096x4096": programs.selective_scan_decl("selective_scan_bf16", 8, 4096, 4096, 16),
    "ssd_chunk_scan_bf16_4x8192x64x64": programs.ssd_chunk_scan_decl("ssd_chunk_scan_bf16", 4, 8192, 64, 64, 128, 1, 256, SSD_WS),
}


def main() -> None:
    for stem, text in PROGRAMS.items():
        path = DATA / f"{stem}.mlir"
        path.write_text(text)
        module = b200.translate_file(str(path))
        (GOLDEN / f"{stem}_b200.py").write_text(ast.unparse(module) + "\n")
        print("wrote", path.name)


if __name__ == "__main__":
    main()
