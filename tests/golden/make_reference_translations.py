#!/usr/bin/env python3
"""Pin attention at shapes and element types the reference never tested, with the reference's own translator.

The reference's Triton translator (src/neptune_mlir/translators/triton.py in the reference tree) is
imported UNMODIFIED, under the module name ``ref_neptune_mlir`` and with the ``mlir`` stand-in of
``tests/golden/mlir_standin`` in place of the LLVM bindings it wants.  HTile text is read and rewritten
(dot-transpose pass) by this build's C++ front end (``neptune_mlir.htile_native``) -- and, as a second
check, by the Python reader and pass -- wrapped in the stand-in's object model and handed to
``Translator().translate``.

1. Check of the stand-in: the reference's own program (tests/data/flash_attention_htile.mlir) must
   translate to all three of its golden texts (tests/golden/flash_attention_{triton,tilelang,cutile}.py)
   byte for byte -- the Triton and cuTile translators after the dot-transpose pass
   (triton.py:479-487, cutile.py:486-493), the TileLang one without it (tilelang.py:560-561).  The
   reference pipeline also runs ``cse,canonicalize``; its one visible effect on that program is
   that a gpu.launch id whose extent is the constant 1 is replaced by the constant 0, which
   ``fold_unit_launch_ids`` restates.
2. Programs written by ``neptune_mlir.programs.attention_htile`` (non-causal: the reference
   translator has no lowering for the mask ops) are translated the same way, executed by the Triton
   interpreter on CPU tensors over their whole grid, and the outputs stored in
   ``reference_translations.npz`` with the SHA-256 of inputs and of the emitted source.

3. The program of the reference's own shape as this build spells it (tests/data/attention_f16_1x32x4096x128.mlir,
   non-causal f16 1x32x4096x128) is translated by all three reference translators and the emitted modules
   are stored as text under ``reference_emitted/``.  They are outputs of the reference, kept so that the
   benchmark can time the reference's GPU path (Triton / TileLang / cuTile JIT of what its translators emit)
   beside this build's kernel on a machine that has no copy of the reference tree.

Usage (needs the reference tree; run from the repository root):
    python tests/golden/make_reference_translations.py /path/to/reference [--emit-only | --check-only]
"""

import ast
import hashlib
import importlib
import importlib.util
import os
import sys
import tempfile
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "mlir-toy_b200"))
sys.path.insert(0, str(HERE / "mlir_standin"))

import mlir.ir as standin_ir  # noqa: E402  (the stand-in)
from neptune_mlir import htile_native, htile_text, passes, programs  # noqa: E402
from oracle.inputs import attention_inputs  # noqa: E402

# name -> (B, H, S, D, dtype, tile_m, tile_n, config index for the input seeds)
CASES = {
    "f32_1x4x256x64": (1, 4, 256, 64, "f32", 128, 64, 11),
    "f16_2x4x512x128": (2, 4, 512, 128, "f16", 128, 64, 12),
}
TORCH = {"f32": torch.float32, "f16": torch.float16}


def load_reference_translator(ref_root: Path):
    pkg_dir = ref_root / "src" / "neptune_mlir"
    spec = importlib.util.spec_from_file_location("ref_neptune_mlir", pkg_dir / "__init__.py",
                                                  submodule_search_locations=[str(pkg_dir)])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules["ref_neptune_mlir"] = pkg
    spec.loader.exec_module(pkg)
    return {name: importlib.import_module(f"ref_neptune_mlir.translators.{name}")
            for name in ("triton", "tilelang", "cutile")}


def fold_unit_launch_ids(module) -> None:
    """gpu.launch ids of an extent that is the constant 1 are the constant 0 (what canonicalize leaves)."""
    for fn in module.functions:
        consts = {id(op.results[0]): op for op in fn.body.operations if op.name == "arith.constant"}
        zero = next((op.results[0] for op in consts.values()
                     if op.attributes["value"] == 0 and str(op.results[0].type) == "index"), None)
        for op in fn.body.operations:
            if op.name != "gpu.launch" or zero is None:
                continue
            body = op.regions[0]
            for i, extent in enumerate(op.operands[:6]):
                c = consts.get(id(extent))
                if c is not None and c.attributes["value"] == 1:
                    passes._replace_all_uses(module, body.arguments[i], zero)


def translate(ref_translator, text: str, run_pass: bool = True, front: str = "native") -> str:
    if front == "native":   # the C++ front end reads, verifies and rewrites
        module = htile_native.parse_module(text, passes.PASS_PIPELINE if run_pass else None)
    else:                   # the Python reader and pass
        module = htile_text.parse_module(text)
        if run_pass:
            passes.dot_transpose_to_load_order(module)
    fold_unit_launch_ids(module)
    return ast.unparse(ref_translator.Translator().translate(standin_ir.from_htile(module)))


def check_standin(ref, ref_root: Path) -> None:
    text = (ref_root / "tests" / "data" / "flash_attention_htile.mlir").read_text()
    for front in ("native", "python"):
        for name, mod in ref.items():
            got = translate(mod, text, run_pass=(name != "tilelang"), front=front)
            want = (ref_root / "tests" / "golden" / f"flash_attention_{name}.py").read_text()
            if got.strip() != want.strip():
                import difflib
                sys.stdout.writelines(difflib.unified_diff(want.splitlines(True), got.splitlines(True), "golden", "stand-in"))
                raise SystemExit(f"{front} front end + stand-in do not reproduce the reference's golden {name} translation")
            print(f"{front} front end + stand-in reproduce tests/golden/flash_attention_{name}.py byte for byte")


def sha_tensors(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def run_source(source: str, name: str, grid, *tensors) -> None:
    with tempfile.TemporaryDirectory() as tmp:  # triton.jit reads the kernel's source from its file
        path = Path(tmp) / f"{name}.py"
        path.write_text(source + "\n")
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        getattr(mod, name)[grid](*tensors)


EMITTED_PROGRAM = "attention_f16_1x32x4096x128"


def emit_reference_modules(ref, check_only: bool = False) -> None:
    """What the three reference translators emit for this build's spelling of the reference-shape program;
    with ``check_only`` the stored files are compared with it instead of being rewritten."""
    text = (ROOT / "tests" / "data" / f"{EMITTED_PROGRAM}.mlir").read_text()
    out_dir = HERE / "reference_emitted"
    out_dir.mkdir(exist_ok=True)
    for name, mod in ref.items():
        source = translate(mod, text, run_pass=(name != "tilelang"))
        header = (f"# Emitted by the reference project's {name} translator (imported unmodified from the reference tree)\n"
                  f"# for tests/data/{EMITTED_PROGRAM}.mlir; written by tests/golden/make_reference_translations.py.\n"
                  "# Not product code: the benchmark launches it as the reference's own GPU path.\n")
        path = out_dir / f"{EMITTED_PROGRAM}_{name}.py"
        if check_only:
            if path.read_text() != header + source + "\n":
                raise SystemExit(f"reference_emitted/{path.name} is not what the reference's {name} translator emits now")
            print(f"reference_emitted/{path.name} is current")
            continue
        path.write_text(header + source + "\n")
        print(f"wrote reference_emitted/{path.name} ({len(source.splitlines())} lines)")


def main() -> None:
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    if not args and "NEPTUNE_REFERENCE_ROOT" not in os.environ:
        raise SystemExit(__doc__)
    ref_root = Path(args[0] if args else os.environ["NEPTUNE_REFERENCE_ROOT"])
    ref = load_reference_translator(ref_root)
    check_standin(ref, ref_root)
    emit_reference_modules(ref, check_only="--check-only" in sys.argv)
    if "--emit-only" in sys.argv or "--check-only" in sys.argv:
        return
    ref_triton = ref["triton"]

    store = {}
    for name, (B, H, S, D, dtype, tm, tn, cfg) in CASES.items():
        fn_name = f"attn_{name}"
        source = translate(ref_triton, programs.attention_htile(fn_name, B, H, S, D, dtype, causal=False,
                                                                tile_m=tm, tile_n=tn))
        q, k, v = attention_inputs(B, H, S, D, TORCH[dtype], config=cfg)
        out = torch.zeros_like(q)
        run_source(source, fn_name, (S // tm, H, B), q, k, v, out)
        store[f"{name}.out"] = out.numpy()
        store[f"{name}.inputs_sha256"] = np.array(sha_tensors(q, k, v))
        store[f"{name}.source_sha256"] = np.array(hashlib.sha256(source.encode()).hexdigest())
        store[f"{name}.spec"] = np.array([B, H, S, D, tm, tn, cfg], dtype=np.int32)
        print(name, "done; |out| max", float(out.float().abs().max()))
    np.savez_compressed(HERE / "reference_translations.npz", **store)


if __name__ == "__main__":
    main()
