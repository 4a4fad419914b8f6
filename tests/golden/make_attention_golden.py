#!/usr/bin/env python3
"""Generate tests/golden/flash_attention_ref_tiles.npz from the reference's own translation.

The reference's golden Triton kernel (tests/golden/flash_attention_triton.py in the reference tree:
the byte-exact output of its Triton translator for tests/data/flash_attention_htile.mlir) is run on
CPU tensors by the Triton interpreter (TRITON_INTERPRET=1).  Shape, dtype and non-causality are
baked into that kernel (1 x 32 x 4096 x 128, f16).  A handful of programs (one 128-row query block
of one head each) are evaluated; a program is selected by offsetting the tensor base pointers so
that program id (0, 0, 0) lands on the wanted head and row block.

Inputs come from oracle.inputs.attention_inputs(..., config=0); their SHA-256 is stored with the
tiles so that a consumer can tell whether it regenerated the same bits.

Usage (needs the reference tree; run from the repository root):
    python tests/golden/make_attention_golden.py /path/to/reference
"""

import hashlib
import importlib.util
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle.inputs import attention_inputs  # noqa: E402

SHAPE = (1, 32, 4096, 128)
PROGRAMS = [(0, 0), (0, 31), (17, 5), (31, 13)]  # (head, 128-row block)


def sha(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.int16).numpy().tobytes())
    return h.hexdigest()


def main() -> None:
    if len(sys.argv) < 2 and "NEPTUNE_REFERENCE_ROOT" not in os.environ:
        raise SystemExit(__doc__)
    ref_root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["NEPTUNE_REFERENCE_ROOT"])
    spec = importlib.util.spec_from_file_location(
        "ref_flash_attention_triton", ref_root / "tests" / "golden" / "flash_attention_triton.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    q, k, v = attention_inputs(*SHAPE, torch.float16, config=0)
    out = torch.zeros(SHAPE, dtype=torch.float16)
    tiles = []
    for head, blk in PROGRAMS:
        r0 = blk * 128
        # pid = (0,0,0): Q/out bases moved to (head, r0); K/V bases moved to the head.
        mod.flash_attention_htile[(1, 1, 1)](
            q[0, head, r0:], k[0, head], v[0, head], out[0, head, r0:])
        tiles.append(out[0, head, r0:r0 + 128].clone().numpy())
    np.savez_compressed(
        Path(__file__).with_name("flash_attention_ref_tiles.npz"),
        programs=np.array(PROGRAMS, dtype=np.int32),
        tiles=np.stack(tiles),
        inputs_sha256=np.array(sha(q, k, v)),
        shape=np.array(SHAPE, dtype=np.int32),
    )
    print("wrote", len(tiles), "tiles; inputs sha256", sha(q, k, v))


if __name__ == "__main__":
    main()
