#!/usr/bin/env python3
"""Build libnb200.so (the sm_100a kernel library) in-tree with nvcc.

Every .cu under csrc/ is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``; plain ``-arch=sm_100a`` assembles for sm_100 in some
toolkits and rejects tcgen05) and linked, with a static CUDA runtime, into
``neptune_mlir/_native/libnb200.so`` -- the first place the loader looks
(neptune_mlir.plugin.find_library_path).  Objects are rebuilt only when a source or header is newer.

    python mlir-toy_b200/build_native.py [--force] [--verbose]
"""

from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
OBJ_DIR = PKG / "build"
OUT = PKG / "neptune_mlir" / "_native" / "libnb200.so"
FRONT_SRC = CSRC / "htile_front" / "htile_front.cpp"
FRONT_OUT = PKG / "neptune_mlir" / "_native" / "libhtile_front.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    f"-I{INCLUDE}", f"-I{CSRC}",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the nb200 kernel library cannot be built")
    return exe


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def _compile(src: Path, obj: Path, verbose: bool) -> str:
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    log = res.stderr
    (obj.with_suffix(".ptxas.txt")).write_text(log)
    if verbose:
        print(log)
    return log


def build_front(force: bool = False) -> Path:
    """The HTile front end: host C++ only (g++), a shared library of its own next to the kernel library."""
    FRONT_OUT.parent.mkdir(parents=True, exist_ok=True)
    newest = max(FRONT_SRC.stat().st_mtime, (INCLUDE / "htile_front.h").stat().st_mtime)
    if force or not FRONT_OUT.exists() or FRONT_OUT.stat().st_mtime < newest:
        gxx = shutil.which("g++") or shutil.which("c++")
        if gxx is None:
            raise RuntimeError("g++ not found; the HTile front end cannot be built")
        cmd = [gxx, "-O2", "-std=c++17", "-Wall", "-Wextra", "-shared", "-fPIC", f"-I{INCLUDE}", "-o", str(FRONT_OUT),
               str(FRONT_SRC)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"g++ failed on {FRONT_SRC.name}:\n{res.stdout}\n{res.stderr}")
    return FRONT_OUT


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    OUT.parent.mkdir(parents=True, exist_ok=True)
    build_front(force)
    sources = sorted(CSRC.glob("*.cu"))
    hdr_time = max(_newest_header(), Path(__file__).stat().st_mtime)
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for fut in [ex.submit(_compile, s, o, verbose) for s, o in jobs]:
                fut.result()
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    if jobs or not OUT.exists() or any(o.stat().st_mtime > OUT.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
               "-o", str(OUT), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return OUT


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(args.force, args.verbose))


if __name__ == "__main__":
    sys.exit(main())
