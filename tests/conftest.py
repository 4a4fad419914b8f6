"""Test configuration: import paths, the `gpu` marker, and an in-tree build of the kernel library."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "mlir-toy_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def native_lib():
    """Path of libnb200.so, building it (nvcc) and the HTile front end (g++) if either is not there yet; no GPU
    is needed to build."""
    from neptune_mlir.plugin import find_front_path, find_library_path

    path = find_library_path()
    if path is None or find_front_path() is None:
        import importlib.util

        spec = importlib.util.spec_from_file_location("nb200_build_native", PKG / "build_native.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        path = mod.build()
    return path


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked `gpu` ran without a CUDA device")
    return torch.device("cuda", 0)
