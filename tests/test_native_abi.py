"""The C-ABI library loads without a GPU, exports what include/nb200.h declares, and rejects bad calls."""

import ctypes
import re
from pathlib import Path

import pytest

from neptune_mlir import native, plugin

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "nb200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(nb200_\w+)\s*\(", text)))


def test_header_and_binding_list_the_same_symbols():
    assert declared_symbols() == sorted(native.SYMBOLS)


def test_library_exports_every_declared_symbol(native_lib):
    cdll = ctypes.CDLL(str(native_lib))
    for name in declared_symbols():
        assert hasattr(cdll, name), f"{native_lib} does not export {name}"


def test_loader_resolution_order(native_lib, tmp_path, monkeypatch):
    assert plugin.find_library_path() == Path(native_lib).resolve()
    fake = tmp_path / "libnb200.so"
    fake.write_bytes(b"")
    monkeypatch.setenv(plugin.DEFAULT_LIBRARY_ENV, str(fake))
    assert plugin.find_library_path() == fake.resolve()                      # env beats the package dir
    other = tmp_path / "explicit.so"
    other.write_bytes(b"")
    assert plugin.find_library_path(str(other)) == other.resolve()           # explicit beats env
    assert plugin.find_plugin_path() is None or plugin.find_plugin_path().name.startswith("libHTileDialectPlugin")


def test_missing_library_raises(monkeypatch):
    monkeypatch.setattr(native, "find_library_path", lambda path=None: None)
    monkeypatch.setattr(native, "_LIB", None)
    with pytest.raises(native.NativeLibraryError, match="no CPU or PyTorch fallback"):
        native.lib()


def test_version_and_argument_errors_without_a_gpu(native_lib):
    lib = native.load(str(native_lib))
    assert lib.nb200_version() >= 100
    rc = lib.nb200_attn_fwd(None, None, None, None, 1, 1, 128, 128, 128, 1, 0.1, 0, None, None)
    assert rc == -1 and b"null pointer" in lib.nb200_last_error()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    p += (-p) % 16
    rc = lib.nb200_decode_splitk(p, p, p, p, 1, 8, 2, 1024, 64, 4, 1, 0.1, None, None)
    assert rc == -2 and b"only 128" in lib.nb200_last_error()
    rc = lib.nb200_decode_splitk(p, p, p, p, 1, 8, 3, 1024, 128, 4, 1, 0.1, None, None)
    assert rc == -2
    rc = lib.nb200_selective_scan_fwd(p, p, p, p, p, p, p, p, 1, 64, 100, 16, 1, None)
    assert rc == -2 and b"multiple of 64" in lib.nb200_last_error()
    rc = lib.nb200_ssd_chunk_scan_fwd(p, p, p, p, p, p, p, 1, 256, 4, 32, 128, 1, 64, 1, None)
    assert rc == -2
    rc = lib.nb200_attn_fwd(p, p, p, p, 1, 1, 128, 64, 128, 1, 0.1, 1, None, None)
    assert rc == -2 and b"causal" in lib.nb200_last_error()
    with pytest.raises(NotImplementedError):
        native.check(rc, "attn")


def test_nccl_merge_rejects_bad_calls_without_a_gpu(native_lib):
    lib = native.load(str(native_lib))
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    p += (-p) % 16
    assert lib.nb200_decode_merge_workspace_bytes(32, 128, 8) == 8 * 32 * 130 * 4
    assert lib.nb200_decode_merge_workspace_bytes(0, 128, 8) == 0
    rc = lib.nb200_decode_merge_nccl(p, p, p, 32, 128, 2, 1, None, None)
    assert rc == -1 and b"null communicator" in lib.nb200_last_error()
    rc = lib.nb200_decode_merge_nccl(p, p, p, 32, 64, 2, 1, p, None)
    assert rc == -2 and b"only 128" in lib.nb200_last_error()
    rc = lib.nb200_decode_merge_nccl(None, p, p, 32, 128, 2, 1, p, None)
    assert rc == -1


def test_paged_decode_rejects_bad_calls_without_a_gpu(native_lib):
    lib = native.load(str(native_lib))
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    p += (-p) % 16
    rc = lib.nb200_decode_paged_splitk(p, p, p, p, p, p, 2, 8, 2, 40, 16, 32, 128, 4, 1, 0.1, None, None)
    assert rc == -2 and b"only 64 rows per page" in lib.nb200_last_error()
    rc = lib.nb200_decode_paged_splitk(p, p, p, None, p, p, 2, 8, 2, 40, 16, 64, 128, 4, 1, 0.1, None, None)
    assert rc == -1
    rc = lib.nb200_decode_paged_splitk(p, p, p, p, p, p, 2, 8, 3, 40, 16, 64, 128, 4, 1, 0.1, None, None)
    assert rc == -2


def test_combine_and_static_decode_reject_a_misaligned_output_without_a_gpu(native_lib):
    """16-bit outputs are written four elements (8 bytes) at a time: an output that starts at an odd element is
    refused on the host instead of faulting on the device."""
    lib = native.load(str(native_lib))
    buf = ctypes.create_string_buffer(128)
    p = ctypes.addressof(buf)
    p += (-p) % 16
    rc = lib.nb200_decode_combine(p, p + 2, 8, 128, 4, 4 * 130, 130, 1, None)
    assert rc == -1 and b"out must be 8-byte aligned" in lib.nb200_last_error()
    rc = lib.nb200_decode_combine(p, p + 2, 8, 128, 4, 4 * 130, 130, 2, None)
    assert rc == -1 and b"out must be 4-byte aligned" in lib.nb200_last_error()
    rc = lib.nb200_decode_fwd_static(p, p, p, p + 4, 1, 8, 2, 1024, 128, 4, 1, 0.1, None)
    assert rc == -1 and b"out must be 8-byte aligned" in lib.nb200_last_error()
    assert lib.nb200_decode_auto_splits(0, 8, 1024, 0) == 0


def test_nccl_communicator_argument_checks():
    from neptune_mlir import nccl_comm
    with pytest.raises(ValueError, match="128 bytes"):
        nccl_comm.Communicator(0, 2, b"short")
    with pytest.raises(ValueError, match="outside world"):
        nccl_comm.Communicator(2, 2, bytes(128))


def test_workspace_sizes(native_lib):
    lib = native.load(str(native_lib))
    assert lib.nb200_decode_workspace_bytes(64, 32, 128, 16) == 64 * 32 * 16 * 130 * 4
    # status words (padded to 256) + at most 512 CTAs' worth of segments: 4 per sequence here, 3 hand-over slots
    # of one total (fp32) and one 128 x 64 fp32 state per (batch, head)
    slots = 4 * 64 * 3
    assert lib.nb200_ssd_workspace_bytes(4, 8192, 64, 64, 128, 1, 256) == 256 + slots * 4 + slots * 8192 * 4
    assert lib.nb200_ssd_workspace_bytes(64, 8192, 64, 64, 128, 1, 256) == 256     # enough chains: never cut
    assert lib.nb200_ssd_workspace_bytes(4, 8192, 64, 32, 128, 1, 256) == 0


def test_runtime_rejects_cpu_tensors(native_lib):
    import torch

    from neptune_mlir import runtime

    t = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA tensor"):
        runtime.attn_fwd(t, t, t, t, shape=(1, 1, 128, 128), kv_len=128, dtype="bf16", scale_log2=0.1, causal=False)
    with pytest.raises(TypeError, match="torch.Tensor"):
        runtime.attn_fwd(1, t, t, t, shape=(1, 1, 128, 128), kv_len=128, dtype="bf16", scale_log2=0.1, causal=False)


def test_torch_library_ops_are_registered_and_refuse_cpu_tensors(native_lib):
    import torch

    from neptune_mlir import torch_ops

    for name in torch_ops.OPS:
        assert hasattr(torch.ops.nb200, name)
    q = torch.zeros((1, 1, 128, 128), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA tensor"):
        torch.ops.nb200.attn_fwd(q, q, q, torch.empty_like(q), 0.1, True)
