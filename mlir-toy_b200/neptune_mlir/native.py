"""ctypes binding of the nb200 C ABI (include/nb200.h).

There is no fallback: if the shared library cannot be found or loaded, ``lib()`` raises, and every
operator raises with it.  ``SYMBOLS`` lists every entry point the header declares, with its ctypes
signature, so that a test can check the library exports all of them.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_uint, c_void_p
from pathlib import Path

from .plugin import find_library_path

NB200_OK = 0
ERROR_NAMES = {-1: "bad argument", -2: "unsupported", -3: "launch failure", -4: "device wait timeout", -5: "NCCL failure"}
DTYPE_CODES = {"f16": 0, "bf16": 1, "f32": 2}
STATUS_WORDS = 4

# name -> (restype, argtypes)
SYMBOLS: dict[str, tuple] = {
    "nb200_version": (c_int, []),
    "nb200_last_error": (c_char_p, []),
    "nb200_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_float, c_int, c_void_p, c_void_p]),
    "nb200_status_read": (c_int, [c_void_p, c_void_p, c_void_p]),
    "nb200_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "nb200_decode_splitk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_float, c_void_p, c_void_p]),
    "nb200_decode_auto_splits": (c_int, [c_int, c_int, c_int, c_int]),
    "nb200_decode_paged_splitk": (c_int, [c_void_p] * 6 + [c_int] * 9 + [c_float, c_void_p, c_void_p]),
    "nb200_decode_combine": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
                                     c_void_p]),
    "nb200_decode_merge_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "nb200_decode_merge_nccl": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                        c_void_p]),
    "nb200_decode_merge_peer_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "nb200_decode_merge_peer": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_uint, c_int,
                                        c_longlong, c_void_p, c_void_p]),
    "nb200_decode_sharded_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "nb200_decode_sharded_fwd": (c_int, [c_void_p] * 6 + [c_int] * 6 + [c_float, c_int, c_int, c_uint, c_int, c_longlong,
                                                                       c_void_p, c_void_p]),
    "nb200_peer_buffer_alloc": (c_int, [c_size_t, c_void_p, c_void_p]),
    "nb200_peer_buffer_open": (c_int, [c_void_p, c_void_p]),
    "nb200_peer_buffer_close": (c_int, [c_void_p]),
    "nb200_peer_buffer_free": (c_int, [c_void_p]),
    "nb200_decode_fwd_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_float, c_void_p]),
    "nb200_selective_scan_fwd": (c_int, [c_void_p] * 8 + [c_int] * 5 + [c_void_p]),
    "nb200_ssd_workspace_bytes": (c_size_t, [c_int] * 7),
    "nb200_ssd_launches": (c_int, [c_int] * 7),
    "nb200_ssd_chunk_scan_fwd": (c_int, [c_void_p] * 7 + [c_int] * 8 + [c_void_p]),
}


class NativeLibraryError(RuntimeError):
    """The nb200 shared library is missing, or a call into it failed."""


_LIB: ctypes.CDLL | None = None
_LIB_PATH: Path | None = None


def load(path=None) -> ctypes.CDLL:
    """Load (or reload from an explicit path) the kernel library and declare its prototypes."""
    global _LIB, _LIB_PATH
    resolved = find_library_path(path)
    if resolved is None:
        raise NativeLibraryError(
            "the nb200 kernel library (libnb200.so) was not found; build it with "
            "`python mlir-toy_b200/build_native.py` or point $NEPTUNE_B200_LIB at it. "
            "There is no CPU or PyTorch fallback for the HTile B200 target.")
    if _LIB is not None and _LIB_PATH == resolved:
        return _LIB
    cdll = ctypes.CDLL(str(resolved))
    for name, (restype, argtypes) in SYMBOLS.items():
        try:
            fn = getattr(cdll, name)
        except AttributeError as exc:
            raise NativeLibraryError(f"{resolved} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB, _LIB_PATH = cdll, resolved
    return cdll


def lib() -> ctypes.CDLL:
    return _LIB if _LIB is not None else load()


def library_path() -> Path | None:
    return _LIB_PATH


def check(rc: int, what: str) -> None:
    """Raise if a C-ABI call returned an error code, with the library's own message."""
    if rc == NB200_OK:
        return
    msg = lib().nb200_last_error().decode("utf-8", "replace")
    exc = NotImplementedError if rc == -2 else (ValueError if rc == -1 else NativeLibraryError)
    raise exc(f"{what}: {ERROR_NAMES.get(rc, rc)}: {msg}")
