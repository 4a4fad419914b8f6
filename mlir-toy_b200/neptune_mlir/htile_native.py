"""Binding of the C++ HTile front end (include/htile_front.h, libhtile_front.so).

``parse_module`` and ``run_pipeline`` do in native code what ``htile_text.parse_module`` and
``passes.run_pipeline`` do in Python -- read HTile text, verify the htile ops, apply the
dot-transpose-to-load-order rewrite -- and hand the result back as the same object model
(``htile_text.Module`` / ``Func`` / ``Block`` / ``Op`` / ``Value``), rebuilt from the library's JSON
view, so the translators run unchanged on either reader.  This is the part of the pipeline the
reference implements in C++ (its dialect plugin inside ``mlir-opt``).
"""

from __future__ import annotations

import ctypes
import json
from ctypes import c_char_p, c_int, c_size_t, c_void_p
from pathlib import Path

from . import htile_text as ht
from .plugin import find_front_path

_ERR_LEN = 1024
_LIB: ctypes.CDLL | None = None
_LIB_PATH: Path | None = None

SYMBOLS = {
    "htf_version": (c_int, []),
    "htf_parse": (c_void_p, [c_char_p, c_char_p, c_size_t]),
    "htf_free": (None, [c_void_p]),
    "htf_verify": (c_int, [c_void_p, c_char_p, c_size_t]),
    "htf_run_pipeline": (c_int, [c_void_p, c_char_p, c_char_p, c_size_t]),
    "htf_to_json": (c_void_p, [c_void_p]),
    "htf_print": (c_void_p, [c_void_p]),
    "htf_string_free": (None, [c_void_p]),
}


class FrontEndUnavailable(RuntimeError):
    pass


def load(path=None) -> ctypes.CDLL:
    global _LIB, _LIB_PATH
    resolved = find_front_path(path)
    if resolved is None:
        raise FrontEndUnavailable("libhtile_front.so was not found; build it with `python mlir-toy_b200/build_native.py` "
                                  "or point $NEPTUNE_HTILE_FRONT_LIB at it")
    if _LIB is not None and _LIB_PATH == resolved:
        return _LIB
    cdll = ctypes.CDLL(str(resolved))
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(cdll, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB, _LIB_PATH = cdll, resolved
    return cdll


def available() -> bool:
    return find_front_path() is not None


def _take_string(lib, ptr) -> str:
    if not ptr:
        raise RuntimeError("the HTile front end returned no text")
    try:
        return ctypes.string_at(ptr).decode("utf-8")
    finally:
        lib.htf_string_free(ptr)


class NativeModule:
    """Owns one ``htf_module``; use as a context manager or call ``close``."""

    def __init__(self, text: str, path=None):
        self._lib = load(path)
        err = ctypes.create_string_buffer(_ERR_LEN)
        self._handle = self._lib.htf_parse(text.encode("utf-8"), err, _ERR_LEN)
        if not self._handle:
            raise ht.HTileSyntaxError(err.value.decode("utf-8", "replace"))

    def close(self) -> None:
        if self._handle:
            self._lib.htf_free(self._handle)
            self._handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def __del__(self):
        self.close()

    def verify(self) -> None:
        err = ctypes.create_string_buffer(_ERR_LEN)
        if self._lib.htf_verify(self._handle, err, _ERR_LEN) != 0:
            raise ht.HTileSyntaxError(err.value.decode("utf-8", "replace"))

    def run_pipeline(self, pipeline: str) -> None:
        from .passes import PassError

        err = ctypes.create_string_buffer(_ERR_LEN)
        if self._lib.htf_run_pipeline(self._handle, pipeline.encode("utf-8"), err, _ERR_LEN) != 0:
            raise PassError(err.value.decode("utf-8", "replace"))

    def json(self) -> dict:
        return json.loads(_take_string(self._lib, self._lib.htf_to_json(self._handle)))

    def text(self) -> str:
        return _take_string(self._lib, self._lib.htf_print(self._handle))

    def to_module(self) -> ht.Module:
        return module_from_json(self.json())


def module_from_json(doc: dict) -> ht.Module:
    """Rebuild the Python object model from the front end's JSON view."""
    values: dict[int, ht.Value] = {}

    def define(d: dict, owner, index: int) -> ht.Value:
        v = ht.Value(d["name"], ht.parse_type(d["type"]), owner, index)
        values[d["id"]] = v
        return v

    def block(d: dict, parent_op) -> ht.Block:
        b = ht.Block(parent_op=parent_op)
        b.arguments = [define(a, b, i) for i, a in enumerate(d["arguments"])]
        for od in d["operations"]:
            op = ht.Op(od["name"])
            op.parent = b
            op.operands = [values[i] for i in od["operands"]]
            op.attributes = dict(od["attributes"])
            op.regions = [block(r, op) for r in od["regions"]]
            op.results = [define(r, op, i) for i, r in enumerate(od["results"])]
            b.operations.append(op)
        return b

    funcs = []
    for fd in doc["functions"]:
        body = block(fd["body"], None)
        funcs.append(ht.Func(fd["name"], body.arguments, dict(fd["attributes"]), body))
    return ht.Module(funcs)


def parse_module(text: str, pipeline: str | None = None, verify: bool = True) -> ht.Module:
    """Read (and verify) HTile text with the C++ front end, optionally run a pass pipeline there."""
    with NativeModule(text) as nm:
        if verify:
            nm.verify()
        if pipeline:
            nm.run_pipeline(pipeline)
            if verify:
                nm.verify()
        return nm.to_module()


def parse_file(path, pipeline: str | None = None) -> ht.Module:
    with open(path, "r", encoding="utf-8") as f:
        return parse_module(f.read(), pipeline)
