"""An NCCL communicator of this process's own, for the one collective of the operator set.

``torch.distributed`` does not hand out the ``ncclComm_t`` of its process groups, and the C ABI
(``nb200_decode_merge_nccl``) takes one.  This module creates a communicator directly on the NCCL
library that the process already has loaded (the one torch brought in), using ``torch.distributed``
only to carry the 128-byte unique id from rank 0 to the others.  One GPU per process, the current
CUDA device at the time of construction.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

_UNIQUE_ID_BYTES = 128


class _UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * _UNIQUE_ID_BYTES)]


class NcclError(RuntimeError):
    pass


_LIB: ctypes.CDLL | None = None


def _loaded_nccl_path() -> str | None:
    try:
        with open("/proc/self/maps") as maps:
            for line in maps:
                path = line.split()[-1]
                if "libnccl" in os.path.basename(path):
                    return path
    except OSError:
        pass
    return None


def library() -> ctypes.CDLL:
    """The NCCL shared library of this process (already loaded copy, else $NEPTUNE_B200_NCCL, else libnccl.so.2)."""
    global _LIB
    if _LIB is None:
        path = _loaded_nccl_path() or os.environ.get("NEPTUNE_B200_NCCL") or "libnccl.so.2"
        try:
            cdll = ctypes.CDLL(path)
        except OSError as exc:
            raise NcclError(f"cannot load NCCL from {path}: {exc}") from exc
        cdll.ncclGetErrorString.restype = ctypes.c_char_p
        cdll.ncclGetErrorString.argtypes = [ctypes.c_int]
        cdll.ncclGetUniqueId.argtypes = [ctypes.POINTER(_UniqueId)]
        cdll.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _UniqueId, ctypes.c_int]
        cdll.ncclCommDestroy.argtypes = [ctypes.c_void_p]
        _LIB = cdll
    return _LIB


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise NcclError(f"{what}: {library().ncclGetErrorString(rc).decode()}")


class Communicator:
    """Owns one ``ncclComm_t``; ``handle`` is the pointer value the C ABI takes."""

    def __init__(self, rank: int, world: int, unique_id: bytes):
        if len(unique_id) != _UNIQUE_ID_BYTES:
            raise ValueError(f"an NCCL unique id has {_UNIQUE_ID_BYTES} bytes, got {len(unique_id)}")
        if not (0 <= rank < world):
            raise ValueError(f"rank {rank} outside world of {world}")
        uid = _UniqueId()
        ctypes.memmove(ctypes.byref(uid), unique_id, _UNIQUE_ID_BYTES)
        comm = ctypes.c_void_p()
        _check(library().ncclCommInitRank(ctypes.byref(comm), world, uid, rank), "ncclCommInitRank")
        self._comm = comm
        self.rank, self.world = rank, world

    @staticmethod
    def new_unique_id() -> bytes:
        uid = _UniqueId()
        _check(library().ncclGetUniqueId(ctypes.byref(uid)), "ncclGetUniqueId")
        return bytes(uid)

    @classmethod
    def from_process_group(cls, group=None) -> "Communicator":
        """One communicator over the ranks of a ``torch.distributed`` group (default: the world)."""
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [cls.new_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        with torch.cuda.device(torch.cuda.current_device()):
            return cls(rank, world, box[0])

    @property
    def handle(self) -> int:
        if self._comm is None or not self._comm.value:
            raise NcclError("the communicator has been destroyed")
        return self._comm.value

    def destroy(self) -> None:
        if self._comm is not None and self._comm.value:
            _check(library().ncclCommDestroy(self._comm), "ncclCommDestroy")
        self._comm = None
