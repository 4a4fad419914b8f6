"""Peer-mapped workspace for the single-sequence decode merge (``nb200_decode_merge_peer``).

One symmetric buffer per rank, allocated and exported by the kernel library (CUDA IPC), the handles carried to
the other ranks by ``torch.distributed`` (an object all-gather at set-up time, nothing on the data path).  After
that a merge is one kernel launch per rank: stores into the peers' buffers, flags, a bounded wait, the combine.
One GPU per process; the current CUDA device at construction is the one the buffer lives on.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import native, runtime


class PeerWorkspace:
    """Owns this rank's symmetric buffer and the mappings of the other ranks' buffers."""

    DEFAULT_WAIT_NS = 2_000_000_000

    def __init__(self, rows: int, D: int, group=None):
        lib = native.lib()
        self.rows, self.D = rows, D
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        size = lib.nb200_decode_merge_peer_workspace_bytes(rows, D, self.world)
        if size == 0:
            raise NotImplementedError(f"peer merge: rows={rows}, D={D}, world={self.world} is not supported")
        own, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        native.check(lib.nb200_peer_buffer_alloc(size, ctypes.byref(own), handle), "nb200_peer_buffer_alloc")
        self._own = own.value
        handles: list = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._ptrs: list[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self._ptrs.append(self._own)
                continue
            p = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            native.check(lib.nb200_peer_buffer_open(buf, ctypes.byref(p)), f"nb200_peer_buffer_open (rank {r})")
            self._ptrs.append(p.value)
        self._array = (ctypes.c_void_p * self.world)(*self._ptrs)
        self.generation = 0
        dist.barrier(group)          # every rank has mapped every buffer before the first merge

    def merge(self, local_partial: torch.Tensor, out: torch.Tensor, out_dtype: str, wait_ns: int | None = None) -> None:
        """Enqueue the merge on the current stream; every rank must call it the same number of times."""
        rows, D = self.rows, self.D
        runtime._check("local_partial", local_partial, (rows, D + 2), torch.float32)
        runtime._check("out", out, (rows, D + 2 if out_dtype == "f32" else D), out_dtype)
        dev = runtime._same_device(local_partial, out)
        self.generation += 1
        with torch.cuda.device(dev):
            rc = native.lib().nb200_decode_merge_peer(
                local_partial.data_ptr(), self._array, out.data_ptr(), rows, D, self.world, self.rank, self.generation,
                native.DTYPE_CODES[out_dtype], wait_ns or self.DEFAULT_WAIT_NS, runtime.status_buffer(dev).data_ptr(),
                runtime._stream(dev))
        native.check(rc, "nb200_decode_merge_peer")

    def sharded_decode(self, q, k, v, workspace, out, *, Hq, Hkv, L, D, n_splits, dtype, scale_log2, out_dtype,
                       wait_ns: int | None = None) -> None:
        """This rank's whole share of a single-sequence decode as one launch (``nb200_decode_sharded_fwd``):
        ``k``/``v`` are the rank's slice [1, Hkv, L, D]; ``workspace`` is a uint8 tensor of
        ``nb200_decode_sharded_workspace_bytes`` bytes that was zeroed once."""
        runtime._check("q", q, (1, Hq, D), dtype)
        runtime._check("k", k, (1, Hkv, L, D), dtype)
        runtime._check("v", v, (1, Hkv, L, D), dtype)
        runtime._check("out", out, (Hq, D + 2 if out_dtype == "f32" else D), out_dtype)
        dev = runtime._same_device(q, k, v, workspace, out)
        self.generation += 1
        with torch.cuda.device(dev):
            rc = native.lib().nb200_decode_sharded_fwd(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), workspace.data_ptr(), self._array, out.data_ptr(), Hq, Hkv, L, D,
                n_splits, native.DTYPE_CODES[dtype], float(scale_log2), self.world, self.rank, self.generation,
                native.DTYPE_CODES[out_dtype], wait_ns or self.DEFAULT_WAIT_NS, runtime.status_buffer(dev).data_ptr(),
                runtime._stream(dev))
        native.check(rc, "nb200_decode_sharded_fwd")

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (call on every rank, after synchronising)."""
        lib = native.lib()
        for r, p in enumerate(self._ptrs):
            if r != self.rank and p:
                lib.nb200_peer_buffer_close(ctypes.c_void_p(p))
        self._ptrs = []
        if self._own:
            lib.nb200_peer_buffer_free(ctypes.c_void_p(self._own))
            self._own = 0
