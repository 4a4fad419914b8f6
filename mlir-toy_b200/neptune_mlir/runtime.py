"""Run-time support for modules emitted by ``neptune_mlir.translators.b200``.

An emitted module contains one function per ``func.func`` of the HTile program; its body is a single
call into this module with the tensors the caller passed (in memref-argument order, outputs written
in place, as with the reference's emitted kernels -- tests/test_translators.py:184-194) and the
static facts read from the program (shapes, dtype, constants).  Each function here checks the
tensors against those facts, then passes raw device pointers and torch's current CUDA stream to the
nb200 C ABI.  Launches are asynchronous; the caller synchronises.  Nothing here computes: without
the kernel library every call raises.
"""

from __future__ import annotations

import torch

from . import native

_TORCH_DTYPES = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
_status_buffers: dict[int, torch.Tensor] = {}


def _check(name: str, t, shape, dtype: str | torch.dtype) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name}: expected a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA tensor (the B200 target has no CPU path)")
    want = _TORCH_DTYPES[dtype] if isinstance(dtype, str) else dtype
    if t.dtype != want:
        raise TypeError(f"{name}: dtype {t.dtype}, the program says {want}")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name}: shape {tuple(t.shape)}, the program says {tuple(shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: tensor must be contiguous row-major")


def _same_device(*tensors) -> torch.device:
    dev = tensors[0].device
    for t in tensors[1:]:
        if t.device != dev:
            raise ValueError("all tensors of one call must live on the same CUDA device")
    return dev


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def status_buffer(dev: torch.device) -> torch.Tensor:
    """Per-device int32[4] that kernels with bounded device-side waits report into."""
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    buf = _status_buffers.get(idx)
    if buf is None:
        buf = torch.zeros(native.STATUS_WORDS, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_buffers[idx] = buf
    return buf


def check_status(device=None) -> None:
    """Synchronise and raise if a kernel reported an expired device-side wait on ``device``."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    buf = status_buffer(dev)
    rc = native.lib().nb200_status_read(buf.data_ptr(), None, _stream(dev))
    if rc != 0:
        buf.zero_()
    native.check(rc, "nb200 status")


def attn_fwd(q, k, v, out, *, shape, kv_len, dtype, scale_log2, causal) -> None:
    """Fused attention forward; ``shape`` = (B, H, Sq, D) of q and out, k/v are (B, H, kv_len, D)."""
    B, H, Sq, D = shape
    _check("q", q, shape, dtype)
    _check("k", k, (B, H, kv_len, D), dtype)
    _check("v", v, (B, H, kv_len, D), dtype)
    _check("out", out, shape, dtype)
    dev = _same_device(q, k, v, out)
    with torch.cuda.device(dev):
        rc = native.lib().nb200_attn_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, Sq, kv_len, D,
            native.DTYPE_CODES[dtype], float(scale_log2), int(bool(causal)),
            status_buffer(dev).data_ptr(), _stream(dev))
    native.check(rc, "nb200_attn_fwd")


def decode_workspace_floats(B, Hq, D, n_splits) -> int:
    return native.lib().nb200_decode_workspace_bytes(B, Hq, D, n_splits) // 4


def decode_splitk(q, k, v, partials, out, *, B, Hq, Hkv, L, D, n_splits, dtype, scale_log2) -> None:
    """Split-K flash-decoding + LSE combine; ``partials`` is fp32 [B, Hq, n_splits, D + 2] scratch.

    ``n_splits = 0`` lets the library choose the count for the GPU it runs on (nb200_decode_auto_splits), bounded
    by the third extent of ``partials``, of which the first B*Hq*n*(D+2) floats are then used.
    """
    _check("q", q, (B, Hq, D), dtype)
    _check("k", k, (B, Hkv, L, D), dtype)
    _check("v", v, (B, Hkv, L, D), dtype)
    cap = n_splits if n_splits > 0 else (partials.shape[2] if isinstance(partials, torch.Tensor) and partials.dim() == 4 else 0)
    _check("partials", partials, (B, Hq, cap, D + 2), torch.float32)
    _check("out", out, (B, Hq, D), dtype)
    dev = _same_device(q, k, v, partials, out)
    lib = native.lib()
    with torch.cuda.device(dev):
        st = _stream(dev)
        if n_splits == 0:
            n_splits = lib.nb200_decode_auto_splits(B, Hkv, L, cap)
            if n_splits <= 0:
                raise native.NativeLibraryError("nb200_decode_auto_splits could not choose a split count")
        rc = lib.nb200_decode_splitk(q.data_ptr(), k.data_ptr(), v.data_ptr(), partials.data_ptr(), B, Hq, Hkv,
                                     L, D, n_splits, native.DTYPE_CODES[dtype], float(scale_log2),
                                     status_buffer(dev).data_ptr(), st)
        native.check(rc, "nb200_decode_splitk")
        rc = lib.nb200_decode_combine(partials.data_ptr(), out.data_ptr(), B * Hq, D, n_splits,
                                      n_splits * (D + 2), D + 2, native.DTYPE_CODES[dtype], st)
        native.check(rc, "nb200_decode_combine")


def decode_paged(q, k_pages, v_pages, block_table, seq_lens, partials, out, *, B, Hq, Hkv, max_pages, page_size, D,
                 n_splits, dtype, scale_log2) -> None:
    """Split-K decode over a paged KV cache + combine; pools are [num_pages, Hkv, page_size, D]."""
    _check("q", q, (B, Hq, D), dtype)
    for name, pool in (("k_pages", k_pages), ("v_pages", v_pages)):
        if not (isinstance(pool, torch.Tensor) and pool.is_cuda and pool.is_contiguous() and pool.dim() == 4
                and tuple(pool.shape[1:]) == (Hkv, page_size, D) and pool.dtype == _TORCH_DTYPES[dtype]):
            raise ValueError(f"{name}: expected a contiguous CUDA [num_pages, {Hkv}, {page_size}, {D}] {dtype} tensor")
    if k_pages.shape[0] != v_pages.shape[0]:
        raise ValueError("k_pages and v_pages must hold the same number of pages")
    _check("block_table", block_table, (B, max_pages), torch.int32)
    _check("seq_lens", seq_lens, (B,), torch.int32)
    _check("partials", partials, (B, Hq, n_splits, D + 2), torch.float32)
    _check("out", out, (B, Hq, D), dtype)
    dev = _same_device(q, k_pages, v_pages, block_table, seq_lens, partials, out)
    lib = native.lib()
    with torch.cuda.device(dev):
        st = _stream(dev)
        rc = lib.nb200_decode_paged_splitk(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
                                           seq_lens.data_ptr(), partials.data_ptr(), B, Hq, Hkv, int(k_pages.shape[0]),
                                           max_pages, page_size, D, n_splits, native.DTYPE_CODES[dtype],
                                           float(scale_log2), status_buffer(dev).data_ptr(), st)
        native.check(rc, "nb200_decode_paged_splitk")
        rc = lib.nb200_decode_combine(partials.data_ptr(), out.data_ptr(), B * Hq, D, n_splits,
                                      n_splits * (D + 2), D + 2, native.DTYPE_CODES[dtype], st)
        native.check(rc, "nb200_decode_combine")


def decode_combine(partials, out, *, rows, D, n_splits, row_stride, split_stride, out_dtype) -> None:
    """LSE combine with explicit strides (in floats); out_dtype 'f32' writes a partial of D + 2 floats."""
    if not (partials.is_cuda and out.is_cuda and partials.dtype == torch.float32):
        raise ValueError("decode_combine: partials must be a CUDA fp32 tensor and out a CUDA tensor")
    if not (partials.is_contiguous() and out.is_contiguous()):
        raise ValueError("decode_combine: tensors must be contiguous")
    need = (rows - 1) * row_stride + (n_splits - 1) * split_stride + D + 2
    if partials.numel() < need:
        raise ValueError(f"decode_combine: partials has {partials.numel()} floats, the strides need {need}")
    out_elems = rows * (D + 2 if out_dtype == "f32" else D)
    if out.numel() != out_elems or out.dtype != _TORCH_DTYPES[out_dtype]:
        raise ValueError("decode_combine: out has the wrong size or dtype")
    dev = _same_device(partials, out)
    with torch.cuda.device(dev):
        rc = native.lib().nb200_decode_combine(partials.data_ptr(), out.data_ptr(), rows, D, n_splits,
                                               row_stride, split_stride, native.DTYPE_CODES[out_dtype],
                                               _stream(dev))
    native.check(rc, "nb200_decode_combine")


def decode_merge_nccl(local_partial, gathered, out, *, rows, D, world, out_dtype, comm) -> None:
    """All-gather per-rank partials over ``comm`` (a ``nccl_comm.Communicator``) and combine across ranks."""
    _check("local_partial", local_partial, (rows, D + 2), torch.float32)
    _check("gathered", gathered, (world, rows, D + 2), torch.float32)
    _check("out", out, (rows, D + 2 if out_dtype == "f32" else D), out_dtype)
    dev = _same_device(local_partial, gathered, out)
    with torch.cuda.device(dev):
        rc = native.lib().nb200_decode_merge_nccl(local_partial.data_ptr(), gathered.data_ptr(), out.data_ptr(),
                                                  rows, D, world, native.DTYPE_CODES[out_dtype], comm.handle,
                                                  _stream(dev))
    native.check(rc, "nb200_decode_merge_nccl")


def selective_scan(u, delta, A, Bm, Cm, Dskip, z, out, *, B, Dm, L, N, dtype) -> None:
    """Mamba-1 selective scan forward (layouts in include/nb200.h)."""
    _check("u", u, (B, Dm, L), dtype)
    _check("delta", delta, (B, Dm, L), dtype)
    _check("A", A, (Dm, N), torch.float32)
    _check("Bm", Bm, (B, N, L), dtype)
    _check("Cm", Cm, (B, N, L), dtype)
    _check("Dskip", Dskip, (Dm,), torch.float32)
    _check("z", z, (B, Dm, L), dtype)
    _check("out", out, (B, Dm, L), dtype)
    dev = _same_device(u, delta, A, Bm, Cm, Dskip, z, out)
    with torch.cuda.device(dev):
        rc = native.lib().nb200_selective_scan_fwd(
            u.data_ptr(), delta.data_ptr(), A.data_ptr(), Bm.data_ptr(), Cm.data_ptr(), Dskip.data_ptr(),
            z.data_ptr(), out.data_ptr(), B, Dm, L, N, native.DTYPE_CODES[dtype], _stream(dev))
    native.check(rc, "nb200_selective_scan_fwd")


def check_workspace_status(workspace) -> None:
    """Synchronise and raise if the SSD kernel recorded an expired device-side wait in ``workspace``."""
    dev = workspace.device
    rc = native.lib().nb200_status_read(workspace.data_ptr(), None, _stream(dev))
    native.check(rc, "nb200 ssd status")


def ssd_workspace_bytes(B, L, H, P, N, G, chunk) -> int:
    return native.lib().nb200_ssd_workspace_bytes(B, L, H, P, N, G, chunk)


def ssd_launches(B, L, H, P, N, G, chunk) -> int:
    """Kernel launches one SSD call makes on the current device (2 when the sequences are cut into segments)."""
    return native.lib().nb200_ssd_launches(B, L, H, P, N, G, chunk)


def ssd_chunk_scan(x, dt, A, Bm, Cm, workspace, y, *, B, L, H, P, N, G, chunk, dtype) -> None:
    """Mamba-2 SSD chunked scan forward; ``workspace`` is a uint8 tensor of ssd_workspace_bytes(...)."""
    _check("x", x, (B, L, H, P), dtype)
    _check("dt", dt, (B, L, H), torch.float32)
    _check("A", A, (H,), torch.float32)
    _check("Bm", Bm, (B, L, G, N), dtype)
    _check("Cm", Cm, (B, L, G, N), dtype)
    _check("y", y, (B, L, H, P), dtype)
    need = ssd_workspace_bytes(B, L, H, P, N, G, chunk)
    if not (isinstance(workspace, torch.Tensor) and workspace.is_cuda and workspace.is_contiguous()
            and workspace.numel() * workspace.element_size() >= need):
        raise ValueError(f"workspace: need a contiguous CUDA tensor of at least {need} bytes")
    dev = _same_device(x, dt, A, Bm, Cm, workspace, y)
    with torch.cuda.device(dev):
        rc = native.lib().nb200_ssd_chunk_scan_fwd(
            x.data_ptr(), dt.data_ptr(), A.data_ptr(), Bm.data_ptr(), Cm.data_ptr(), y.data_ptr(),
            workspace.data_ptr(), B, L, H, P, N, G, chunk, native.DTYPE_CODES[dtype], _stream(dev))
    native.check(rc, "nb200_ssd_chunk_scan_fwd")
