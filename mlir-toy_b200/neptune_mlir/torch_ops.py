"""The operators of the kernel library as ``torch.library`` custom ops (namespace ``nb200``).

For callers that live inside a PyTorch program rather than calling an emitted HTile module: the ops
take the tensors in the same order as the emitted functions, write their outputs in place (declared
through ``mutates_args``) and launch on torch's current stream, so they compose with CUDA-graph
capture and with ``torch.compile`` graphs as opaque calls.  They are thin: every op forwards to
``neptune_mlir.runtime``, which checks the tensors and calls the C ABI.  Importing this module
registers the ops; nothing else in the package depends on it.
"""

from __future__ import annotations

import math

import torch

from . import runtime

_DTYPE_NAMES = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}


def _name(t: torch.Tensor) -> str:
    try:
        return _DTYPE_NAMES[t.dtype]
    except KeyError:
        raise TypeError(f"nb200 operators take f16, bf16 or f32 tensors, got {t.dtype}") from None


@torch.library.custom_op("nb200::attn_fwd", mutates_args=("out",))
def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, scale: float,
             causal: bool) -> None:
    """out = softmax(q k^T * scale) v for [B, H, S, D] tensors (k, v may have another sequence length)."""
    runtime.attn_fwd(q, k, v, out, shape=tuple(q.shape), kv_len=k.shape[2], dtype=_name(q),
                     scale_log2=math.log2(math.e) * scale, causal=causal)


@torch.library.custom_op("nb200::decode_splitk", mutates_args=("partials", "out"))
def decode_splitk(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, partials: torch.Tensor, out: torch.Tensor,
                  scale: float) -> None:
    """Split-K decode + combine: q [B, Hq, D], k/v [B, Hkv, L, D], partials fp32 [B, Hq, splits, D + 2]."""
    B, Hq, D = q.shape
    runtime.decode_splitk(q, k, v, partials, out, B=B, Hq=Hq, Hkv=k.shape[1], L=k.shape[2], D=D,
                          n_splits=partials.shape[2], dtype=_name(q), scale_log2=math.log2(math.e) * scale)


@torch.library.custom_op("nb200::decode_paged", mutates_args=("partials", "out"))
def decode_paged(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                 seq_lens: torch.Tensor, partials: torch.Tensor, out: torch.Tensor, scale: float) -> None:
    """Split-K decode over a paged cache: pools [num_pages, Hkv, 64, D], block_table int32 [B, max_pages], seq_lens int32 [B]."""
    B, Hq, D = q.shape
    runtime.decode_paged(q, k_pages, v_pages, block_table, seq_lens, partials, out, B=B, Hq=Hq, Hkv=k_pages.shape[1],
                         max_pages=block_table.shape[1], page_size=k_pages.shape[2], D=D, n_splits=partials.shape[2],
                         dtype=_name(q), scale_log2=math.log2(math.e) * scale)


@torch.library.custom_op("nb200::selective_scan", mutates_args=("out",))
def selective_scan(u: torch.Tensor, delta: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
                   Dskip: torch.Tensor, z: torch.Tensor, out: torch.Tensor) -> None:
    """Mamba-1 selective scan: u, delta, z, out [B, D, L]; A [D, N]; Bm, Cm [B, N, L]; Dskip [D]."""
    B, Dm, L = u.shape
    runtime.selective_scan(u, delta, A, Bm, Cm, Dskip, z, out, B=B, Dm=Dm, L=L, N=A.shape[1], dtype=_name(u))


@torch.library.custom_op("nb200::ssd_chunk_scan", mutates_args=("workspace", "y"))
def ssd_chunk_scan(x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
                   workspace: torch.Tensor, y: torch.Tensor, chunk: int) -> None:
    """Mamba-2 SSD scan: x, y [B, L, H, P]; dt [B, L, H]; A [H]; Bm, Cm [B, L, G, N]; workspace uint8."""
    B, L, H, P = x.shape
    runtime.ssd_chunk_scan(x, dt, A, Bm, Cm, workspace, y, B=B, L=L, H=H, P=P, N=Bm.shape[3], G=Bm.shape[2],
                           chunk=chunk, dtype=_name(x))


OPS = ("attn_fwd", "decode_splitk", "decode_paged", "selective_scan", "ssd_chunk_scan")
