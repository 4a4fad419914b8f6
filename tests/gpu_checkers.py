"""Checkers that run on the GPU, for parity tests over whole benchmark configurations.

Two kinds, both used only by tests (never by the product path):

* fp64 evaluations, in plain torch on the device, of the same definitions that ``oracle/`` states on the CPU
  (``tests/test_gpu_pins.py`` ties each of them to its CPU twin on a small case).  They make it possible to
  compare every element of a full-size output instead of a sample.
* third-party kernels that ship in this image (PyTorch's scaled_dot_product_attention, flash-attn, FlashInfer,
  vLLM's Mamba operators), written by other people from the published definitions of these operators.  The
  reference project computes none of causal attention, decode or the scans, so these are the only independent
  implementations the kernels can be compared with; a disagreement with them would contradict this build's own
  oracle.  Each wrapper raises ``Unavailable`` when its package cannot be imported or cannot run on this GPU.
"""

from __future__ import annotations

import math

import torch


class Unavailable(RuntimeError):
    pass


def _import(path: str, name: str):
    import importlib

    try:
        return getattr(importlib.import_module(path), name)
    except Exception as exc:  # noqa: BLE001 - any import-time failure means "not usable here"
        raise Unavailable(f"{path}.{name}: {type(exc).__name__}: {exc}") from exc


# ------------------------------------------------------------------------------------------ attention
def sdpa_math(q, k, v, causal: bool, dtype=torch.float32, scale=None, gqa=False):
    """softmax(q k^T * scale) v with PyTorch's unfused 'math' backend in ``dtype`` (lower-right aligned when
    Skv > Sq is never needed here: callers pass Sq == Skv or a single query)."""
    from torch.nn.attention import SDPBackend, sdpa_kernel

    with sdpa_kernel(SDPBackend.MATH):
        return torch.nn.functional.scaled_dot_product_attention(
            q.to(dtype), k.to(dtype), v.to(dtype), is_causal=causal, scale=scale, enable_gqa=gqa)


def flash_attn_prefill(q, k, v, causal: bool):
    """flash-attn's fused forward on [B, H, S, D] 16-bit tensors; returns [B, H, S, D]."""
    fn = _import("flash_attn", "flash_attn_func")
    try:
        out = fn(q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous(),
                 causal=causal)
    except RuntimeError as exc:
        raise Unavailable(f"flash_attn_func: {exc}") from exc
    return out.transpose(1, 2)


def flash_attn_decode(q, k, v):
    """flash-attn's KV-cache decode: q [B, Hq, D], k/v [B, Hkv, L, D] -> [B, Hq, D]."""
    fn = _import("flash_attn", "flash_attn_with_kvcache")
    try:
        out = fn(q[:, None].contiguous(), k.transpose(1, 2), v.transpose(1, 2), causal=True)
    except RuntimeError as exc:
        raise Unavailable(f"flash_attn_with_kvcache: {exc}") from exc
    return out[:, 0]


def flashinfer_decode_one(q, k, v):
    """FlashInfer's single-request decode: q [Hq, D], k/v [Hkv, L, D] -> [Hq, D]."""
    fn = _import("flashinfer", "single_decode_with_kv_cache")
    try:
        return fn(q, k, v, kv_layout="HND")
    except RuntimeError as exc:
        raise Unavailable(f"flashinfer.single_decode_with_kv_cache: {exc}") from exc


def decode_fp32(q, k, v, batch_chunk: int = 8):
    """Direct softmax over the whole cache in fp32 (PyTorch math backend, grouped-query), a few sequences at a time."""
    outs = []
    for b0 in range(0, q.shape[0], batch_chunk):
        sl = slice(b0, b0 + batch_chunk)
        outs.append(sdpa_math(q[sl, :, None], k[sl], v[sl], causal=False, gqa=True)[:, :, 0])
    return torch.cat(outs)


# ------------------------------------------------------------------------------------------ Mamba-1
def selective_scan_fp64(u, delta, A, Bm, Cm, Dskip, z):
    """h <- exp(delta A) h + delta B u; y = C.h + D u; out = y silu(z) -- sequential over L in fp64 on the device."""
    Bsz, Dm, L = u.shape
    f = torch.float64
    uf, df, zf = u.to(f), delta.to(f), z.to(f)
    Bf, Cf, Af = Bm.to(f), Cm.to(f), A.to(f)
    h = torch.zeros((Bsz, Dm, A.shape[1]), dtype=f, device=u.device)
    y = torch.empty((Bsz, Dm, L), dtype=f, device=u.device)
    for t in range(L):
        dt = df[:, :, t]
        h = torch.exp(dt[:, :, None] * Af[None]) * h + (dt * uf[:, :, t])[:, :, None] * Bf[:, None, :, t]
        y[:, :, t] = (h * Cf[:, None, :, t]).sum(dim=-1)
    y = y + Dskip.to(f)[None, :, None] * uf
    return y * zf * torch.sigmoid(zf)


def vllm_selective_scan(u, delta, A, Bm, Cm, Dskip, z):
    """vLLM's CUDA selective scan (no initial state, delta already soft-plused); returns [B, D, L] in u's dtype."""
    fn = _import("vllm.model_executor.layers.mamba.ops.mamba_ssm", "selective_scan_fn")
    Bsz, Dm, _ = u.shape
    states = torch.zeros((Bsz, Dm, A.shape[1]), dtype=torch.float32, device=u.device)
    try:
        return fn(u.clone(), states, delta.clone(), A, Bm.clone(), Cm.clone(), Dskip, z.clone(), None, False,
                  has_initial_state=torch.zeros(Bsz, dtype=torch.bool, device=u.device))
    except RuntimeError as exc:
        raise Unavailable(f"vllm selective_scan_fn: {exc}") from exc


# ------------------------------------------------------------------------------------------ Mamba-2
def ssd_fp64(x, dt, A, Bm, Cm):
    """S <- exp(dt A) S + dt x (outer) B; y = S.C -- sequential over L in fp64 on the device."""
    Bsz, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    rep = H // G
    f = torch.float64
    xf, dtf, Af = x.to(f), dt.to(f), A.to(f)
    Bf, Cf = Bm.to(f), Cm.to(f)
    S = torch.zeros((Bsz, H, P, N), dtype=f, device=x.device)
    y = torch.empty((Bsz, L, H, P), dtype=f, device=x.device)
    for t in range(L):
        a = torch.exp(dtf[:, t] * Af[None])
        Bt = Bf[:, t].repeat_interleave(rep, dim=1)
        Ct = Cf[:, t].repeat_interleave(rep, dim=1)
        dx = dtf[:, t][:, :, None] * xf[:, t]
        S = a[:, :, None, None] * S + dx[:, :, :, None] * Bt[:, :, None, :]
        y[:, t] = torch.einsum("bhpn,bhn->bhp", S, Ct)
    return y


def vllm_ssd(x, dt, A, Bm, Cm, chunk: int):
    """vLLM's Triton chunked SSD scan (its variable-length entry point, fed B equal-length sequences)."""
    fn = _import("vllm.model_executor.layers.mamba.ops.ssd_combined", "mamba_chunk_scan_combined_varlen")
    Bsz, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    T, dev = Bsz * L, x.device
    per_seq = L // chunk
    cu_seqlens = torch.arange(0, T + 1, L, dtype=torch.int32, device=dev)
    cu_chunks = torch.arange(0, T + 1, chunk, dtype=torch.int32, device=dev)
    last_chunk = torch.arange(1, Bsz + 1, dtype=torch.int32, device=dev) * per_seq - 1
    seq_idx = torch.arange(T // chunk, dtype=torch.int32, device=dev) // per_seq
    out = torch.empty((T, H, P), dtype=x.dtype, device=dev)
    try:
        fn(x.reshape(T, H, P), dt.reshape(T, H), A, Bm.reshape(T, G, N), Cm.reshape(T, G, N), chunk, cu_seqlens,
           cu_chunks, last_chunk, seq_idx, out)
    except RuntimeError as exc:
        raise Unavailable(f"vllm mamba_chunk_scan_combined_varlen: {exc}") from exc
    return out.view(Bsz, L, H, P)


def flashinfer_ssd(x, dt, A, Bm, Cm, chunk: int = 128):
    """FlashInfer's Blackwell SSD kernel (bf16 I/O, dt and the carried state rounded to bf16 inside)."""
    cls = _import("flashinfer.mamba", "SSDCombined")
    Bsz, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    try:
        op = cls(chunk_size=chunk, nheads=H, headdim=P, dstate=N, ngroups=G, has_d=False)
        out, _ = op.run(x, dt, A, Bm, Cm)
    except Exception as exc:  # noqa: BLE001 - a JIT failure of any kind means "not usable here"
        raise Unavailable(f"flashinfer SSDCombined: {type(exc).__name__}: {exc}") from exc
    return out.reshape(Bsz, L, H, P)


# ------------------------------------------------------------------------------------------ error measures
def bf16_neighbours(ref: torch.Tensor):
    """The two bf16 values that bracket each element of ``ref`` (equal when ref is itself a bf16 value)."""
    r = ref.float()
    near = r.to(torch.bfloat16)
    bits = near.view(torch.int16).to(torch.int32)
    nf = near.float()
    # step one unit in the last place towards ref on the other side of `near`
    away_up = nf < r                     # nearest lies below ref: the other neighbour is one ulp up
    away_dn = nf > r
    sign_neg = nf < 0
    step = torch.zeros_like(bits)
    step = torch.where(away_up, torch.where(sign_neg, -1, 1), step)
    step = torch.where(away_dn, torch.where(sign_neg, 1, -1), step)
    # crossing zero (near == +-0 exactly) does not occur for these data; guard anyway
    other_bits = torch.where(nf == 0, bits, bits + step)
    other = other_bits.to(torch.int16).view(torch.bfloat16)
    lo = torch.minimum(nf, other.float())
    hi = torch.maximum(nf, other.float())
    return lo, hi


def parity_stats(out: torch.Tensor, ref: torch.Tensor, atol: float) -> dict:
    """Error of a bf16 result against a high-precision reference, three ways:
    max abs error; the share of elements that are neither within ``atol`` nor one of the two bf16 neighbours of
    the reference value (i.e. wrong by more than the output format's own rounding); and rms error over rms(ref)."""
    o, r = out.double(), ref.double()
    err = (o - r).abs()
    lo, hi = bf16_neighbours(ref)
    of = out.float()
    ok = (err <= atol) | (of == lo) | (of == hi)
    return {
        "max_abs_err": err.max().item(),
        "rms_rel": (err.pow(2).mean().sqrt() / r.pow(2).mean().sqrt()).item(),
        "rms_ref": r.pow(2).mean().sqrt().item(),
        "max_abs_ref": r.abs().max().item(),
        "outside": int((~ok).sum().item()),
        "outside_share": (~ok).double().mean().item(),
        # error of the worst failing element in units in the last place of bf16 at the reference's magnitude
        "worst_ulps": ((err / torch.exp2(torch.floor(torch.log2(r.abs().clamp_min(1e-30))) - 7))[~ok].max().item()
                       if bool((~ok).any()) else 0.0),
        "elements": o.numel(),
    }


def log2e() -> float:
    return math.log2(math.e)
