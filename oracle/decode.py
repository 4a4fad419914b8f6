"""CPU restatement of split-K flash-decoding with GQA (test infrastructure; see package docstring).

The reference has no decode operator; the definition below is this build's own (parity unpinned).
Layouts follow the reference's [B, H, S, D] convention (tests/data/flash_attention_htile.mlir:12-15):
q [B, Hq, D], k and v [B, Hkv, L, D]; query head h reads kv head h // (Hq // Hkv).
"""

from __future__ import annotations

import math

import torch


def decode_reference(q, k, v, scale: float | None = None, kv_chunk: int = 4096):
    """Direct softmax over all L tokens, fp32 math on storage-rounded inputs; returns fp32 [B,Hq,D].

    K/V are converted to fp32 one (batch, chunk) slice at a time so that a cache of several GiB in
    bf16 never exists as a whole in fp32.
    """
    B, Hq, D = q.shape
    Hkv, L = k.shape[1], k.shape[2]
    group = Hq // Hkv
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    out = torch.empty((B, Hq, D), dtype=torch.float32)
    for b in range(B):
        qg = q[b].float().view(Hkv, group, D)
        m = torch.full((Hkv, group), float("-inf"))
        l = torch.zeros((Hkv, group))
        o = torch.zeros((Hkv, group, D))
        for t0 in range(0, L, kv_chunk):
            kc = k[b, :, t0:t0 + kv_chunk].float()
            vc = v[b, :, t0:t0 + kv_chunk].float()
            x = torch.matmul(qg, kc.transpose(-1, -2)) * scale       # [Hkv, group, T]
            m_new = torch.maximum(m, x.amax(dim=-1))
            p = torch.exp(x - m_new[..., None])
            a = torch.exp(m - m_new)
            l = l * a + p.sum(dim=-1)
            o = o * a[..., None] + torch.matmul(p, vc)
            m = m_new
        out[b] = (o / l[..., None]).view(Hq, D)
    return out


def decode_partials(q, k, v, n_splits: int, scale: float | None = None):
    """Per-split (m, l, o): x_t = q.k_t*scale, m_s = max x_t, l_s = sum e^(x_t-m_s), o_s = sum e^(x_t-m_s) v_t.

    Split s covers rows [floor(s*L/n), floor((s+1)*L/n)).
    Returns m, l [B,Hq,n_splits] and o [B,Hq,n_splits,D], all fp32, natural-exponent domain.
    """
    B, Hq, D = q.shape
    Hkv, L = k.shape[1], k.shape[2]
    group = Hq // Hkv
    assert 0 < n_splits <= L
    edges = [s * L // n_splits for s in range(n_splits + 1)]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    m = torch.empty((B, Hq, n_splits))
    l = torch.empty((B, Hq, n_splits))
    o = torch.empty((B, Hq, n_splits, D))
    for b in range(B):
        qg = q[b].float().view(Hkv, group, D)
        for s in range(n_splits):
            kc = k[b, :, edges[s]:edges[s + 1]].float()
            vc = v[b, :, edges[s]:edges[s + 1]].float()
            x = torch.matmul(qg, kc.transpose(-1, -2)) * scale
            ms = x.amax(dim=-1)
            p = torch.exp(x - ms[..., None])
            m[b, :, s] = ms.view(Hq)
            l[b, :, s] = p.sum(dim=-1).view(Hq)
            o[b, :, s] = torch.matmul(p, vc).view(Hq, D)
    return m, l, o


def combine_partials(m, l, o):
    """LSE combine: M = max_s m_s; out = sum_s e^(m_s-M) o_s / sum_s e^(m_s-M) l_s (fp32).

    The same function merges per-GPU partials when one sequence's KV is sharded over GPUs.
    """
    M = m.amax(dim=-1, keepdim=True)
    w = torch.exp(m - M)
    num = (w[..., None] * o).sum(dim=-2)
    den = (w * l).sum(dim=-1)
    return num / den[..., None]
