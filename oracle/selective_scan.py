"""CPU restatement of the Mamba-1 selective scan (test infrastructure; see package docstring).

The reference has no scan operator; this definition is this build's own (parity unpinned).

Layouts: u, delta, z, out [B, D, L] (L contiguous); A [D, N] fp32; Bm, Cm [B, N, L]; Dskip [D] fp32.
delta arrives already soft-plused.  h starts at zero:

    h[b,d,n] <- exp(delta[b,d,t] * A[d,n]) * h[b,d,n] + delta[b,d,t] * Bm[b,n,t] * u[b,d,t]
    y[b,d,t]  = sum_n Cm[b,n,t] * h[b,d,n] + Dskip[d] * u[b,d,t]
    out       = y * z * sigmoid(z)                       (SiLU gate), rounded to the storage dtype

All arithmetic is fp32 on storage-rounded inputs.
"""

from __future__ import annotations

import torch


def selective_scan_reference(u, delta, A, Bm, Cm, Dskip, z):
    """Sequential over L, vectorised over (B, D, N); returns fp32 [B, D, L] (not yet rounded)."""
    Bsz, Dm, L = u.shape
    N = A.shape[1]
    uf, df, zf = u.float(), delta.float(), z.float()
    Bf, Cf = Bm.float(), Cm.float()
    A = A.float()
    h = torch.zeros((Bsz, Dm, N), dtype=torch.float32)
    y = torch.empty((Bsz, Dm, L), dtype=torch.float32)
    for t in range(L):
        dt = df[:, :, t]                                     # [B, D]
        a = torch.exp(dt[:, :, None] * A[None])              # [B, D, N]
        bu = (dt * uf[:, :, t])[:, :, None] * Bf[:, None, :, t]
        h = a * h + bu
        y[:, :, t] = (h * Cf[:, None, :, t]).sum(dim=-1)
    y = y + Dskip.float()[None, :, None] * uf
    return y * zf * torch.sigmoid(zf)
