"""CPU restatement of the Mamba-2 SSD scan (test infrastructure; see package docstring).

The reference has no SSD operator; this definition is this build's own (parity unpinned).

Layouts: x, y [B, L, H, P]; dt [B, L, H] fp32 (already soft-plused); A [H] fp32 (negative);
Bm, Cm [B, L, G, N] with head h reading group h // (H // G).  The state S[b,h] is a P x N matrix,
zero at t = 0:

    S <- exp(dt[b,t,h] * A[h]) * S + dt[b,t,h] * x[b,t,h,:] (outer) Bm[b,t,g,:]
    y[b,t,h,:] = S . Cm[b,t,g,:]

``ssd_reference`` is that recurrence (the oracle of record); ``ssd_chunked`` is the chunked
algorithm the kernel implements and must give the same numbers.
"""

from __future__ import annotations

import torch


def ssd_reference(x, dt, A, Bm, Cm):
    """Sequential definition; fp32 math on storage-rounded inputs; returns fp32 [B, L, H, P]."""
    Bsz, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    rep = H // G
    xf, Bf, Cf = x.float(), Bm.float(), Cm.float()
    dt = dt.float()
    A = A.float()
    S = torch.zeros((Bsz, H, P, N), dtype=torch.float32)
    y = torch.empty((Bsz, L, H, P), dtype=torch.float32)
    for t in range(L):
        a = torch.exp(dt[:, t] * A[None])                                # [B, H]
        Bt = Bf[:, t].repeat_interleave(rep, dim=1)                      # [B, H, N]
        Ct = Cf[:, t].repeat_interleave(rep, dim=1)
        dx = dt[:, t][:, :, None] * xf[:, t]                             # [B, H, P]
        S = a[:, :, None, None] * S + dx[:, :, :, None] * Bt[:, :, None, :]
        y[:, t] = torch.einsum("bhpn,bhn->bhp", S, Ct)
    return y


def ssd_chunked(x, dt, A, Bm, Cm, chunk: int, round_to=None):
    """Chunked form: intra-chunk masked products + fp32 state passed between chunks.

    With ``round_to`` (a 16-bit dtype) the three places where the kernel feeds a computed fp32 value
    back into a tensor-core product are rounded to that dtype, as the kernel must: the masked decayed
    C.B^T block, the decay-weighted x of the chunk state, and the state entering a chunk (the fp32
    master copy of the state is still what is carried).  This "kernel-faithful" form separates the
    kernel's own arithmetic from the unavoidable operand rounding when outputs reach magnitudes of
    several hundred.

    Per chunk with cum_i = sum_{s<=i} dt_s*A:
      Y_intra[i] = sum_{j<=i} (C_i.B_j) e^(cum_i-cum_j) dt_j x_j
      Z          = sum_j e^(cum_Q-cum_j) dt_j x_j (outer) B_j
      S_in(c)    = e^(cum_Q(c-1)) S_in(c-1) + Z(c-1)
      Y_inter[i] = e^(cum_i) (S_in . C_i)
    """
    Bsz, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    rep = H // G
    assert L % chunk == 0
    nc = L // chunk
    xf = x.float().view(Bsz, nc, chunk, H, P)
    dtc = dt.float().view(Bsz, nc, chunk, H)
    Bf = Bm.float().view(Bsz, nc, chunk, G, N).repeat_interleave(rep, dim=3)
    Cf = Cm.float().view(Bsz, nc, chunk, G, N).repeat_interleave(rep, dim=3)
    cum = torch.cumsum(dtc * A.float()[None, None, None, :], dim=2)       # [B, nc, Q, H]
    y = torch.empty((Bsz, nc, chunk, H, P), dtype=torch.float32)
    S = torch.zeros((Bsz, H, P, N), dtype=torch.float32)
    tri = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool))

    def rnd(t):
        return t if round_to is None else t.to(round_to).float()

    for c in range(nc):
        cb = torch.einsum("bihn,bjhn->bhij", Cf[:, c], Bf[:, c])           # [B, H, Q, Q]
        ci = cum[:, c].permute(0, 2, 1)                                   # [B, H, Q]
        decay = torch.exp((ci[:, :, :, None] - ci[:, :, None, :]).masked_fill(~tri, float("-inf")))
        w = cb * decay * dtc[:, c].permute(0, 2, 1)[:, :, None, :]
        y_intra = torch.einsum("bhij,bjhp->bihp", rnd(w), xf[:, c])
        y_inter = torch.einsum("bhpn,bihn->bihp", rnd(S), Cf[:, c]) * torch.exp(ci).permute(0, 2, 1)[..., None]
        y[:, c] = y_intra + y_inter
        last = ci[:, :, -1]                                               # [B, H]
        wz = torch.exp(last[:, :, None] - ci) * dtc[:, c].permute(0, 2, 1)  # [B, H, Q]
        xs = rnd(wz.permute(0, 2, 1)[..., None] * xf[:, c])                 # [B, Q, H, P]
        Z = torch.einsum("bjhp,bjhn->bhpn", xs, Bf[:, c])
        S = torch.exp(last)[:, :, None, None] * S + Z
    return y.view(Bsz, L, H, P)
