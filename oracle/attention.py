"""CPU restatements of the attention forward pass (test infrastructure; see package docstring).

Two forms are kept on purpose:

``attention_reference``
    The reference's check function (tests/test_translators.py:122-135): fp32, blocks of 128 query
    rows, full-row softmax with the natural exponential.  The causal mask (``j <= i``) is an
    addition of this build; the reference has no causal case (parity unpinned for it).

``attention_program``
    A literal reading of the HTile program (tests/data/flash_attention_htile.mlir:40-143): online
    softmax in the exp2 domain over KV blocks, scale constant rounded to fp32, running maximum
    initialised to -FLT_MAX (:23), row sum taken from the *unrounded* probabilities (:81-91), the
    probabilities rounded to the storage dtype before the PV product (:93-100), output rounded to
    the storage dtype (:139-140).
"""

from __future__ import annotations

import math

import torch

REF_BLOCK_ROWS = 128  # tests/test_translators.py:37
NEG_FLT_MAX = -3.4028234663852886e38  # tests/data/flash_attention_htile.mlir:23


def scale_log2(head_dim: int) -> float:
    """fl32(log2(e) / sqrt(D)), the constant at tests/data/flash_attention_htile.mlir:24."""
    return float(torch.tensor(math.log2(math.e) / math.sqrt(head_dim), dtype=torch.float32))


def attention_reference(q, k, v, causal: bool = False, scale: float | None = None):
    """softmax(Q K^T * scale) V in fp32; returns fp32 [B,H,Sq,D].

    Follows tests/test_translators.py:122-135 line by line (128-row query blocks, fp32 matmuls,
    torch.softmax); with ``causal`` a query row i only sees keys j <= i + (Skv - Sq).
    """
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    ref = torch.empty((B, H, Sq, v.shape[-1]), dtype=torch.float32)
    k_t = k.transpose(-1, -2).float()
    v_f = v.float()
    cols = torch.arange(Skv)
    for row_start in range(0, Sq, REF_BLOCK_ROWS):
        row_end = min(row_start + REF_BLOCK_ROWS, Sq)
        q_block = q[:, :, row_start:row_end, :].float()
        scores = torch.matmul(q_block, k_t) * scale
        if causal:
            rows = torch.arange(row_start, row_end) + (Skv - Sq)
            scores = scores.masked_fill(cols[None, :] > rows[:, None], float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        ref[:, :, row_start:row_end, :] = torch.matmul(probs, v_f)
    return ref


def attention_program(q, k, v, causal: bool = False, kv_block: int = 64, c: float | None = None):
    """The HTile program evaluated op by op on CPU; returns the storage dtype of ``q``.

    One loop iteration = tests/data/flash_attention_htile.mlir:47-127.  Masked scores take the value
    -FLT_MAX before the running maximum (the builder-defined causal extension), and contribute a
    probability of exactly zero.
    """
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    dt = q.dtype
    c = scale_log2(D) if c is None else c
    qf, kf, vf = q.float(), k.float(), v.float()
    m = torch.full((B, H, Sq), NEG_FLT_MAX, dtype=torch.float32)
    l = torch.zeros((B, H, Sq), dtype=torch.float32)
    acc = torch.zeros((B, H, Sq, v.shape[-1]), dtype=torch.float32)
    rows = torch.arange(Sq) + (Skv - Sq)
    for j0 in range(0, Skv, kv_block):
        j1 = min(j0 + kv_block, Skv)
        s = torch.matmul(qf, kf[:, :, j0:j1].transpose(-1, -2)) * c          # :52-59
        if causal:
            masked = torch.arange(j0, j1)[None, :] > rows[:, None]
            s = s.masked_fill(masked, NEG_FLT_MAX)
        m_new = torch.maximum(m, s.amax(dim=-1))                               # :61-64
        p = torch.exp2(s - m_new[..., None])                                   # :76-79
        if causal:
            p = p.masked_fill(masked, 0.0)
        alpha = torch.exp2(m - m_new)                                          # :84-87
        l = l * alpha + p.sum(dim=-1)                                          # :81-91
        acc = acc * alpha[..., None] + torch.matmul(p.to(dt).float(), vf[:, :, j0:j1])  # :93-122
        m = m_new
    return (acc / l[..., None]).to(dt)                                         # :130-140
