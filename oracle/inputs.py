"""Seeded synthetic inputs for the five benchmark configurations (test infrastructure).

One ``torch.Generator(device="cpu")`` per tensor, seed = base_seed + 1000*config + tensor_index,
values drawn in fp32 and then rounded to the storage dtype, so that the CPU oracle and the GPU
kernels consume identical bits (the reference seeds a CUDA generator, tests/test_translators.py:106-119,
whose stream cannot be reproduced on a CPU).  Every generator takes the problem sizes as arguments
so that tests can shrink them; the defaults are the sizes the benchmark configurations state.
"""

from __future__ import annotations

import math

import torch


def _gen(config: int, index: int, base_seed: int = 0) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(base_seed + 1000 * config + index)
    return g


def _randn(shape, config, index, dtype, base_seed=0):
    return torch.randn(shape, generator=_gen(config, index, base_seed), dtype=torch.float32).to(dtype)


def _rand(shape, config, index, base_seed=0):
    return torch.rand(shape, generator=_gen(config, index, base_seed), dtype=torch.float32)


def attention_inputs(B, H, S, D, dtype, config=2, base_seed=0, Skv=None):
    """Q, K, V ~ N(0,1) in [B, H, S, D]."""
    Skv = S if Skv is None else Skv
    q = _randn((B, H, S, D), config, 0, dtype, base_seed)
    k = _randn((B, H, Skv, D), config, 1, dtype, base_seed)
    v = _randn((B, H, Skv, D), config, 2, dtype, base_seed)
    return q, k, v


def decode_inputs(B=64, Hq=32, Hkv=8, L=32768, D=128, dtype=torch.bfloat16, config=3, base_seed=0):
    """q [B,Hq,D]; K, V [B,Hkv,L,D], all ~ N(0,1)."""
    q = _randn((B, Hq, D), config, 0, dtype, base_seed)
    k = _randn((B, Hkv, L, D), config, 1, dtype, base_seed)
    v = _randn((B, Hkv, L, D), config, 2, dtype, base_seed)
    return q, k, v


def selective_scan_inputs(B=8, Dm=4096, L=4096, N=16, dtype=torch.bfloat16, config=4, base_seed=0):
    """u, delta, A, Bm, Cm, Dskip, z for the Mamba-1 scan.

    delta = softplus(N(0,1) + dt_bias) with dt_bias a per-channel vector drawn once as the inverse
    soft-plus of dt ~ logU(1e-3, 1e-1) (the benchmark configuration leaves dt_bias unspecified; this
    is the usual initialisation of that parameter).  A = -exp(U(ln 1, ln 16)).
    """
    u = _randn((B, Dm, L), config, 0, dtype, base_seed)
    dt0 = torch.exp(_rand((Dm,), config, 7, base_seed) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    dt_bias = dt0 + torch.log(-torch.expm1(-dt0))
    raw = torch.randn((B, Dm, L), generator=_gen(config, 1, base_seed), dtype=torch.float32)
    delta = torch.nn.functional.softplus(raw + dt_bias[None, :, None]).to(dtype)
    A = -torch.exp(_rand((Dm, N), config, 2, base_seed) * math.log(16.0))
    Bm = _randn((B, N, L), config, 3, dtype, base_seed)
    Cm = _randn((B, N, L), config, 4, dtype, base_seed)
    Dskip = _randn((Dm,), config, 5, torch.float32, base_seed)
    z = _randn((B, Dm, L), config, 6, dtype, base_seed)
    return u, delta, A, Bm, Cm, Dskip, z


def ssd_inputs(B=4, L=8192, H=64, P=64, N=128, G=1, dtype=torch.bfloat16, config=5, base_seed=0):
    """x, dt, A, Bm, Cm for the Mamba-2 SSD scan: dt = softplus(N(0,1)) fp32, A = -exp(U(ln 1, ln 16))."""
    x = _randn((B, L, H, P), config, 0, dtype, base_seed)
    dt = torch.nn.functional.softplus(
        torch.randn((B, L, H), generator=_gen(config, 1, base_seed), dtype=torch.float32))
    A = -torch.exp(_rand((H,), config, 2, base_seed) * math.log(16.0))
    Bm = _randn((B, L, G, N), config, 3, dtype, base_seed)
    Cm = _randn((B, L, G, N), config, 4, dtype, base_seed)
    return x, dt, A, Bm, Cm
