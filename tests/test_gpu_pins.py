"""Whole-configuration parity on the GPU, and independent pins for the operators the reference does not have.

The reference project evaluates only non-causal f16 attention; causal / bf16 attention, split-K decode and both
scans are defined by this build's oracle alone.  These tests (a) compare EVERY element of the full benchmark
configurations with an fp64 / fp32 evaluation of the oracle's definitions on the device (the sampled CPU
comparisons in the other test files cover a few units only), and (b) compare the kernels with third-party
implementations of the same operators that ship in this image, which were written independently of this build.
Every test prints the measured error so that a run with ``-s`` doubles as the parity report.

Tolerances: max-abs-error 2e-2 for bf16 outputs and 1e-4 for fp32 outputs, as the benchmark specification says.
For the two scans, whose outputs are not bounded by the inputs (|y| reaches several hundred, where one bf16
unit in the last place is 2.0), an element also passes if it is one of the two bf16 values that bracket the fp64
result, i.e. if it is as close as the output format can express; what may fall outside both rules is bounded
and stated per test.
"""

import math

import pytest
import torch

import gpu_checkers as chk
from gpu_util import finish, translate_data
from oracle import attention, decode, inputs, selective_scan, ssd

pytestmark = pytest.mark.gpu

BF16_ATOL = 2e-2
F32_ATOL = 1e-4
LOG2E = math.log2(math.e)


def _report(name, **kv):
    print(f"[parity] {name}: " + ", ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in kv.items()))


def _third_party(fn, *args, **kw):
    try:
        return fn(*args, **kw)
    except chk.Unavailable as exc:
        pytest.skip(f"third-party checker not usable on this machine: {exc}")


# ------------------------------------------------------------------ the device-side checkers against the CPU oracle
def test_device_checkers_agree_with_the_cpu_oracle(cuda):
    """Small cases: the fp64 device evaluations and the CPU oracle are the same functions."""
    q, k, v = inputs.attention_inputs(1, 2, 256, 64, torch.float32, config=1)
    ref = attention.attention_reference(q, k, v, causal=True)
    got = chk.sdpa_math(q.to(cuda), k.to(cuda), v.to(cuda), causal=True, dtype=torch.float64)
    assert (got.cpu().float() - ref).abs().max().item() <= 2e-6
    dq, dk, dv = inputs.decode_inputs(B=2, Hq=8, Hkv=2, L=512, D=128)
    assert (chk.decode_fp32(dq.to(cuda), dk.to(cuda), dv.to(cuda)).cpu() - decode.decode_reference(dq, dk, dv)).abs().max() <= 2e-6
    args = inputs.selective_scan_inputs(B=1, Dm=32, L=128, N=16)
    got = chk.selective_scan_fp64(*(a.to(cuda) for a in args)).cpu().float()
    ref = selective_scan.selective_scan_reference(*args)
    assert (got - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())
    sargs = inputs.ssd_inputs(B=1, L=128, H=2, P=64, N=128, G=1)
    got = chk.ssd_fp64(*(a.to(cuda) for a in sargs)).cpu().float()
    ref = ssd.ssd_reference(*sargs)
    assert (got - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())
    # the bracket helper: every bf16 value is its own bracket, anything else sits strictly inside one ulp
    r = torch.tensor([1.0, 1.001, -3.3, 300.7, -0.0123, 0.0], device=cuda)
    lo, hi = chk.bf16_neighbours(r)
    assert bool(((lo <= r) & (r <= hi)).all()) and lo[0] == hi[0] == 1.0 and hi[3] - lo[3] == 2.0


# ------------------------------------------------------------------ attention
def test_config1_fp32_causal_whole_against_fp64(cuda, native_lib):
    q, k, v = (t.to(cuda) for t in inputs.attention_inputs(1, 4, 256, 64, torch.float32, config=1))
    mod = translate_data("attention_causal_f32_1x4x256x64")
    out = torch.full((1, 4, 256, 64), float("nan"), device=cuda)
    mod.attention_causal_f32(q, k, v, out)
    finish()
    ref = chk.sdpa_math(q, k, v, causal=True, dtype=torch.float64)
    err = (out.double() - ref).abs().max().item()
    _report("config 1 attention fp32 vs fp64 softmax", max_abs_err=err)
    assert err <= F32_ATOL


def test_config2_whole_against_fp32_softmax_and_flash_attn(cuda, native_lib):
    """B=8, H=32, S=4096, D=128 causal bf16: all 134 M output elements."""
    B, H, S, D = 8, 32, 4096, 128
    gen = torch.Generator(device=cuda).manual_seed(2000)
    q, k, v = (torch.randn((B, H, S, D), device=cuda, dtype=torch.bfloat16, generator=gen) for _ in range(3))
    mod = translate_data("attention_causal_bf16_8x32x4096x128")
    out = torch.full((B, H, S, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.attention_causal_bf16(q, k, v, out)
    finish()
    assert bool(torch.isfinite(out).all())
    worst = 0.0
    for b in range(B):
        for h0 in range(0, H, 8):           # 8 heads at a time: 8 x 4096^2 fp32 scores = 0.5 GB
            ref = chk.sdpa_math(q[b:b + 1, h0:h0 + 8], k[b:b + 1, h0:h0 + 8], v[b:b + 1, h0:h0 + 8], causal=True)
            worst = max(worst, (out[b:b + 1, h0:h0 + 8].float() - ref).abs().max().item())
    _report("config 2 attention bf16 vs fp32 softmax (whole)", max_abs_err=worst)
    assert worst <= BF16_ATOL
    other = _third_party(chk.flash_attn_prefill, q, k, v, True)
    diff = (out.float() - other.float()).abs().max().item()
    _report("config 2 attention bf16 vs flash-attn (whole)", max_abs_diff=diff)
    assert diff <= BF16_ATOL


# ------------------------------------------------------------------ decode
def _decode_config3(cuda):
    B, Hq, Hkv, L, D, S = 64, 32, 8, 32768, 128, 16
    gen = torch.Generator(device=cuda).manual_seed(3000)
    q = torch.randn((B, Hq, D), device=cuda, dtype=torch.bfloat16, generator=gen)
    k = torch.randn((B, Hkv, L, D), device=cuda, dtype=torch.bfloat16, generator=gen)
    v = torch.randn((B, Hkv, L, D), device=cuda, dtype=torch.bfloat16, generator=gen)
    mod = translate_data("decode_splitk_bf16_64x32x8x32768x128")
    partials = torch.full((B, Hq, S, D + 2), float("nan"), device=cuda)
    out = torch.full((B, Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.decode_splitk_bf16(q, k, v, partials, out)
    finish()
    return q, k, v, out


def test_config3_whole_against_fp32_softmax_and_third_party_decoders(cuda, native_lib):
    """All 64 sequences of B=64, Hq=32, Hkv=8, L=32768, D=128."""
    q, k, v, out = _decode_config3(cuda)
    assert bool(torch.isfinite(out).all())
    ref = chk.decode_fp32(q, k, v)
    err = (out.float() - ref).abs().max().item()
    _report("config 3 decode bf16 vs fp32 softmax (whole)", max_abs_err=err)
    assert err <= BF16_ATOL
    try:
        fa = chk.flash_attn_decode(q, k, v)
        d = (out.float() - fa.float()).abs().max().item()
        _report("config 3 decode vs flash-attn kv-cache decode (whole)", max_abs_diff=d)
        assert d <= BF16_ATOL
    except chk.Unavailable as exc:
        print(f"[parity] flash-attn decode unavailable: {exc}")
    try:
        worst = 0.0
        for b in (0, 17, 63):
            fi = chk.flashinfer_decode_one(q[b], k[b], v[b])
            worst = max(worst, (out[b].float() - fi.float()).abs().max().item())
        _report("config 3 decode vs FlashInfer single decode (3 sequences)", max_abs_diff=worst)
        assert worst <= BF16_ATOL
    except chk.Unavailable as exc:
        print(f"[parity] FlashInfer decode unavailable: {exc}")
    del k, v
    torch.cuda.empty_cache()


# ------------------------------------------------------------------ Mamba-1
def test_config4_whole_against_fp64_and_vllm(cuda, native_lib):
    """B=8, D=4096, L=4096, N=16: every element against the fp64 recurrence, and against vLLM's CUDA scan."""
    B, Dm, L, N = 8, 4096, 4096, 16
    args = [a.to(cuda) for a in inputs.selective_scan_inputs(B=B, Dm=Dm, L=L, N=N)]
    mod = translate_data("selective_scan_bf16_8x4096x4096")
    out = torch.full((B, Dm, L), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.selective_scan_bf16(*args, out)
    finish()
    assert bool(torch.isfinite(out).all())
    ref = chk.selective_scan_fp64(*args)
    st = chk.parity_stats(out, ref, BF16_ATOL)
    _report("config 4 selective scan vs fp64 (whole)", **st)
    # every element is within 2e-2 or is one of the two bf16 values around the exact result
    assert st["outside"] == 0, st
    assert st["rms_rel"] <= 2.0 ** -8
    other = _third_party(chk.vllm_selective_scan, *args)
    st_other = chk.parity_stats(other, ref, BF16_ATOL)
    _report("vLLM selective scan vs fp64 (whole), for comparison", **st_other)
    diff = (out.float() - other.float()).abs()
    lo, hi = chk.bf16_neighbours(ref)
    # two implementations that each land next to the exact value differ by at most two brackets (hi - lo)
    excess = (diff - torch.maximum(2 * (hi - lo), torch.full_like(diff, BF16_ATOL))).max().item()
    _report("config 4 selective scan vs vLLM (whole)", max_abs_diff=diff.max().item(), excess_over_two_ulps=excess)
    assert excess <= 0
    assert st["max_abs_err"] <= 1.5 * st_other["max_abs_err"] + BF16_ATOL


# ------------------------------------------------------------------ Mamba-2
def test_config5_whole_against_fp64_and_third_party(cuda, native_lib):
    """B=4, L=8192, H=64, P=64, N=128, chunk 256: every element against the fp64 recurrence.

    The intra-chunk products run on bf16 tensor-core operands (the specification asks for exactly that), three of
    which are computed values rounded to bf16 (decayed C.B^T, decay-weighted x, the state entering a step), so an
    error of a few 2^-9 of the summed terms' magnitude is inherent; vLLM's and FlashInfer's kernels make the same
    roundings and are measured beside it."""
    from neptune_mlir import runtime

    B, L, H, P, N, G, chunk = 4, 8192, 64, 64, 128, 1, 256
    args = [a.to(cuda) for a in inputs.ssd_inputs(B=B, L=L, H=H, P=P, N=N, G=G)]
    x, dt, A, Bm, Cm = args
    mod = translate_data("ssd_chunk_scan_bf16_4x8192x64x64")
    ws = torch.empty(runtime.ssd_workspace_bytes(B, L, H, P, N, G, chunk), dtype=torch.uint8, device=cuda)
    y = torch.full((B, L, H, P), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.ssd_chunk_scan_bf16(x, dt, A, Bm, Cm, ws, y)
    finish()
    runtime.check_workspace_status(ws)
    assert bool(torch.isfinite(y).all())
    ref = chk.ssd_fp64(*args)
    st = chk.parity_stats(y, ref, BF16_ATOL)
    _report("config 5 SSD vs fp64 (whole)", **st)
    assert st["rms_rel"] <= 2.0 ** -8
    assert st["max_abs_err"] <= BF16_ATOL * st["rms_ref"] + 2.0 ** -7 * st["max_abs_ref"]
    measured = {}
    for name, fn in (("vLLM", lambda: chk.vllm_ssd(x, dt, A, Bm, Cm, chunk)),
                     ("FlashInfer", lambda: chk.flashinfer_ssd(x, dt, A, Bm, Cm, 128))):
        try:
            other = fn()
        except chk.Unavailable as exc:
            print(f"[parity] {name} SSD unavailable: {exc}")
            continue
        measured[name] = chk.parity_stats(other, ref, BF16_ATOL)
        _report(f"{name} SSD vs fp64 (whole), for comparison", **measured[name])
        _report(f"config 5 SSD vs {name} (whole)", max_abs_diff=(y.float() - other.float()).abs().max().item())
    if not measured:
        pytest.skip("no third-party SSD kernel usable on this machine")
    # no worse than the best independent kernel by more than a rounding's worth
    best = min(m["rms_rel"] for m in measured.values())
    assert st["rms_rel"] <= 1.25 * best + 2.0 ** -10, (st, measured)
    best_out = min(m["outside_share"] for m in measured.values())
    assert st["outside_share"] <= 1.25 * best_out + 1e-4, (st, measured)
