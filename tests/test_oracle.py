"""The CPU oracle against the reference-derived golden tiles, and its own forms against each other."""

import hashlib
from pathlib import Path

import numpy as np
import torch

from oracle import attention, decode, inputs, selective_scan, ssd

GOLDEN = Path(__file__).parent / "golden" / "flash_attention_ref_tiles.npz"


def _sha(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.int16).numpy().tobytes())
    return h.hexdigest()


def test_attention_oracle_matches_reference_golden_tiles():
    """Tiles produced by the reference's own Triton translation (run by the Triton interpreter)."""
    g = np.load(GOLDEN)
    shape = tuple(int(s) for s in g["shape"])
    q, k, v = inputs.attention_inputs(*shape, torch.float16, config=0)
    assert _sha(q, k, v) == str(g["inputs_sha256"]), "seeded inputs differ from the ones the tiles were made from"
    for (head, blk), tile in zip(g["programs"], g["tiles"]):
        r0 = int(blk) * 128
        qs, ks, vs = q[:, head:head + 1, r0:r0 + 128], k[:, head:head + 1], v[:, head:head + 1]
        want = torch.from_numpy(tile).float()
        ref = attention.attention_reference(qs, ks, vs)[0, 0]
        prog = attention.attention_program(qs, ks, vs)[0, 0].float()
        # tests/test_translators.py:143 of the reference: rtol=0, atol=1e-3
        torch.testing.assert_close(ref, want, rtol=0, atol=1e-3)
        torch.testing.assert_close(prog, want, rtol=0, atol=1e-3)
        # the program-faithful form reproduces the reference's f16 bits almost everywhere
        assert (prog == want).float().mean() > 0.98
        assert (prog - want).abs().max() <= 2 ** -13


TRANSLATIONS = Path(__file__).parent / "golden" / "reference_translations.npz"
TRANSLATION_CASES = {"f32_1x4x256x64": (torch.float32, 1e-4), "f16_2x4x512x128": (torch.float16, 1e-3)}


def _sha_bytes(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def test_attention_oracle_matches_reference_translator_at_other_shapes():
    """Outputs of kernels that the UNMODIFIED reference translator emitted for fp32 and for another f16 shape
    (tests/golden/make_reference_translations.py), run over their whole grids by the Triton interpreter."""
    g = np.load(TRANSLATIONS)
    for name, (dtype, atol) in TRANSLATION_CASES.items():
        B, H, S, D, tm, tn, cfg = (int(x) for x in g[f"{name}.spec"])
        q, k, v = inputs.attention_inputs(B, H, S, D, dtype, config=cfg)
        assert _sha_bytes(q, k, v) == str(g[f"{name}.inputs_sha256"])
        want = torch.from_numpy(g[f"{name}.out"]).float()
        ref = attention.attention_reference(q, k, v)
        prog = attention.attention_program(q, k, v, kv_block=tn).float()
        torch.testing.assert_close(ref, want, rtol=0, atol=atol)
        torch.testing.assert_close(prog, want, rtol=0, atol=atol)


def test_attention_forms_agree_causal_and_not():
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2), (torch.float16, 2e-3)):
        q, k, v = inputs.attention_inputs(1, 2, 256, 64, dtype, config=1)
        for causal in (False, True):
            ref = attention.attention_reference(q, k, v, causal=causal)
            prog = attention.attention_program(q, k, v, causal=causal).float()
            assert (ref - prog).abs().max() < tol


def test_attention_causal_first_row_is_v0():
    q, k, v = inputs.attention_inputs(1, 1, 128, 64, torch.float32, config=1)
    ref = attention.attention_reference(q, k, v, causal=True)
    torch.testing.assert_close(ref[0, 0, 0], v[0, 0, 0])


def test_decode_split_equals_direct():
    q, k, v = inputs.decode_inputs(B=2, Hq=8, Hkv=2, L=512, D=128)
    direct = decode.decode_reference(q, k, v)
    m, l, o = decode.decode_partials(q, k, v, n_splits=4)
    torch.testing.assert_close(decode.combine_partials(m, l, o), direct, rtol=1e-5, atol=1e-5)
    # merging merged partials (the cross-GPU step) gives the same result
    m2 = torch.stack([m[..., :2].amax(-1), m[..., 2:].amax(-1)], dim=-1)
    w = torch.exp(m.view(2, 8, 2, 2) - m2[..., None])
    l2 = (w * l.view(2, 8, 2, 2)).sum(-1)
    o2 = (w[..., None] * o.view(2, 8, 2, 2, 128)).sum(-2)
    torch.testing.assert_close(decode.combine_partials(m2, l2, o2), direct, rtol=1e-5, atol=1e-5)


def test_selective_scan_against_scalar_loops():
    u, delta, A, Bm, Cm, Dk, z = inputs.selective_scan_inputs(B=1, Dm=3, L=12, N=4, dtype=torch.float32)
    got = selective_scan.selective_scan_reference(u, delta, A, Bm, Cm, Dk, z)
    for d in range(3):
        h = [0.0] * 4
        for t in range(12):
            y = 0.0
            for n in range(4):
                h[n] = float(torch.exp(delta[0, d, t] * A[d, n])) * h[n] + float(delta[0, d, t] * Bm[0, n, t] * u[0, d, t])
                y += float(Cm[0, n, t]) * h[n]
            y += float(Dk[d] * u[0, d, t])
            zz = float(z[0, d, t])
            assert abs(y * zz / (1 + np.exp(-zz)) - float(got[0, d, t])) < 1e-4


def test_ssd_chunked_equals_sequential():
    x, dt, A, Bm, Cm = inputs.ssd_inputs(B=1, L=256, H=4, P=64, N=128, G=1, dtype=torch.float32)
    seq = ssd.ssd_reference(x, dt, A, Bm, Cm)
    for chunk in (64, 128, 256):
        torch.testing.assert_close(ssd.ssd_chunked(x, dt, A, Bm, Cm, chunk), seq, rtol=1e-4, atol=1e-3)


def test_ssd_groups():
    x, dt, A, Bm, Cm = inputs.ssd_inputs(B=1, L=128, H=4, P=64, N=128, G=2, dtype=torch.float32)
    seq = ssd.ssd_reference(x, dt, A, Bm, Cm)
    torch.testing.assert_close(ssd.ssd_chunked(x, dt, A, Bm, Cm, 64), seq, rtol=1e-4, atol=1e-3)
