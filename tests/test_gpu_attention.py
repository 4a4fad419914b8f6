"""GPU parity of the attention path, called through the translator's emitted module and the C ABI."""

import math
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import assert_storage_close, finish, translate_data, translate_text
from oracle import attention, inputs

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).parent / "golden" / "flash_attention_ref_tiles.npz"
BF16_ATOL = 2e-2   # max-abs-error bound for bf16 outputs
F32_ATOL = 1e-4    # max-abs-error bound for fp32 outputs
REF_F16_ATOL = 1e-3  # the reference's own bound for its f16 program (tests/test_translators.py:143)


def test_reference_shape_f16_matches_reference_golden_tiles(cuda, native_lib):
    """Non-causal f16 1x32x4096x128: the reference's problem, checked against tiles its own kernel produced."""
    g = np.load(GOLDEN)
    shape = tuple(int(s) for s in g["shape"])
    q, k, v = inputs.attention_inputs(*shape, torch.float16, config=0)
    mod = translate_data("attention_f16_1x32x4096x128")
    qd, kd, vd = q.to(cuda), k.to(cuda), v.to(cuda)
    out = torch.full(shape, float("nan"), dtype=torch.float16, device=cuda)
    mod.attention_f16(qd, kd, vd, out)
    finish()
    assert tuple(out.shape) == shape and out.dtype == torch.float16
    assert bool(torch.isfinite(out).all())
    for (head, blk), tile in zip(g["programs"], g["tiles"]):
        r0 = int(blk) * 128
        got = out[0, head, r0:r0 + 128].float().cpu()
        torch.testing.assert_close(got, torch.from_numpy(tile).float(), rtol=0, atol=REF_F16_ATOL)
    # and against the restated check function of the reference on a few whole heads
    for head in (3, 30):
        ref = attention.attention_reference(q[:, head:head + 1], k[:, head:head + 1], v[:, head:head + 1])
        torch.testing.assert_close(out[:, head:head + 1].float().cpu(), ref, rtol=0, atol=REF_F16_ATOL)


def test_other_shapes_match_kernels_emitted_by_the_reference_translator(cuda, native_lib):
    """fp32 1x4x256x64 (exact-fp32 kernel) and f16 2x4x512x128 (tcgen05 kernel), non-causal, against outputs of the
    kernels the unmodified reference translator emitted for the same HTile programs (Triton interpreter, CPU)."""
    from neptune_mlir import programs

    g = np.load(Path(__file__).parent / "golden" / "reference_translations.npz")
    for name, dtype_name, dtype, atol in (("f32_1x4x256x64", "f32", torch.float32, F32_ATOL),
                                          ("f16_2x4x512x128", "f16", torch.float16, REF_F16_ATOL)):
        B, H, S, D, tm, tn, cfg = (int(x) for x in g[f"{name}.spec"])
        q, k, v = inputs.attention_inputs(B, H, S, D, dtype, config=cfg)
        fn = f"attn_{name}"
        mod = translate_text(programs.attention_htile(fn, B, H, S, D, dtype_name, causal=False, tile_m=tm, tile_n=tn),
                             f"translated_{fn}")
        out = torch.full((B, H, S, D), float("nan"), dtype=dtype, device=cuda)
        getattr(mod, fn)(q.to(cuda), k.to(cuda), v.to(cuda), out)
        finish()
        want = torch.from_numpy(g[f"{name}.out"]).float()
        torch.testing.assert_close(out.float().cpu(), want, rtol=0, atol=atol)


@pytest.mark.parametrize("dtype,name,atol", [(torch.float16, "f16", REF_F16_ATOL), (torch.float32, "f32", F32_ATOL)])
def test_level1_program_lowered_to_htile_runs(cuda, native_lib, dtype, name, atol):
    """A Level-1 (scheduled tile IR) attention program goes through the L1 -> HTile lowering and the translator."""
    import ast
    import tempfile

    from gpu_util import exec_translated_module
    from neptune_mlir import l1, programs

    B, H, S, D = (2, 4, 512, 128) if name == "f16" else (1, 4, 256, 64)
    with tempfile.NamedTemporaryFile("w", suffix=".mlir", delete=False) as f:
        f.write(programs.attention_l1("attn_from_l1", B, H, S, D, name))
    mod = exec_translated_module(l1.translate_file(f.name), f"attn_from_l1_{name}")
    assert isinstance(l1.translate_file(f.name), ast.Module)
    q, k, v = inputs.attention_inputs(B, H, S, D, dtype, config=13)
    out = torch.full((B, H, S, D), float("nan"), dtype=dtype, device=cuda)
    mod.attn_from_l1(q.to(cuda), k.to(cuda), v.to(cuda), out)
    finish()
    torch.testing.assert_close(out.float().cpu(), attention.attention_reference(q, k, v), rtol=0, atol=atol)


def test_config1_fp32_causal(cuda, native_lib):
    """B=1, H=4, S=256, D=64 fp32 causal (exact-fp32 kernel)."""
    q, k, v = inputs.attention_inputs(1, 4, 256, 64, torch.float32, config=1)
    mod = translate_data("attention_causal_f32_1x4x256x64")
    out = torch.full((1, 4, 256, 64), float("nan"), device=cuda)
    mod.attention_causal_f32(q.to(cuda), k.to(cuda), v.to(cuda), out)
    finish()
    assert_storage_close(out, attention.attention_reference(q, k, v, causal=True), F32_ATOL)


@pytest.mark.parametrize("dtype,name,atol", [(torch.bfloat16, "bf16", BF16_ATOL), (torch.float16, "f16", 2e-3)])
@pytest.mark.parametrize("causal", [False, True])
def test_tensor_core_path_small(cuda, native_lib, dtype, name, atol, causal):
    """Ragged work per tile (1..4 kv blocks), several heads; every element against the oracle."""
    from neptune_mlir import programs

    B, H, S, D = 2, 3, 512, 128
    q, k, v = inputs.attention_inputs(B, H, S, D, dtype, config=2)
    mod = translate_text(programs.attention_htile("attn_small", B, H, S, D, name, causal=causal),
                         f"attn_small_{name}_{int(causal)}")
    out = torch.full((B, H, S, D), float("nan"), dtype=dtype, device=cuda)
    mod.attn_small(q.to(cuda), k.to(cuda), v.to(cuda), out)
    finish()
    assert_storage_close(out, attention.attention_reference(q, k, v, causal=causal), atol)
    # the program-faithful oracle (P rounded before PV, exp2 domain) is matched at least as well
    assert_storage_close(out, attention.attention_program(q, k, v, causal=causal), atol)


def test_single_tile_and_determinism(cuda, native_lib):
    from neptune_mlir import runtime

    q, k, v = (t.to(cuda) for t in inputs.attention_inputs(1, 1, 128, 128, torch.bfloat16, config=2))
    outs = []
    for _ in range(2):
        out = torch.empty_like(q)
        runtime.attn_fwd(q, k, v, out, shape=(1, 1, 128, 128), kv_len=128, dtype="bf16",
                         scale_log2=attention.scale_log2(128), causal=True)
        finish()
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    ref = attention.attention_reference(q.cpu(), k.cpu(), v.cpu(), causal=True)
    assert_storage_close(outs[0], ref, BF16_ATOL)
    torch.testing.assert_close(outs[0][0, 0, 0].float(), v[0, 0, 0].float())  # row 0 sees only key 0


def test_causal_with_longer_kv_and_large_scores(cuda, native_lib):
    """Skv > Sq (diagonal offset) and scores scaled up so that row maxima move by more than the rescale threshold."""
    from neptune_mlir import runtime

    B, H, Sq, Skv, D = 1, 2, 256, 512, 128
    q, k, v = inputs.attention_inputs(B, H, Sq, D, torch.bfloat16, config=2, Skv=Skv)
    q = (q.float() * 6).to(torch.bfloat16)
    out = torch.empty((B, H, Sq, D), dtype=torch.bfloat16, device=cuda)
    runtime.attn_fwd(q.to(cuda), k.to(cuda), v.to(cuda), out, shape=(B, H, Sq, D), kv_len=Skv, dtype="bf16",
                     scale_log2=attention.scale_log2(D), causal=True)
    finish()
    assert_storage_close(out, attention.attention_reference(q, k, v, causal=True), BF16_ATOL)


@pytest.mark.parametrize("Sq,Skv,causal", [(100, 100, True), (200, 333, True), (129, 1000, False), (1, 77, True),
                                           (300, 300, False)])
def test_lengths_that_are_not_multiples_of_the_tiles(cuda, native_lib, Sq, Skv, causal):
    """Any Sq, Skv on the tensor-core path: partial last tiles, and a neighbouring head full of infinities that
    must not leak into this head (rows past the end of a slice load as zeros, not as the next slice)."""
    from neptune_mlir import runtime

    B, H, D = 1, 3, 128
    q, k, v = inputs.attention_inputs(B, H, Sq, D, torch.bfloat16, config=51, Skv=Skv)
    k[:, 1] = float("inf")
    v[:, 1] = float("inf")
    out = torch.full((B, H, Sq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    runtime.attn_fwd(q.to(cuda), k.to(cuda), v.to(cuda), out, shape=(B, H, Sq, D), kv_len=Skv, dtype="bf16",
                     scale_log2=attention.scale_log2(D), causal=causal)
    finish()
    for h in (0, 2):
        ref = attention.attention_reference(q[:, h:h + 1], k[:, h:h + 1], v[:, h:h + 1], causal=causal)
        assert_storage_close(out[:, h:h + 1], ref, BF16_ATOL)


@pytest.mark.parametrize("Sq,Skv,causal", [(128, 128, True), (200, 200, True), (128, 300, False), (384, 384, True)])
def test_more_short_tiles_than_sms(cuda, native_lib, Sq, Skv, causal):
    """Hundreds of tiles of one to three KV blocks each: the persistent CTAs take tile after tile from the global
    counter, and the roles of a CTA run several tiles apart.  Every element against the oracle."""
    from neptune_mlir import runtime

    B, H, D = 2, 150, 128
    q, k, v = inputs.attention_inputs(B, H, Sq, D, torch.bfloat16, config=61, Skv=Skv)
    out = torch.full((B, H, Sq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    for _ in range(2):   # the second launch takes another tile counter
        runtime.attn_fwd(q.to(cuda), k.to(cuda), v.to(cuda), out, shape=(B, H, Sq, D), kv_len=Skv, dtype="bf16",
                         scale_log2=attention.scale_log2(D), causal=causal)
    finish()
    assert_storage_close(out, attention.attention_reference(q, k, v, causal=causal), BF16_ATOL)


def test_config2_full_size_sampled(cuda, native_lib):
    """B=8, H=32, S=4096, D=128 bf16 causal; sampled (batch, head, row block) tiles against the oracle."""
    B, H, S, D = 8, 32, 4096, 128
    gen = torch.Generator(device=cuda).manual_seed(2000)
    q, k, v = (torch.randn((B, H, S, D), device=cuda, dtype=torch.bfloat16, generator=gen) for _ in range(3))
    mod = translate_data("attention_causal_bf16_8x32x4096x128")
    out = torch.full((B, H, S, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.attention_causal_bf16(q, k, v, out)
    finish()
    assert bool(torch.isfinite(out).all())
    for b, h, blk in ((0, 0, 0), (0, 0, 31), (3, 17, 7), (7, 31, 31), (5, 9, 16)):
        r0 = blk * 128
        qs = q[b:b + 1, h:h + 1, r0:r0 + 128].cpu()
        ks, vs = k[b:b + 1, h:h + 1, :r0 + 128].cpu(), v[b:b + 1, h:h + 1, :r0 + 128].cpu()
        ref = attention.attention_reference(qs, ks, vs, causal=True)  # Skv - Sq offset = r0 puts the tile on the diagonal
        assert_storage_close(out[b:b + 1, h:h + 1, r0:r0 + 128], ref, BF16_ATOL)
    # softmax rows are convex combinations of V rows: outputs stay inside V's range
    assert out.float().abs().max() <= v.float().abs().max() + 1e-2


def test_runtime_checks_tensors_against_the_program(cuda, native_lib):
    mod = translate_data("attention_causal_f32_1x4x256x64")
    good = torch.zeros((1, 4, 256, 64), device=cuda)
    with pytest.raises(ValueError, match="shape"):
        mod.attention_causal_f32(good, good, good[:, :2], good)
    with pytest.raises(TypeError, match="dtype"):
        mod.attention_causal_f32(good, good, good.half(), good)
    strided = torch.zeros((1, 4, 256, 128), device=cuda)[..., ::2]
    with pytest.raises(ValueError, match="contiguous"):
        mod.attention_causal_f32(good, good, strided, good)
