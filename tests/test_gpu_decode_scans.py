"""GPU parity of split-K decode, the Mamba-1 selective scan and the Mamba-2 SSD scan."""

import math

import pytest
import torch

from gpu_util import assert_rms_close, assert_storage_close, finish, translate_data, translate_text
from oracle import decode, inputs, selective_scan, ssd

pytestmark = pytest.mark.gpu

BF16_ATOL = 2e-2
BF16_ULP = 2.0 ** -8   # one bf16 unit in the last place, relative
LOG2E = math.log2(math.e)


# ------------------------------------------------------------------ decode
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4), (4, 2), (8, 1)])
def test_decode_small_all_group_sizes(cuda, native_lib, Hq, Hkv):
    from neptune_mlir import programs

    B, L, D, S = 2, 1024, 128, 4
    q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D)
    mod = translate_text(programs.decode_splitk_decl("dec", B, Hq, Hkv, L, D, S), f"dec_{Hq}_{Hkv}")
    partials = torch.full((B, Hq, S, D + 2), float("nan"), device=cuda)
    out = torch.full((B, Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.dec(q.to(cuda), k.to(cuda), v.to(cuda), partials, out)
    finish()
    assert_storage_close(out, decode.decode_reference(q, k, v), BF16_ATOL)
    # per-split partials against the oracle's split form (kernel keeps m in the exp2 domain)
    m, l, o = decode.decode_partials(q, k, v, S)
    p = partials.cpu()
    torch.testing.assert_close(p[..., D], m * LOG2E, rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(p[..., D + 1], l, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(p[..., :D], o, rtol=1e-3, atol=2e-3)


@pytest.mark.parametrize("dtype,name,tile_n,atol", [(torch.bfloat16, "bf16", 64, 2e-2), (torch.float16, "f16", 128, 2e-3)])
def test_decode_program_spelled_in_htile_ops(cuda, native_lib, dtype, name, tile_n, atol):
    """The decode + combine program written op by op in HTile (two gpu.launch regions) runs through the translator
    like the declaration does, partials included."""
    from neptune_mlir import programs

    B, Hq, Hkv, L, D, S = 2, 16, 4, 2048, 128, 8
    q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D, dtype=dtype)
    mod = translate_text(programs.decode_splitk_htile("dec_prog", B, Hq, Hkv, L, D, S, name, tile_n=tile_n), f"dec_prog_{name}")
    partials = torch.full((B, Hq, S, D + 2), float("nan"), device=cuda)
    out = torch.full((B, Hq, D), float("nan"), dtype=dtype, device=cuda)
    mod.dec_prog(q.to(cuda), k.to(cuda), v.to(cuda), partials, out)
    finish()
    assert_storage_close(out, decode.decode_reference(q, k, v), atol)
    m, l, o = decode.decode_partials(q, k, v, S)
    p = partials.cpu()
    torch.testing.assert_close(p[..., D] / LOG2E, m, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(p[..., D + 1], l, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(p[..., :D], o, rtol=1e-3, atol=2e-3)


def test_decode_ragged_split_and_f16(cuda, native_lib):
    """Split length 48 is not a multiple of the 64-row CTA step: the tail rows are masked."""
    from neptune_mlir import runtime

    B, Hq, Hkv, L, D, S = 1, 8, 2, 192, 128, 4
    q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D, dtype=torch.float16)
    partials = torch.empty((B, Hq, S, D + 2), device=cuda)
    out = torch.empty((B, Hq, D), dtype=torch.float16, device=cuda)
    runtime.decode_splitk(q.to(cuda), k.to(cuda), v.to(cuda), partials, out, B=B, Hq=Hq, Hkv=Hkv, L=L, D=D,
                          n_splits=S, dtype="f16", scale_log2=LOG2E / math.sqrt(D))
    finish()
    assert_storage_close(out, decode.decode_reference(q, k, v), 2e-3)


def test_decode_splits_that_do_not_divide_the_length(cuda, native_lib):
    """n_splits = 37 over 1000 rows: parts of 27 and 28 rows, per-split partials checked against the oracle."""
    from neptune_mlir import runtime

    B, Hq, Hkv, L, D, S = 2, 8, 2, 1000, 128, 37
    q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D, dtype=torch.bfloat16)
    partials = torch.full((B, Hq, S, D + 2), float("nan"), device=cuda)
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=cuda)
    runtime.decode_splitk(q.to(cuda), k.to(cuda), v.to(cuda), partials, out, B=B, Hq=Hq, Hkv=Hkv, L=L, D=D,
                          n_splits=S, dtype="bf16", scale_log2=LOG2E / math.sqrt(D))
    finish()
    assert_storage_close(out, decode.decode_reference(q, k, v), 2e-2)
    m, l, o = decode.decode_partials(q, k, v, S)
    p = partials.cpu()
    torch.testing.assert_close(p[..., D] / LOG2E, m, rtol=1e-4, atol=1e-4)     # kernel keeps m in the exp2 domain
    torch.testing.assert_close(p[..., D + 1], l, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(p[..., :D], o, rtol=1e-3, atol=2e-3)


@pytest.mark.parametrize("dtype,name,atol", [(torch.bfloat16, "bf16", 2e-2), (torch.float16, "f16", 2e-3)])
def test_decode_long_ragged_splits_through_the_bulk_copy_ring(cuda, native_lib, dtype, name, atol):
    """Splits of 333/334 rows: long enough for the ring of TMA bulk copies, not a multiple of its 64-row stages,
    and with a last stage that is only partly filled."""
    from neptune_mlir import runtime

    B, Hq, Hkv, L, D, S = 2, 8, 2, 1000, 128, 3
    q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D, dtype=dtype)
    partials = torch.full((B, Hq, S, D + 2), float("nan"), device=cuda)
    out = torch.full((B, Hq, D), float("nan"), dtype=dtype, device=cuda)
    runtime.decode_splitk(q.to(cuda), k.to(cuda), v.to(cuda), partials, out, B=B, Hq=Hq, Hkv=Hkv, L=L, D=D,
                          n_splits=S, dtype=name, scale_log2=LOG2E / math.sqrt(D))
    finish()
    assert_storage_close(out, decode.decode_reference(q, k, v), atol)
    m, l, o = decode.decode_partials(q, k, v, S)
    p = partials.cpu()
    torch.testing.assert_close(p[..., D] / LOG2E, m, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(p[..., D + 1], l, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(p[..., :D], o, rtol=1e-3, atol=2e-3)


@pytest.mark.parametrize("Hq,Hkv,n_splits", [(8, 2, 3), (8, 8, 1), (16, 2, 4)])
def test_decode_over_a_paged_cache_with_ragged_lengths(cuda, native_lib, Hq, Hkv, n_splits):
    """Pages of 64 rows scattered through a pool, one block table row per sequence, lengths from 0 to 1000
    (0 rows -> zeros; lengths that end inside a page; fewer pages than splits)."""
    from neptune_mlir import runtime

    D, page = 128, 64
    lens = [1000, 0, 1, 63, 64, 65, 500]
    B, max_pages = len(lens), 16
    q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=max_pages * page, D=D, dtype=torch.bfloat16, config=41)
    used_pages = B * max_pages + 5
    num_pages = used_pages + 1                          # one more page, which no sequence owns (see below)
    gen = torch.Generator().manual_seed(7)
    perm = torch.randperm(used_pages, generator=gen)[:B * max_pages].view(B, max_pages).to(torch.int32)
    k_pool = torch.zeros((num_pages, Hkv, page, D), dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    for b in range(B):
        for p in range(max_pages):
            k_pool[perm[b, p]] = k[b, :, p * page:(p + 1) * page]
            v_pool[perm[b, p]] = v[b, :, p * page:(p + 1) * page]
    # entries past a sequence's last page must not be read: point them at a page of the pool that holds NaN, so
    # that a stray read shows up as a wrong (non-finite) result rather than as an access outside the pool
    sentinel = num_pages - 1
    assert sentinel not in perm
    k_pool[sentinel] = float("nan")
    v_pool[sentinel] = float("nan")
    table = perm.clone()
    for b, n in enumerate(lens):
        table[b, (n + page - 1) // page:] = sentinel
    partials = torch.full((B, Hq, n_splits, D + 2), float("nan"), device=cuda)
    out = torch.full((B, Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    if n_splits == 3:  # once through an emitted module, the way the other operators are called
        from neptune_mlir import programs

        mod = translate_text(programs.decode_paged_decl("dp", B, Hq, Hkv, num_pages, max_pages, D, n_splits), "paged_dp")
        mod.dp(q.to(cuda), k_pool.to(cuda), v_pool.to(cuda), table.to(cuda),
               torch.tensor(lens, dtype=torch.int32, device=cuda), partials, out)
    else:
        runtime.decode_paged(q.to(cuda), k_pool.to(cuda), v_pool.to(cuda), table.to(cuda),
                             torch.tensor(lens, dtype=torch.int32, device=cuda), partials, out, B=B, Hq=Hq, Hkv=Hkv,
                             max_pages=max_pages, page_size=page, D=D, n_splits=n_splits, dtype="bf16",
                             scale_log2=LOG2E / math.sqrt(D))
    finish()
    for b, n in enumerate(lens):
        if n == 0:
            assert bool((out[b] == 0).all())
            continue
        ref = decode.decode_reference(q[b:b + 1], k[b:b + 1, :, :n], v[b:b + 1, :, :n])
        assert_storage_close(out[b:b + 1], ref, BF16_ATOL)


def test_paged_decode_refuses_a_table_entry_outside_the_pool(cuda, native_lib):
    """A block-table entry that is not a page of the pool is never dereferenced: the split that meets it yields
    NaN, the status words name the entry, and the other sequences are computed as usual.  A length beyond what a
    table row can address is cut to the row."""
    from neptune_mlir import native, runtime

    D, page, Hq, Hkv, n_splits = 128, 64, 8, 2, 2
    B, max_pages = 3, 8
    num_pages = B * max_pages
    L = max_pages * page
    q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D, dtype=torch.bfloat16, config=42)
    table = torch.arange(num_pages, dtype=torch.int32).view(B, max_pages)
    k_pool = k.view(B, Hkv, max_pages, page, D).permute(0, 2, 1, 3, 4).reshape(num_pages, Hkv, page, D).contiguous()
    v_pool = v.view(B, Hkv, max_pages, page, D).permute(0, 2, 1, 3, 4).reshape(num_pages, Hkv, page, D).contiguous()
    lens = torch.tensor([L, L + 1000, L], dtype=torch.int32)          # sequence 1 claims more rows than its row holds
    bad = table.clone()
    bad[2, 5] = num_pages + 7                                         # sequence 2 has an entry outside the pool
    partials = torch.full((B, Hq, n_splits, D + 2), float("nan"), device=cuda)
    out = torch.full((B, Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    finish()                                                          # status words clear before the call
    runtime.decode_paged(q.to(cuda), k_pool.to(cuda), v_pool.to(cuda), bad.to(cuda), lens.to(cuda), partials, out,
                         B=B, Hq=Hq, Hkv=Hkv, max_pages=max_pages, page_size=page, D=D, n_splits=n_splits, dtype="bf16",
                         scale_log2=LOG2E / math.sqrt(D))
    torch.cuda.synchronize()
    with pytest.raises(ValueError, match=f"block table entry {num_pages + 7} is outside the page pool"):
        runtime.check_status(cuda)
    runtime.check_status(cuda)                                        # reading the status cleared it
    assert bool(torch.isnan(out[2].float()).all())
    for b in (0, 1):
        ref = decode.decode_reference(q[b:b + 1], k[b:b + 1], v[b:b + 1])
        assert_storage_close(out[b:b + 1], ref, BF16_ATOL)
    assert native.lib().nb200_last_error() is not None


def test_decode_auto_split_count(cuda, native_lib):
    """n_splits = 0 in the declaration: the library picks the count for this GPU, bounded by the partials memref."""
    from neptune_mlir import native, programs

    B, Hq, Hkv, L, D, cap = 2, 8, 2, 8192, 128, 64
    n = native.lib().nb200_decode_auto_splits(B, Hkv, L, cap)
    assert 1 <= n <= cap and L // n >= 64
    q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D)
    mod = translate_text(programs.decode_splitk_decl("dec_auto", B, Hq, Hkv, L, D, cap, auto_splits=True), "dec_auto")
    partials = torch.full((B, Hq, cap, D + 2), float("nan"), device=cuda)
    out = torch.full((B, Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.dec_auto(q.to(cuda), k.to(cuda), v.to(cuda), partials, out)
    finish()
    assert_storage_close(out, decode.decode_reference(q, k, v), BF16_ATOL)
    # a whole number of waves where the problem is large enough to have a choice
    sms = torch.cuda.get_device_properties(cuda).multi_processor_count
    big = native.lib().nb200_decode_auto_splits(8, 8, 32768, 0)
    waves = big * 64 / (2 * sms)
    assert waves - int(waves) > 0.9 or waves == int(waves), (big, waves)


def test_combine_with_gather_strides_and_partial_output(cuda, native_lib):
    """The cross-GPU merge: per-rank partials laid out [rank, rows, D+2] merge to the same answer."""
    from neptune_mlir import runtime
    from neptune_mlir.sharding import gathered_strides

    B, Hq, Hkv, L, D, R = 1, 8, 2, 2048, 128, 4
    q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D)
    qd = q.to(cuda)
    per_rank = []
    for r in range(R):                                     # each "rank" owns a quarter of the sequence
        ks = k[:, :, r * L // R:(r + 1) * L // R].contiguous().to(cuda)
        vs = v[:, :, r * L // R:(r + 1) * L // R].contiguous().to(cuda)
        partials = torch.empty((B, Hq, 2, D + 2), device=cuda)
        tmp = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=cuda)
        runtime.decode_splitk(qd, ks, vs, partials, tmp, B=B, Hq=Hq, Hkv=Hkv, L=L // R, D=D, n_splits=2,
                              dtype="bf16", scale_log2=LOG2E / math.sqrt(D))
        local = torch.empty((B * Hq, D + 2), device=cuda)
        runtime.decode_combine(partials, local, rows=B * Hq, D=D, n_splits=2, row_stride=2 * (D + 2),
                               split_stride=D + 2, out_dtype="f32")
        per_rank.append(local)
    gathered = torch.stack(per_rank)                       # what an all-gather delivers
    rs, ss = gathered_strides(B * Hq, D + 2)
    out = torch.empty((B * Hq, D), dtype=torch.bfloat16, device=cuda)
    runtime.decode_combine(gathered, out, rows=B * Hq, D=D, n_splits=R, row_stride=rs, split_stride=ss,
                           out_dtype="bf16")
    finish()
    assert_storage_close(out.view(B, Hq, D), decode.decode_reference(q, k, v), BF16_ATOL)


def test_decode_config3_full_size_sampled(cuda, native_lib):
    """B=64, Hq=32, Hkv=8, L=32768, D=128, 16 splits; sampled sequences against the oracle."""
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
    assert bool(torch.isfinite(out).all())
    for b in (0, 31, 63):
        ref = decode.decode_reference(q[b:b + 1].cpu(), k[b:b + 1].cpu(), v[b:b + 1].cpu())
        assert_storage_close(out[b:b + 1], ref, BF16_ATOL)
    del k, v
    torch.cuda.empty_cache()


# ------------------------------------------------------------------ Mamba-1
@pytest.mark.parametrize("dtype,name", [(torch.bfloat16, "bf16"), (torch.float16, "f16")])
def test_selective_scan_small(cuda, native_lib, dtype, name):
    from neptune_mlir import programs

    B, Dm, L, N = 2, 64, 256, 16
    args = inputs.selective_scan_inputs(B=B, Dm=Dm, L=L, N=N, dtype=dtype)
    mod = translate_text(programs.selective_scan_decl("scan", B, Dm, L, N, name), f"scan_{name}")
    out = torch.full((B, Dm, L), float("nan"), dtype=dtype, device=cuda)
    mod.scan(*(a.to(cuda) for a in args), out)
    finish()
    ref = selective_scan.selective_scan_reference(*args)
    assert_storage_close(out, ref, BF16_ATOL if dtype == torch.bfloat16 else 4e-3,
                         BF16_ULP if dtype == torch.bfloat16 else 2.0 ** -10, scale_by_rms=True)
    assert_rms_close(out, ref, 2.0 ** -8)


def test_selective_scan_mid_size_takes_four_states_per_thread(cuda, native_lib):
    """B=4, D=4096, L=128: 512 CTAs, the size at which the launcher picks 4 states per thread on a 148-SM GPU
    (the small cases above take 2, the full configuration 8); sampled channels against the oracle."""
    from neptune_mlir import runtime

    B, Dm, L, N = 4, 4096, 128, 16
    args = inputs.selective_scan_inputs(B=B, Dm=Dm, L=L, N=N, dtype=torch.bfloat16)
    out = torch.full((B, Dm, L), float("nan"), dtype=torch.bfloat16, device=cuda)
    runtime.selective_scan(*(a.to(cuda) for a in args), out, B=B, Dm=Dm, L=L, N=N, dtype="bf16")
    finish()
    assert bool(torch.isfinite(out.float()).all())
    ref = selective_scan.selective_scan_reference(*args)
    assert_storage_close(out, ref, BF16_ATOL, BF16_ULP, scale_by_rms=True)
    assert_rms_close(out, ref, 2.0 ** -8)


def test_selective_scan_config4_full_size_sampled(cuda, native_lib):
    """B=8, D=4096, L=4096, N=16: channels are independent, so a sample of them is checked in full."""
    B, Dm, L, N = 8, 4096, 4096, 16
    u, delta, A, Bm, Cm, Dk, z = (a.to(cuda) for a in inputs.selective_scan_inputs(B=B, Dm=Dm, L=L, N=N))
    mod = translate_data("selective_scan_bf16_8x4096x4096")
    out = torch.full((B, Dm, L), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.selective_scan_bf16(u, delta, A, Bm, Cm, Dk, z, out)
    finish()
    assert bool(torch.isfinite(out).all())
    ch = torch.tensor([0, 1, 31, 32, 2047, 4095], device=cuda)
    ref = selective_scan.selective_scan_reference(
        u[:, ch].cpu(), delta[:, ch].cpu(), A[ch].cpu(), Bm.cpu(), Cm.cpu(), Dk[ch].cpu(), z[:, ch].cpu())
    assert_storage_close(out[:, ch], ref, BF16_ATOL, BF16_ULP, scale_by_rms=True)
    assert_rms_close(out[:, ch], ref, 2.0 ** -8)


# ------------------------------------------------------------------ Mamba-2
@pytest.mark.parametrize("chunk", [64, 128, 256])
@pytest.mark.parametrize("G", [1, 2])
def test_ssd_small(cuda, native_lib, chunk, G):
    from neptune_mlir import programs, runtime

    B, L, H, P, N = 2, 512, 4, 64, 128
    x, dt, A, Bm, Cm = inputs.ssd_inputs(B=B, L=L, H=H, P=P, N=N, G=G)
    ws_bytes = runtime.ssd_workspace_bytes(B, L, H, P, N, G, chunk)
    mod = translate_text(programs.ssd_chunk_scan_decl("ssd_small", B, L, H, P, N, G, chunk, ws_bytes), f"ssd_{chunk}_{G}")
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=cuda)
    y = torch.full((B, L, H, P), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.ssd_small(x.to(cuda), dt.to(cuda), A.to(cuda), Bm.to(cuda), Cm.to(cuda), ws, y)
    finish()
    runtime.check_workspace_status(ws)
    ref = ssd.ssd_reference(x, dt, A, Bm, Cm)
    assert_storage_close(y, ref, BF16_ATOL, 2 * BF16_ULP, scale_by_rms=True)
    assert_rms_close(y, ref, 2.0 ** -8)
    # against the chunked form with the kernel's operand roundings the average error is an output ulp
    faithful = ssd.ssd_chunked(x, dt, A, Bm, Cm, chunk, round_to=torch.bfloat16)
    assert_rms_close(y, faithful, 2.0 ** -8)


def test_ssd_head_count_not_a_multiple_of_four(cuda, native_lib):
    """With H % 4 != 0 a row of dt is not a multiple of 16 bytes: the kernel reads dt with plain loads instead of TMA."""
    from neptune_mlir import runtime

    B, L, H, P, N, G, chunk = 1, 384, 3, 64, 128, 1, 128
    x, dt, A, Bm, Cm = inputs.ssd_inputs(B=B, L=L, H=H, P=P, N=N, G=G)
    ws = torch.empty(runtime.ssd_workspace_bytes(B, L, H, P, N, G, chunk), dtype=torch.uint8, device=cuda)
    y = torch.full((B, L, H, P), float("nan"), dtype=torch.bfloat16, device=cuda)
    runtime.ssd_chunk_scan(x.to(cuda), dt.to(cuda), A.to(cuda), Bm.to(cuda), Cm.to(cuda), ws, y, B=B, L=L, H=H, P=P,
                           N=N, G=G, chunk=chunk, dtype="bf16")
    finish()
    runtime.check_workspace_status(ws)
    ref = ssd.ssd_reference(x, dt, A, Bm, Cm)
    assert_storage_close(y, ref, BF16_ATOL, 2 * BF16_ULP, scale_by_rms=True)
    assert_rms_close(y, ref, 2.0 ** -8)


@pytest.mark.parametrize("segments,H,G", [(2, 4, 1), (3, 4, 2), (8, 4, 1), (4, 3, 1), (2, 6, 2)])
def test_ssd_sequences_cut_into_segments(cuda, native_lib, monkeypatch, segments, H, G):
    """A sequence cut into segments that run as separate CTAs: the state entering each later segment comes from
    the segment-state kernel and the recurrence over its results.  NB200_SSD_SEGMENTS forces the cut that the library would only choose
    for a problem with few (batch, head) pairs.  Head counts 3 and 6 with 2 groups run one head per CTA (no pair
    shares B and C); 8 segments of a 1024-row sequence are one step each."""
    from neptune_mlir import runtime

    B, L, P, N, chunk = 2, 1024, 64, 128, 128
    args = inputs.ssd_inputs(B=B, L=L, H=H, P=P, N=N, G=G, config=52)
    dev_args = [a.to(cuda) for a in args]
    ws = torch.empty(runtime.ssd_workspace_bytes(B, L, H, P, N, G, chunk), dtype=torch.uint8, device=cuda)
    outs = {}
    for k in (1, segments):
        monkeypatch.setenv("NB200_SSD_SEGMENTS", str(k))
        assert runtime.ssd_launches(B, L, H, P, N, G, chunk) == (1 if k == 1 else 2)
        y = torch.full((B, L, H, P), float("nan"), dtype=torch.bfloat16, device=cuda)
        runtime.ssd_chunk_scan(*dev_args, ws, y, B=B, L=L, H=H, P=P, N=N, G=G, chunk=chunk, dtype="bf16")
        finish()
        runtime.check_workspace_status(ws)
        outs[k] = y
    ref = ssd.ssd_reference(*args)
    for k, y in outs.items():
        assert_storage_close(y, ref, BF16_ATOL, 2 * BF16_ULP, scale_by_rms=True)
        assert_rms_close(y, ref, 2.0 ** -8)
    # the first segment is computed exactly as in the uncut run
    rows = (L // 128 + segments - 1) // segments * 128
    assert torch.equal(outs[1][:, :rows], outs[segments][:, :rows])


def test_ssd_config5_full_size_sampled(cuda, native_lib):
    """B=4, L=8192, H=64, P=64, N=128, chunk 256; heads are independent, a sample is checked in full."""
    from neptune_mlir import runtime

    B, L, H, P, N, G, chunk = 4, 8192, 64, 64, 128, 1, 256
    x, dt, A, Bm, Cm = (a.to(cuda) for a in inputs.ssd_inputs(B=B, L=L, H=H, P=P, N=N, G=G))
    mod = translate_data("ssd_chunk_scan_bf16_4x8192x64x64")
    ws = torch.empty(runtime.ssd_workspace_bytes(B, L, H, P, N, G, chunk), dtype=torch.uint8, device=cuda)
    y = torch.full((B, L, H, P), float("nan"), dtype=torch.bfloat16, device=cuda)
    mod.ssd_chunk_scan_bf16(x, dt, A, Bm, Cm, ws, y)
    finish()
    runtime.check_workspace_status(ws)
    assert bool(torch.isfinite(y).all())
    heads = [0, 63]
    ref = ssd.ssd_reference(x[:1, :, heads].cpu(), dt[:1, :, heads].cpu(), A[heads].cpu(), Bm[:1].cpu(), Cm[:1].cpu())
    assert_storage_close(y[:1, :, heads], ref, BF16_ATOL, 2 * BF16_ULP, scale_by_rms=True)
    assert_rms_close(y[:1, :, heads], ref, 2.0 ** -8)
