"""The status words: how an expired device-side wait (or refused device-side data) reaches the host.

Nothing here makes a kernel wait: the status buffer is written from the host, which is exactly what a kernel
whose wait ran out leaves behind, and the tests check what the next launches and nb200_status_read do with it.
"""

import ctypes

import pytest
import torch

from oracle import attention, inputs

pytestmark = pytest.mark.gpu


def test_attention_skips_and_status_read_reports_after_a_recorded_timeout(cuda, native_lib):
    from neptune_mlir import native, runtime

    lib = native.load(str(native_lib))
    q, k, v = (t.to(cuda) for t in inputs.attention_inputs(1, 2, 256, 128, torch.bfloat16, config=2))
    status = torch.tensor([3, 17, 5, 96], dtype=torch.int32, device=cuda)   # "code 3 in block 17, detail 5, thread 96"
    out = torch.full_like(q, 7.0)
    st = torch.cuda.current_stream(cuda).cuda_stream
    rc = lib.nb200_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 1, 2, 256, 256, 128, 1,
                            attention.scale_log2(128), 1, status.data_ptr(), st)
    assert rc == 0                                       # the launch itself is fine
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                      # every CTA saw the non-zero word and left the output alone
    host = (ctypes.c_int * 4)()
    rc = lib.nb200_status_read(status.data_ptr(), host, st)
    assert rc == -4 and list(host) == [3, 17, 5, 96]
    msg = lib.nb200_last_error().decode()
    assert "code 3" in msg and "block 17" in msg
    with pytest.raises(native.NativeLibraryError, match="device wait timeout"):
        native.check(rc, "status")
    # cleared, the same call computes
    status.zero_()
    rc = lib.nb200_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 1, 2, 256, 256, 128, 1,
                            attention.scale_log2(128), 1, status.data_ptr(), st)
    assert rc == 0 and lib.nb200_status_read(status.data_ptr(), None, st) == 0
    ref = attention.attention_reference(q.cpu(), k.cpu(), v.cpu(), causal=True)
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2


def test_runtime_check_status_raises_once_and_clears(cuda, native_lib):
    from neptune_mlir import native, runtime

    runtime.check_status(cuda)
    runtime.status_buffer(cuda).copy_(torch.tensor([2, 1, 0, 0], dtype=torch.int32))
    with pytest.raises(native.NativeLibraryError, match="device-side wait expired"):
        runtime.check_status(cuda)
    runtime.check_status(cuda)


def test_ssd_clears_its_status_words_on_entry_and_reports_through_the_workspace(cuda, native_lib):
    """The SSD call zeroes the status words in its workspace before launching, so a stale record cannot make a
    later call skip; a record found after the call is reported by check_workspace_status."""
    from neptune_mlir import native, runtime
    from oracle import ssd

    B, L, H, P, N, G, chunk = 1, 256, 4, 64, 128, 1, 128
    args = inputs.ssd_inputs(B=B, L=L, H=H, P=P, N=N, G=G)
    x, dt, A, Bm, Cm = (a.to(cuda) for a in args)
    ws = torch.zeros(max(16, runtime.ssd_workspace_bytes(B, L, H, P, N, G, chunk)), dtype=torch.uint8, device=cuda)
    ws.view(torch.int32)[:4] = torch.tensor([12, 3, 9, 160], dtype=torch.int32, device=cuda)   # a stale record
    y = torch.full((B, L, H, P), float("nan"), dtype=torch.bfloat16, device=cuda)
    runtime.ssd_chunk_scan(x, dt, A, Bm, Cm, ws, y, B=B, L=L, H=H, P=P, N=N, G=G, chunk=chunk, dtype="bf16")
    torch.cuda.synchronize()
    runtime.check_workspace_status(ws)
    ref = ssd.ssd_reference(*args)
    assert bool(torch.isfinite(y).all())
    assert (y.float().cpu() - ref).pow(2).mean().sqrt().item() <= 2.0 ** -8 * ref.pow(2).mean().sqrt().item()
    ws.view(torch.int32)[:4] = torch.tensor([13, 0, 42, 7], dtype=torch.int32, device=cuda)
    with pytest.raises(native.NativeLibraryError, match="code 13"):
        runtime.check_workspace_status(ws)
