"""The allocation-free decode entry point against the workspace entry points, through the C ABI.

Collected last on purpose (file name), so that a run that stops at the first failure has already
gone through every other test.  The entry point exists for hosts that cannot allocate device memory
once they are serving (see include/nb200.h): the partials go to a scratch array built into the
library, which every call on the device shares and which still holds the previous call's data --
hence two calls in a row, of different sizes, each compared with the ordinary path.
"""

import math

import pytest
import torch

from oracle import decode, inputs

pytestmark = pytest.mark.gpu

BF16_ATOL = 2e-2
STATIC_SCRATCH_BYTES = 4 << 20


def _run_both(lib, cuda, B, Hq, Hkv, L, D, S, seed):
    from neptune_mlir import native

    q, k, v = (t.to(cuda) for t in inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D, base_seed=seed))
    scale_log2 = math.log2(math.e) / math.sqrt(D)
    st = torch.cuda.current_stream(cuda).cuda_stream
    # ordinary path: caller-provided workspace
    partials = torch.empty((B, Hq, S, D + 2), device=cuda)
    want = torch.full((B, Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    native.check(lib.nb200_decode_splitk(q.data_ptr(), k.data_ptr(), v.data_ptr(), partials.data_ptr(), B, Hq, Hkv,
                                         L, D, S, 1, scale_log2, None, st), "splitk")
    native.check(lib.nb200_decode_combine(partials.data_ptr(), want.data_ptr(), B * Hq, D, S, S * (D + 2), D + 2, 1, st),
                 "combine")
    # allocation-free path: inputs and output only
    got = torch.full((B, Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    native.check(lib.nb200_decode_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), got.data_ptr(), B, Hq, Hkv,
                                             L, D, S, 1, scale_log2, st), "decode_fwd_static")
    torch.cuda.synchronize()
    return got, want, decode.decode_reference(q.cpu(), k.cpu(), v.cpu())


def test_static_scratch_decode_matches_workspace_decode_twice(cuda, native_lib):
    from neptune_mlir import native

    lib = native.load(str(native_lib))
    # first call: larger problem; second call: smaller one, which finds the first call's partials still in the array
    for (B, Hq, Hkv, L, S), seed in (((4, 16, 4, 2048, 8), 0), ((2, 8, 2, 1024, 4), 7)):
        got, want, oracle_out = _run_both(lib, cuda, B, Hq, Hkv, L, 128, S, seed)
        assert bool(torch.isfinite(got).all())
        err = (got.float() - want.float()).abs().max().item()
        assert err <= BF16_ATOL, f"max abs err {err}"
        assert torch.equal(got, want)  # same kernels, same order of operations
        assert (got.float().cpu() - oracle_out).abs().max().item() <= BF16_ATOL   # and both agree with the CPU oracle


def test_static_scratch_decode_rejects_oversized_problems(cuda, native_lib):
    from neptune_mlir import native

    lib = native.load(str(native_lib))
    t = torch.zeros(16, device=cuda)
    B, Hq, S, D = 64, 32, 16, 128
    assert B * Hq * S * (D + 2) * 4 > STATIC_SCRATCH_BYTES
    rc = lib.nb200_decode_fwd_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), B, Hq, 8, 32768, D, S, 1,
                                     0.1, None)
    assert rc == -2
    msg = lib.nb200_last_error().decode()
    assert str(B * Hq * S * (D + 2) * 4) in msg and str(STATIC_SCRATCH_BYTES) in msg
