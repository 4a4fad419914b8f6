"""The peer-memory merge of the sharded decode (nb200_decode_merge_peer) on one GPU.

The kernel of one rank waits only for flags that OTHER ranks' kernels write.  With one GPU the other rank is
played by the host: its partial and its arrival flag are written into the buffer before the launch, so nothing
ever waits for a later launch; both "ranks'" buffers live in this GPU's memory.  The real thing, two processes
on two GPUs mapped through CUDA IPC, is covered by tests/test_gpu_multi.py.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

D, ROWS, MAXW = 128, 32, 16


def _layout(world):
    area = world * ROWS * (D + 2)
    flags = (2 * area + 31) // 32 * 32
    return area, flags


def _torch_combine(parts):
    """parts [world, rows, D+2] (o, m in the exp2 domain, l) -> [rows, D]"""
    M = parts[..., D].amax(dim=0)
    w = torch.exp2(parts[..., D] - M[None])
    return (w[..., None] * parts[..., :D]).sum(0) / (w * parts[..., D + 1]).sum(0)[..., None]


def _partials(world, cuda, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    p = torch.randn((world, ROWS, D + 2), generator=g)
    p[..., D + 1] = p[..., D + 1].abs() + 0.5          # l > 0
    return p.to(cuda)


def _merge(lib, local, bufs, out, world, rank, gen, wait_ns, status):
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    st = torch.cuda.current_stream().cuda_stream
    return lib.nb200_decode_merge_peer(local.data_ptr(), arr, out.data_ptr(), ROWS, D, world, rank, gen, 1, wait_ns,
                                       status.data_ptr(), st)


def test_two_ranks_played_on_one_gpu_over_two_generations(cuda, native_lib):
    from neptune_mlir import native

    lib = native.load(str(native_lib))
    world = 2
    size = lib.nb200_decode_merge_peer_workspace_bytes(ROWS, D, world)
    area, flags = _layout(world)
    assert size == (flags + 2 * MAXW) * 4
    bufs = [torch.zeros(size // 4, device=cuda) for _ in range(world)]
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    for gen in (1, 2, 3):
        parts = _partials(world, cuda, gen)
        want = _torch_combine(parts)
        s = gen & 1
        # the host plays rank 1 towards rank 0: its partial and its flag are in rank 0's buffer before the launch
        bufs[0][s * area + ROWS * (D + 2):s * area + 2 * ROWS * (D + 2)] = parts[1].reshape(-1)
        bufs[0].view(torch.int32)[flags + s * MAXW + 1] = gen
        outs = []
        for rank in (0, 1):   # rank 1's launch finds rank 0's partial and flag already delivered by rank 0's kernel
            out = torch.full((ROWS, D), float("nan"), dtype=torch.bfloat16, device=cuda)
            native.check(_merge(lib, parts[rank].contiguous(), bufs, out, world, rank, gen, 200_000_000, status), "merge_peer")
            outs.append(out)
        torch.cuda.synchronize()
        assert lib.nb200_status_read(status.data_ptr(), None, None) == 0
        for out in outs:
            assert (out.float() - want).abs().max().item() <= 2e-2
        assert torch.equal(outs[0], outs[1])


def test_a_rank_that_never_arrives_is_reported_not_waited_for(cuda, native_lib):
    """The wait is bounded: with nobody playing rank 1 the kernel gives up after wait_ns, leaves the output alone
    and records who was missing."""
    from neptune_mlir import native

    lib = native.load(str(native_lib))
    world = 2
    size = lib.nb200_decode_merge_peer_workspace_bytes(ROWS, D, world)
    bufs = [torch.zeros(size // 4, device=cuda) for _ in range(world)]
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    parts = _partials(world, cuda, 9)
    out = torch.full((ROWS, D), 5.0, dtype=torch.bfloat16, device=cuda)
    native.check(_merge(lib, parts[0].contiguous(), bufs, out, world, 0, 1, 20_000_000, status), "merge_peer")   # 20 ms
    torch.cuda.synchronize()
    host = (ctypes.c_int * 4)()
    assert lib.nb200_status_read(status.data_ptr(), host, None) == -4
    assert host[0] == 31 and host[2] == 1 and host[3] == 1          # code, missing rank, generation
    assert bool((out == 5.0).all())
    # the context is fine: the same call with rank 1 present completes
    status.zero_()
    area, flags = _layout(world)
    bufs[0][area + ROWS * (D + 2):area + 2 * ROWS * (D + 2)] = parts[1].reshape(-1)
    bufs[0].view(torch.int32)[flags + MAXW + 1] = 1
    native.check(_merge(lib, parts[0].contiguous(), bufs, out, world, 0, 1, 200_000_000, status), "merge_peer")
    torch.cuda.synchronize()
    assert lib.nb200_status_read(status.data_ptr(), None, None) == 0
    assert (out.float() - _torch_combine(parts)).abs().max().item() <= 2e-2


# ------------------------------------------------------------------ the one-launch sharded decode
def _sharded(lib, q, k, v, ws, bufs, out, Hq, Hkv, L, S, world, rank, gen, wait_ns, status, dtype_code=1):
    import math
    arr = (ctypes.c_void_p * max(world, 1))(*[b.data_ptr() for b in bufs]) if bufs else None
    st = torch.cuda.current_stream().cuda_stream
    return lib.nb200_decode_sharded_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), ws.data_ptr(), arr, out.data_ptr(), Hq, Hkv, L,
                                        D, S, dtype_code, math.log2(math.e) / math.sqrt(D), world, rank, gen, dtype_code,
                                        wait_ns, status.data_ptr(), st)


@pytest.mark.parametrize("Hq,Hkv,L,S", [(32, 8, 4096, 9), (8, 8, 1000, 3), (16, 2, 2048, 5), (8, 1, 777, 2), (4, 2, 300, 7)])
def test_one_launch_decode_of_a_whole_sequence(cuda, native_lib, Hq, Hkv, L, S):
    """world == 1: split-K, the combine of the splits and the normalisation in one launch, through the tickets;
    twice in a row on the same workspace (the counters reset themselves)."""
    from neptune_mlir import native
    from oracle import decode, inputs

    lib = native.load(str(native_lib))
    q, k, v = inputs.decode_inputs(B=1, Hq=Hq, Hkv=Hkv, L=L, D=D, config=61)
    ws = torch.zeros(lib.nb200_decode_sharded_workspace_bytes(Hq, Hkv, D, S), dtype=torch.uint8, device=cuda)
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    qd, kd, vd = q.to(cuda), k.to(cuda), v.to(cuda)
    ref = decode.decode_reference(q, k, v)[0]
    for _ in range(2):
        out = torch.full((Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
        native.check(_sharded(lib, qd, kd, vd, ws, None, out, Hq, Hkv, L, S, 1, 0, 0, 0, status), "sharded")
        torch.cuda.synchronize()
        assert lib.nb200_status_read(status.data_ptr(), None, None) == 0
        assert (out.float().cpu() - ref).abs().max().item() <= 2e-2
    assert int(ws[:4 * (2 * Hkv + 1)].view(torch.int32).abs().sum()) == 0  # tickets and chunk counters are back at zero


def test_one_launch_sharded_decode_with_the_other_rank_played_by_the_host(cuda, native_lib):
    """Two ranks, each owning half of the sequence; rank 1's partial and flag are put into rank 0's buffer by the
    host (computed with the ordinary split-K + combine entry points), then rank 0's single launch must produce the
    output of the whole sequence."""
    from neptune_mlir import native, runtime
    from oracle import decode, inputs
    import math

    lib = native.load(str(native_lib))
    Hq, Hkv, L, S, world = 32, 8, 4096, 5, 2
    q, k, v = inputs.decode_inputs(B=1, Hq=Hq, Hkv=Hkv, L=L, D=D, config=62)
    qd = q.to(cuda)
    halves = [(k[:, :, :L // 2].contiguous().to(cuda), v[:, :, :L // 2].contiguous().to(cuda)),
              (k[:, :, L // 2:].contiguous().to(cuda), v[:, :, L // 2:].contiguous().to(cuda))]
    # rank 1's partial through the ordinary entry points
    part = torch.empty((1, Hq, S, D + 2), device=cuda)
    tmp = torch.empty((1, Hq, D), dtype=torch.bfloat16, device=cuda)
    runtime.decode_splitk(qd, halves[1][0], halves[1][1], part, tmp, B=1, Hq=Hq, Hkv=Hkv, L=L // 2, D=D, n_splits=S,
                          dtype="bf16", scale_log2=math.log2(math.e) / math.sqrt(D))
    other = torch.empty((Hq, D + 2), device=cuda)
    runtime.decode_combine(part, other, rows=Hq, D=D, n_splits=S, row_stride=S * (D + 2), split_stride=D + 2, out_dtype="f32")
    size = lib.nb200_decode_merge_peer_workspace_bytes(Hq, D, world)
    bufs = [torch.zeros(size // 4, device=cuda) for _ in range(world)]
    area = world * Hq * (D + 2)
    flags = (2 * area + 31) // 32 * 32
    gen = 1
    bufs[0][area + Hq * (D + 2):area + 2 * Hq * (D + 2)] = other.reshape(-1)
    bufs[0].view(torch.int32)[flags + MAXW + 1] = gen
    ws = torch.zeros(lib.nb200_decode_sharded_workspace_bytes(Hq, Hkv, D, S), dtype=torch.uint8, device=cuda)
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    out = torch.full((Hq, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    native.check(_sharded(lib, qd, halves[0][0], halves[0][1], ws, bufs, out, Hq, Hkv, L // 2, S, world, 0, gen, 200_000_000, status), "sharded")
    torch.cuda.synchronize()
    assert lib.nb200_status_read(status.data_ptr(), None, None) == 0
    ref = decode.decode_reference(q, k, v)[0]
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2
    # rank 0's partial reached "rank 1"'s buffer too, with its flag
    assert int(bufs[1].view(torch.int32)[flags + MAXW + 0]) == gen
