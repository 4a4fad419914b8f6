"""Host-side multi-GPU logic on CPU: unit partitioning and the gloo all-gather of decode partials."""

import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def test_shard_range_covers_everything_once():
    from neptune_mlir.sharding import shard_range

    for n in (1, 7, 8, 256, 1000):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, ret):
    for p in (str(ROOT), str(ROOT / "mlir-toy_b200")):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from neptune_mlir.sharding import gather_partials, gathered_strides, shard_range
        from oracle import decode, inputs

        q, k, v = inputs.decode_inputs(B=1, Hq=8, Hkv=2, L=1024, D=128, dtype=torch.float32)
        lo, hi = shard_range(1024, rank, world)
        # each rank reduces its slice of the sequence to one partial per head: [rows, D+2] = (o, m, l)
        m, l, o = decode.decode_partials(q, k[:, :, lo:hi], v[:, :, lo:hi], n_splits=1)
        local = torch.cat([o[0, :, 0], m[0, :, :1], l[0, :, :1]], dim=-1).contiguous()
        gathered = gather_partials(local)
        assert gathered.shape == (world, 8, 130)
        row_stride, split_stride = gathered_strides(8, 130)
        flat = gathered.reshape(-1)
        # address the gather exactly as nb200_decode_combine does: row*row_stride + split*split_stride
        idx = (torch.arange(8)[:, None] * row_stride + torch.arange(world)[None, :] * split_stride)
        o_g = torch.stack([flat[idx + d] for d in range(128)], dim=-1)
        merged = decode.combine_partials(flat[idx + 128][None], flat[idx + 129][None], o_g[None])
        want = decode.decode_reference(q, k, v)
        torch.testing.assert_close(merged, want, rtol=1e-5, atol=1e-5)
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def test_single_sequence_decode_merge_over_gloo_ranks():
    world = 2
    port = _free_port()
    manager = mp.Manager()
    ret = manager.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world))
