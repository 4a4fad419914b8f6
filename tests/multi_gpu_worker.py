"""Worker of tests/test_gpu_multi.py: one rank of a single-sequence decode sharded along the KV length.

Launched by ``python -m torch.distributed.run``; every rank draws the same seeded sequence on the CPU,
takes its slice, runs split-K + local combine through the C ABI, merges across ranks through ``nb200_decode_merge_nccl``, through ``torch.distributed`` + ``nb200_decode_combine`` and
through the peer-memory kernel ``nb200_decode_merge_peer``, and compares them with the CPU oracle on the whole sequence.  Prints ``OK rank <r>`` on success.
"""

import math
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "mlir-toy_b200"))

from neptune_mlir import native, runtime  # noqa: E402
from neptune_mlir.nccl_comm import Communicator  # noqa: E402
from neptune_mlir.sharding import gather_partials, gathered_strides, shard_range  # noqa: E402
from oracle import decode as oracle_decode  # noqa: E402


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    Hq, Hkv, L, D, splits = 32, 8, 8192, 128, 8
    gen = torch.Generator(device="cpu").manual_seed(4242)
    q = torch.randn((1, Hq, D), generator=gen).to(torch.bfloat16)
    k = torch.randn((1, Hkv, L, D), generator=gen).to(torch.bfloat16)
    v = torch.randn((1, Hkv, L, D), generator=gen).to(torch.bfloat16)
    lo, hi = shard_range(L, rank, world)
    Ll = hi - lo
    qd, kd, vd = q.to(dev), k[:, :, lo:hi].contiguous().to(dev), v[:, :, lo:hi].contiguous().to(dev)
    part = torch.empty((1, Hq, splits, D + 2), device=dev)
    local = torch.empty((Hq, D + 2), device=dev)
    scale_log2 = math.log2(math.e) / math.sqrt(D)
    lib = native.lib()
    st = torch.cuda.current_stream(dev).cuda_stream
    native.check(lib.nb200_decode_splitk(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), part.data_ptr(), 1, Hq, Hkv, Ll,
                                         D, splits, 1, scale_log2, None, st), "decode_splitk")
    runtime.decode_combine(part, local, rows=Hq, D=D, n_splits=splits, row_stride=splits * (D + 2),
                           split_stride=D + 2, out_dtype="f32")

    comm = Communicator.from_process_group()
    gathered = torch.empty((world, Hq, D + 2), device=dev)
    out_c = torch.empty((Hq, D), device=dev, dtype=torch.bfloat16)
    for _ in range(2):  # twice: the scratch is reused
        runtime.decode_merge_nccl(local, gathered, out_c, rows=Hq, D=D, world=world, out_dtype="bf16", comm=comm)
    g = gather_partials(local)
    rs, ss = gathered_strides(Hq, D + 2)
    out_t = torch.empty_like(out_c)
    runtime.decode_combine(g, out_t, rows=Hq, D=D, n_splits=world, row_stride=rs, split_stride=ss, out_dtype="bf16")
    torch.cuda.synchronize(dev)

    # a communicator of the wrong size is refused before anything is enqueued
    try:
        runtime.decode_merge_nccl(local, torch.empty((world + 1, Hq, D + 2), device=dev), out_c, rows=Hq, D=D,
                                  world=world + 1, out_dtype="bf16", comm=comm)
        raise SystemExit("a world size that disagrees with the communicator was accepted")
    except ValueError:
        pass

    ref = oracle_decode.decode_reference(q, k, v)[0]
    err_c = (out_c.float().cpu() - ref).abs().max().item()
    assert torch.equal(out_c, out_t), "C-ABI merge and torch.distributed merge disagree"
    assert torch.equal(gathered, g), "gathered partials differ between the two routes"
    assert err_c <= 2e-2, f"max-abs-err {err_c} > 2e-2"

    # the same merge as one kernel over peer-mapped memory (CUDA IPC), three calls in a row on the same buffers
    from neptune_mlir.peer import PeerWorkspace
    ws = PeerWorkspace(Hq, D)
    for _ in range(3):
        out_p = torch.full((Hq, D), float("nan"), device=dev, dtype=torch.bfloat16)
        ws.merge(local, out_p, "bf16")
        torch.cuda.synchronize(dev)
        runtime.check_status(dev)
        assert torch.equal(out_p, out_c), "peer-memory merge and NCCL merge disagree"
    # and the rank's whole share as ONE launch: split-K, local combine, push, wait, merge
    S1 = 9
    wbytes = lib.nb200_decode_sharded_workspace_bytes(Hq, Hkv, D, S1)
    wsp = torch.zeros(wbytes, dtype=torch.uint8, device=dev)
    for _ in range(3):
        out_s = torch.full((Hq, D), float("nan"), device=dev, dtype=torch.bfloat16)
        ws.sharded_decode(qd, kd, vd, wsp, out_s, Hq=Hq, Hkv=Hkv, L=Ll, D=D, n_splits=S1, dtype="bf16", scale_log2=scale_log2,
                          out_dtype="bf16")
        torch.cuda.synchronize(dev)
        runtime.check_status(dev)
        err_s = (out_s.float().cpu() - ref).abs().max().item()
        assert err_s <= 2e-2, f"one-launch sharded decode: max-abs-err {err_s}"
    dist.barrier()
    ws.close()
    torch.cuda.synchronize(dev)
    comm.destroy()
    dist.barrier()
    dist.destroy_process_group()
    print(f"OK rank {rank} err {err_c:.3e}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
