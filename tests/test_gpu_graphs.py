"""The operators as torch.library ops, and a decode step replayed from a CUDA graph."""

import math

import pytest
import torch

from gpu_util import assert_storage_close, finish
from oracle import attention, decode, inputs

pytestmark = pytest.mark.gpu


def test_custom_ops_match_the_oracle(cuda, native_lib):
    from neptune_mlir import torch_ops  # noqa: F401  (registers the ops)

    q, k, v = inputs.attention_inputs(1, 2, 256, 128, torch.bfloat16, config=21)
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=cuda)
    torch.ops.nb200.attn_fwd(q.to(cuda), k.to(cuda), v.to(cuda), out, 1.0 / math.sqrt(128), True)
    finish()
    assert_storage_close(out, attention.attention_reference(q, k, v, causal=True), 2e-2)


def test_decode_step_replays_from_a_cuda_graph(cuda, native_lib):
    """Split-K + combine are two plain kernel launches on the current stream: capture once, replay on new inputs."""
    from neptune_mlir import torch_ops  # noqa: F401

    B, Hq, Hkv, L, D, S = 2, 8, 2, 2048, 128, 8
    scale = 1.0 / math.sqrt(D)
    qd = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=cuda)
    kd = torch.empty((B, Hkv, L, D), dtype=torch.bfloat16, device=cuda)
    vd = torch.empty_like(kd)
    partials = torch.empty((B, Hq, S, D + 2), device=cuda)
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=cuda)

    def load(cfg):
        q, k, v = inputs.decode_inputs(B=B, Hq=Hq, Hkv=Hkv, L=L, D=D, config=cfg)
        qd.copy_(q)
        kd.copy_(k)
        vd.copy_(v)
        return q, k, v

    load(31)
    side = torch.cuda.Stream(device=cuda)
    side.wait_stream(torch.cuda.current_stream(cuda))
    with torch.cuda.stream(side):  # warm-up outside the capture, as torch asks
        torch.ops.nb200.decode_splitk(qd, kd, vd, partials, out, scale)
    torch.cuda.current_stream(cuda).wait_stream(side)
    finish()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        torch.ops.nb200.decode_splitk(qd, kd, vd, partials, out, scale)
    for cfg in (32, 33):
        q, k, v = load(cfg)
        out.fill_(float("nan"))
        graph.replay()
        finish()
        assert_storage_close(out, decode.decode_reference(q, k, v), 2e-2)


def test_attention_replays_from_a_cuda_graph(cuda, native_lib):
    """The attention launch is a 4-byte memset of its tile counter plus one kernel, both on the current stream:
    it can be captured once and replayed on new inputs (more tiles than SMs, so the dynamic deal is exercised)."""
    from neptune_mlir import torch_ops  # noqa: F401

    B, H, S, D = 1, 6, 4096, 128
    scale = 1.0 / math.sqrt(D)
    qd = torch.empty((B, H, S, D), dtype=torch.bfloat16, device=cuda)
    kd, vd, out = torch.empty_like(qd), torch.empty_like(qd), torch.empty_like(qd)

    def load(cfg):
        q, k, v = inputs.attention_inputs(B, H, S, D, torch.bfloat16, config=cfg)
        qd.copy_(q)
        kd.copy_(k)
        vd.copy_(v)
        return q, k, v

    load(41)
    side = torch.cuda.Stream(device=cuda)
    side.wait_stream(torch.cuda.current_stream(cuda))
    with torch.cuda.stream(side):
        torch.ops.nb200.attn_fwd(qd, kd, vd, out, scale, True)
    torch.cuda.current_stream(cuda).wait_stream(side)
    finish()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        torch.ops.nb200.attn_fwd(qd, kd, vd, out, scale, True)
    for cfg in (42, 43):
        q, k, v = load(cfg)
        out.fill_(float("nan"))
        graph.replay()
        finish()
        ref = attention.attention_reference(q[:, :2], k[:, :2], v[:, :2], causal=True)
        assert_storage_close(out[:, :2], ref, 2e-2)
        assert torch.isfinite(out.float()).all()
