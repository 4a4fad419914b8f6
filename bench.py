#!/usr/bin/env python3
"""Benchmark of the HTile hot path on B200: causal attention prefill (headline), plus split-K decode and both scans.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference] [--skip-extra]

N > 1 is launched by ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...``; the
work of the fixed configuration is partitioned over ranks by independent units ((batch, head) pairs,
sequences, channels, heads) with no data-path collective, so the scaling is *strong*.  Rank 0 prints one
JSON line.  A step is one pass of the workload: one launch of the fused attention kernel over this rank's
(batch, head) units, called through the function the translator emits for the HTile program.

Timing: CUDA events on the launching stream around every step, L2 flushed (a 512 MB fill) before each
timed step, a barrier plus device synchronise on both sides of the timed region, maximum over ranks.
``value`` has its inputs resident in HBM; ``e2e`` runs the same function from pinned host buffers with the
host-to-device and device-to-host copies inside the timed region.  ``--impl reference`` times the CPU
restatement of the reference's own check math (the oracle) on the host cores instead.

Every workload in ``workloads`` carries, beside its device-timed rate and roofline fraction:
``parity`` (the kernel against the CPU oracle on a stated sample of the configuration, same inputs),
``cpu_baseline`` (that oracle evaluation timed on the host cores; rank 0 of a 1-GPU run only) and ``e2e``
(the emitted function fed from pinned host memory, copies inside the timed region).  ``reference_shape``
runs the one program the reference itself has (non-causal f16 1x32x4096x128) through this build's kernel and
through the kernels the reference's own Triton / TileLang / cuTile translators emit for it.
"""

from __future__ import annotations

import argparse
import ast
import importlib.util
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT), str(ROOT / "mlir-toy_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

# ---- the benchmark configurations ------------------------------------------------------------------
ATTN1 = dict(B=1, H=4, S=256, D=64)                         # configs[0]: causal fp32, the reference's CPU-sized case
ATTN = dict(B=8, H=32, S=4096, D=128)                       # configs[1]: causal bf16 prefill
DECODE = dict(B=64, Hq=32, Hkv=8, L=32768, D=128, S=16)     # configs[2]
DECODE1 = dict(B=1, Hq=32, Hkv=8, L=262144, D=128)          # configs[2], single-sequence variant
DECODE1_WAVES = 1                                            # splits = waves * (resident CTA slots / kv heads)
                                                             # per GPU so that one sequence still fills the SMs
SCAN = dict(B=8, Dm=4096, L=4096, N=16)                     # configs[3]
SSD = dict(B=4, L=8192, H=64, P=64, N=128, G=1, chunk=256)  # configs[4]
REF_SHAPE = dict(B=1, H=32, S=4096, D=128)                  # the reference's own program: non-causal f16

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM bytes per launch of the attention kernel, per (batch, head) unit: a profiler capture of 64 units of the
# full-size workload read and wrote 248.4 MB (dram__bytes_read.sum + dram__bytes_write.sum); the traffic grows in
# proportion to the unit count because K/V of a head stay in L2 while its tiles run.  The compulsory traffic is
# 4 * S * D * 2 bytes per unit = 4.19 MB; the capture is 7.4 % below it (part of Q/K/V was still in L2 from the fill).
ATTN_DRAM_TRAFFIC_BYTES_PER_UNIT = 248_423_936 / 64

# Warp instructions per state update of the selective-scan kernel (8 states per thread), from a profiler count of
# smsp__inst_executed.sum over one launch of the full configuration: 382.9 M instructions for 8 * 4096 * 4096 * 16
# updates (45.6 per warp and time step).
SCAN_WARP_INSTR_PER_UPDATE = 382.857e6 / (8 * 4096 * 4096 * 16)

LOG2E = math.log2(math.e)
BF16_ATOL = 2e-2


def attn_flops(units: int, S: int, D: int) -> float:
    """4*D FLOP per unmasked (i, j) pair: 2*D*S*(S+1) per (batch, head) unit."""
    return 2.0 * units * D * S * (S + 1)


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def load_callable(text: str, fn_name: str):
    """HTile text -> emitted module -> the function named after the func.func."""
    from neptune_mlir.translators import b200

    with tempfile.NamedTemporaryFile("w", suffix=".mlir", delete=False) as f:
        f.write(text)
    ns: dict = {}
    exec(compile(ast.unparse(b200.translate_file(f.name)), f"<nb200 {fn_name}>", "exec"), ns)
    os.unlink(f.name)
    return ns[fn_name]


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None and not self.lines:
            time.sleep(0.3)  # a very short timed region: wait for the first sample (the kernels are still the last thing that ran)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


class Dist:
    def __init__(self, n_gpus: int):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != n_gpus:
            if self.world == 1 and n_gpus > 1:
                raise SystemExit(f"--gpus {n_gpus} needs a torchrun launch with {n_gpus} ranks")
            raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={self.world}")
        if self.world > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))

    def barrier(self):
        if self.world > 1:
            dist.barrier()

    def max(self, x: float) -> float:
        if self.world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())


def timed_steps(fn, steps: int, warmup: int, flush: torch.Tensor, d: Dist) -> float:
    """Mean milliseconds per step over `steps` timed calls (max over ranks), L2 flushed before each."""
    for _ in range(warmup):
        flush.fill_(1.0)
        fn()
    torch.cuda.synchronize()
    d.barrier()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush.fill_(float(i))
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    d.barrier()
    torch.cuda.synchronize()
    total = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
    return d.max(total) / steps


def e2e_steps(fn_device, host_in, dev_in, dev_out, host_out, flush, d: Dist, steps: int = 2) -> dict:
    """The emitted function fed from pinned host memory: H2D of every input, the call, D2H of the result, all
    inside the timed region (one stream, so the copies are not hidden; attention has its own overlapped variant)."""
    def step():
        for h, t in zip(host_in, dev_in):
            t.copy_(h, non_blocking=True)
        fn_device()
        host_out.copy_(dev_out, non_blocking=True)

    ms = timed_steps(step, steps, 1, flush, d)
    return {"ms_per_step": ms, "steps": steps,
            "h2d_bytes_per_step": sum(h.numel() * h.element_size() for h in host_in),
            "d2h_bytes_per_step": host_out.numel() * host_out.element_size()}


def pinned(t: torch.Tensor) -> torch.Tensor:
    return t.detach().cpu().pin_memory()


# ---- CPU arm ---------------------------------------------------------------------------------------
def cpu_attention_sample(heads: int) -> tuple[float, float]:
    """Times the oracle (the reference's check math + causal mask) on `heads` (batch, head) units of the
    attention configuration; returns (seconds, TFLOP/s counting the causal FLOPs)."""
    from oracle import attention, inputs

    S, D = ATTN["S"], ATTN["D"]
    q, k, v = inputs.attention_inputs(1, heads, S, D, torch.bfloat16, config=2)
    t0 = time.perf_counter()
    attention.attention_reference(q, k, v, causal=True)
    dt = time.perf_counter() - t0
    return dt, attn_flops(heads, S, D) / dt / 1e12


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    heads = 8  # per step: a bounded sample of the configuration (8 of its 256 (batch, head) units)
    for _ in range(args.warmup):
        cpu_attention_sample(heads)
    secs = [cpu_attention_sample(heads)[0] for _ in range(args.steps)]
    mean = sum(secs) / len(secs)
    value = attn_flops(heads, ATTN["S"], ATTN["D"]) / mean / 1e12
    sample = f"{heads} of {ATTN['B'] * ATTN['H']} (batch, head) units per step, full S={ATTN['S']}"
    print(json.dumps({
        "impl": "reference", "metric": "attn_prefill_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": attn_config(args.gpus) | {"sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def attn_config(n: int) -> dict:
    return {"workload": "causal attention prefill bf16 B=8 H=32 S=4096 D=128 (configs[1])",
            "global_batch": ATTN["B"], "heads": ATTN["H"], "seq_len": ATTN["S"], "head_dim": ATTN["D"],
            "partition": f"(batch, head) units over {n} rank(s), no collective",
            "l2": "flushed before every timed step (512 MB fill)",
            "flop_count": "2*B*H*D*S*(S+1) (unmasked pairs only)"}


def bracket_stats(out: torch.Tensor, ref: torch.Tensor, atol: float) -> dict:
    """max |out - ref|, rms error over rms(ref), and how many elements are neither within `atol` of the reference
    nor within one unit in the last place of the 16-bit output format at the reference's magnitude (i.e. one of
    the two representable values around it) -- for outputs whose magnitude is not bounded by the inputs."""
    o, r = out.detach().double().cpu(), ref.detach().double().cpu()
    err = (o - r).abs()
    res = {"max_abs_err": err.max().item(),
           "rms_rel": (err.pow(2).mean().sqrt() / r.pow(2).mean().sqrt().clamp_min(1e-30)).item(),
           "max_abs_ref": r.abs().max().item()}
    if out.dtype in (torch.bfloat16, torch.float16):
        mant = 7 if out.dtype == torch.bfloat16 else 10
        ulp = torch.exp2(torch.floor(torch.log2(r.abs().clamp_min(1e-30))) - mant)
        ok = (err <= atol) | (err <= ulp)
        res["outside_atol_and_1ulp"] = int((~ok).sum().item())
        res["elements"] = o.numel()
    return res


# ---- GPU arm ---------------------------------------------------------------------------------------
def bench_attention(args, d: Dist, dev, flush, pk, pk_kind) -> dict:
    from neptune_mlir import programs, runtime
    from neptune_mlir.sharding import shard_range

    S, D = ATTN["S"], ATTN["D"]
    total_units = args.attn_units or ATTN["B"] * ATTN["H"]
    lo, hi = shard_range(total_units, d.rank, d.world)
    units = hi - lo
    fn = load_callable(programs.attention_htile("attention_prefill", units, 1, S, D, "bf16", causal=True), "attention_prefill")
    gen = torch.Generator(device=dev).manual_seed(2000 + d.rank)
    q, k, v = (torch.randn((units, 1, S, D), device=dev, dtype=torch.bfloat16, generator=gen) for _ in range(3))
    out = torch.empty_like(q)

    with ClockSampler(dev.index) as clocks:
        ms = timed_steps(lambda: fn(q, k, v, out), args.steps, args.warmup, flush, d)
        if len(clocks.lines) < 3:
            # the timed region was shorter than the sampling period: keep the same kernel running (untimed)
            # until a few samples under load exist
            t_end = time.perf_counter() + 0.5
            while time.perf_counter() < t_end and len(clocks.lines) < 5:
                fn(q, k, v, out)
                torch.cuda.synchronize()
    runtime.check_status(dev)
    flops_total = attn_flops(total_units, S, D)
    value = flops_total / (ms * 1e-3) / 1e12
    # roofline of the dominant (only) kernel, per launch on this rank
    achieved = attn_flops(units, S, D) / (ms * 1e-3) / 1e12
    peak = pk["bf16_tflops"]
    result = {
        "ms": ms, "value": value, "clocks": clocks.summary(),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "traffic": ATTN_DRAM_TRAFFIC_BYTES_PER_UNIT * units, "peak_source": f"of {pk_kind} (burst cuBLAS bf16)",
                     "frac_of_sustained": achieved / pk.get("bf16_tflops_sustained", peak),
                     "kernel": "attn_fwd_tcgen05_kernel<bf16>"},
    }
    result["gpu_launches"] = args.steps

    # parity on a sample of this configuration: the same seeded units through the kernel and through the CPU oracle
    if d.rank == 0 and not args.skip_parity:
        from oracle import attention, inputs
        n_s = 4
        qs, ks, vs = inputs.attention_inputs(n_s, 1, S, D, torch.bfloat16, config=2)
        fn_s = load_callable(programs.attention_htile("attention_sample", n_s, 1, S, D, "bf16", causal=True), "attention_sample")
        os_ = torch.full((n_s, 1, S, D), float("nan"), dtype=torch.bfloat16, device=dev)
        fn_s(qs.to(dev), ks.to(dev), vs.to(dev), os_)
        torch.cuda.synchronize()
        ref = attention.attention_reference(qs, ks, vs, causal=True)
        result["parity"] = {"max_abs_err": (os_.float().cpu() - ref).abs().max().item(), "tolerance": BF16_ATOL,
                            "sample": f"{n_s} of {ATTN['B'] * ATTN['H']} (batch, head) units, full S, against the CPU oracle"}

    if args.skip_e2e:
        result["e2e"] = None
        return result

    # ---- end to end: pinned host buffers, copies inside the timed region, chunked so that copies overlap compute
    chunk_units = max(1, units // 8)
    while units % chunk_units:
        chunk_units -= 1
    n_chunks = units // chunk_units
    fn_chunk = load_callable(programs.attention_htile("attention_chunk", chunk_units, 1, S, D, "bf16", causal=True),
                             "attention_chunk")
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    hout = torch.empty((units, 1, S, D), dtype=torch.bfloat16).pin_memory()
    dq, dk, dv, dout = (torch.empty_like(q) for _ in range(4))
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def e2e_step():
        main = torch.cuda.current_stream(dev)
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for c in range(n_chunks):
            sl = slice(c * chunk_units, (c + 1) * chunk_units)
            with torch.cuda.stream(s_in):
                dq[sl].copy_(hq[sl], non_blocking=True)
                dk[sl].copy_(hk[sl], non_blocking=True)
                dv[sl].copy_(hv[sl], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            main.wait_event(ready)
            fn_chunk(dq[sl], dk[sl], dv[sl], dout[sl])
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                hout[sl].copy_(dout[sl], non_blocking=True)
        main.wait_stream(s_out)

    n_e2e = max(2, min(args.steps, 5))
    ms_e2e = timed_steps(e2e_step, n_e2e, 1, flush, d)
    runtime.check_status(dev)
    elem = 2
    result["e2e"] = {"value": flops_total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                     "h2d_bytes_per_step": 3 * units * S * D * elem, "d2h_bytes_per_step": units * S * D * elem,
                     "ms_per_step": ms_e2e, "steps": n_e2e,
                     "how": f"{n_chunks} chunks of {chunk_units} units through the emitted function; H2D, kernel and "
                            "D2H on three streams from/to pinned host memory"}
    del q, k, v, out, dq, dk, dv, dout
    torch.cuda.empty_cache()
    return result


def bench_extra(args, d: Dist, dev, flush, pk, pk_kind) -> dict:
    """Decode and both scans at their configurations (HBM-bound by the metric): GB/s of algorithmic bytes."""
    from neptune_mlir import native, programs, runtime
    from neptune_mlir.sharding import shard_range

    steps, warm = max(3, min(args.steps, 10)), 3
    hbm = pk["hbm_gbs"]
    want = set(args.extra.split(","))
    out: dict = {}
    gen = torch.Generator(device=dev).manual_seed(3000 + d.rank)
    bf = torch.bfloat16
    do_cpu = d.rank == 0 and d.world == 1 and not args.skip_cpu      # CPU baselines: rank 0 of a 1-GPU run only
    do_parity = d.rank == 0 and not args.skip_parity
    cores = os.cpu_count() or 1
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count

    def rnd(shape, dtype=bf):
        return torch.randn(shape, device=dev, dtype=dtype, generator=gen)

    def record(name, ms, total_bytes, extra=None):
        gbs = total_bytes / (ms * 1e-3) / 1e9
        out[name] = {"ms_per_step": ms, "value": gbs, "unit": "GB/s", "algorithmic_bytes": total_bytes,
                     "roofline": {"bound": "hbm", "achieved": gbs / d.world, "peak": hbm, "unit": "GB/s",
                                  "frac": gbs / d.world / hbm, "peak_source": f"of {pk_kind} (copy)"}} | (extra or {})
        return out[name]

    def cpu_entry(secs, sample_bytes, sample):
        return {"value": sample_bytes / secs / 1e9, "unit": "GB/s", "cores": cores, "kind": "port", "seconds": secs,
                "sample": sample}

    def add_e2e(entry, total_bytes, e):
        entry["e2e"] = {"value": total_bytes / (e["ms_per_step"] * 1e-3) / 1e9, "unit": "GB/s"} | e | {
            "how": "the emitted function fed from pinned host memory on one stream: H2D of all inputs, the call, D2H of the output"}

    # -- configs[0]: causal fp32 attention 1x4x256x64, a parity case (33.7 MFLOP), not a bench line
    def run_attn1():
        if not do_parity:
            return
        from oracle import attention, inputs
        c = ATTN1
        q, k, v = inputs.attention_inputs(c["B"], c["H"], c["S"], c["D"], torch.float32, config=1)
        fn = load_callable(programs.attention_htile("attention_config1", c["B"], c["H"], c["S"], c["D"], "f32", causal=True),
                           "attention_config1")
        o = torch.full((c["B"], c["H"], c["S"], c["D"]), float("nan"), device=dev)
        fn(q.to(dev), k.to(dev), v.to(dev), o)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ref = attention.attention_reference(q, k, v, causal=True)
        secs = time.perf_counter() - t0
        out["attention_config1"] = {
            "config": "causal fp32 B=1 H=4 S=256 D=64 (configs[0]); parity only",
            "parity": {"max_abs_err": (o.cpu() - ref).abs().max().item(), "tolerance": 1e-4,
                       "sample": "the whole configuration against the CPU oracle"},
            "cpu_seconds": secs}

    # -- split-K decode, batch sharded over ranks
    def run_decode():
        c = dict(DECODE, B=args.decode_batch) if args.decode_batch else dict(DECODE)
        lo, hi = shard_range(c["B"], d.rank, d.world)
        Bl = hi - lo
        cap = 64   # the program leaves the split count to the library, bounded by the partials memref
        fn = load_callable(programs.decode_splitk_decl("decode", Bl, c["Hq"], c["Hkv"], c["L"], c["D"], cap, auto_splits=True), "decode")
        q, k, v = rnd((Bl, c["Hq"], c["D"])), rnd((Bl, c["Hkv"], c["L"], c["D"])), rnd((Bl, c["Hkv"], c["L"], c["D"]))
        part = torch.empty((Bl, c["Hq"], cap, c["D"] + 2), device=dev)
        o = torch.empty_like(q)
        ms = timed_steps(lambda: fn(q, k, v, part, o), steps, warm, flush, d)
        runtime.check_status(dev)
        total = 2 * c["B"] * c["Hkv"] * c["L"] * c["D"] * 2 + 2 * c["B"] * c["Hq"] * c["D"] * 2
        n_auto = native.lib().nb200_decode_auto_splits(Bl, c["Hkv"], c["L"], cap)
        entry = record("decode_splitk", ms, total, {
            "config": f"B={c['B']} Hq=32 Hkv=8 L=32768 D=128 (configs[2]); the program leaves the split count to the library "
                      f"(at most {cap}), which chose {n_auto} per (sequence, kv head) on this rank to fill whole waves of CTAs",
            "launches_per_step": 2})
        if not args.skip_e2e:
            hq, hk, hv = pinned(q), pinned(k), pinned(v)
            ho = torch.empty(o.shape, dtype=o.dtype).pin_memory()
            add_e2e(entry, total, e2e_steps(lambda: fn(q, k, v, part, o), (hq, hk, hv), (q, k, v), o, ho, flush, d))
            del hq, hk, hv
        del q, k, v, part, o
        torch.cuda.empty_cache()
        if do_parity:
            from oracle import decode as odec, inputs
            ns = 8
            qs, ks, vs = inputs.decode_inputs(B=ns, Hq=c["Hq"], Hkv=c["Hkv"], L=c["L"], D=c["D"])
            fn_s = load_callable(programs.decode_splitk_decl("decode_sample", ns, c["Hq"], c["Hkv"], c["L"], c["D"], c["S"]), "decode_sample")
            ps = torch.empty((ns, c["Hq"], c["S"], c["D"] + 2), device=dev)
            os_ = torch.full((ns, c["Hq"], c["D"]), float("nan"), dtype=bf, device=dev)
            fn_s(qs.to(dev), ks.to(dev), vs.to(dev), ps, os_)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ref = odec.decode_reference(qs, ks, vs)
            secs = time.perf_counter() - t0
            sample = f"{ns} of {c['B']} sequences, full L, 16 splits, against the CPU oracle (direct softmax)"
            entry["parity"] = {"max_abs_err": (os_.float().cpu() - ref).abs().max().item(), "tolerance": BF16_ATOL, "sample": sample}
            if do_cpu:
                entry["cpu_baseline"] = cpu_entry(secs, total * ns / c["B"], sample)

    # -- single sequence, KV sharded along L over ranks, partials merged over NCCL
    def run_decode1():
        c = dict(DECODE1)
        # one CTA per (split, kv head); two CTAs are resident per SM: fill those slots a whole number of times
        slots = 2 * sm_count
        c["S"] = args.decode1_splits or max(1, slots // c["Hkv"]) * DECODE1_WAVES
        lo, hi = shard_range(c["L"], d.rank, d.world)
        Ll = hi - lo
        rows = c["Hq"]
        q = rnd((1, c["Hq"], c["D"]))
        if d.world > 1:
            dist.broadcast(q, src=0)
        k, v = rnd((1, c["Hkv"], Ll, c["D"])), rnd((1, c["Hkv"], Ll, c["D"]))
        part = torch.empty((1, c["Hq"], c["S"], c["D"] + 2), device=dev)
        local = torch.empty((rows, c["D"] + 2), device=dev)
        o = torch.empty((rows, c["D"]), device=dev, dtype=bf)
        scale_log2 = LOG2E / math.sqrt(c["D"])
        lib = native.lib()

        def stream_part():
            st = torch.cuda.current_stream(dev).cuda_stream
            native.check(lib.nb200_decode_splitk(q.data_ptr(), k.data_ptr(), v.data_ptr(), part.data_ptr(), 1, c["Hq"], c["Hkv"],
                                                 Ll, c["D"], c["S"], 1, scale_log2, runtime.status_buffer(dev).data_ptr(), st),
                         "decode_splitk")
            runtime.decode_combine(part, local, rows=rows, D=c["D"], n_splits=c["S"], row_stride=c["S"] * (c["D"] + 2),
                                   split_stride=c["D"] + 2, out_dtype="f32")

        comm = gathered = peer_ws = None
        peer_note = None
        if d.world > 1:
            from neptune_mlir.nccl_comm import Communicator
            comm = Communicator.from_process_group()
            gathered = torch.empty((d.world, rows, c["D"] + 2), device=dev)
            if args.merge != "nccl":
                try:   # the merge as one kernel over peer-mapped memory; every rank must succeed or none uses it
                    from neptune_mlir.peer import PeerWorkspace
                    peer_ws = PeerWorkspace(rows, c["D"])
                    ok_local = 1.0
                except Exception as exc:  # noqa: BLE001
                    peer_note, ok_local = f"{type(exc).__name__}: {str(exc)[:200]}", 0.0
                flag = torch.tensor([ok_local], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if flag.item() < 1.0:
                    peer_ws = None

        def merge_nccl():
            runtime.decode_merge_nccl(local, gathered, o, rows=rows, D=c["D"], world=d.world, out_dtype="bf16", comm=comm)

        def merge_part():
            if d.world > 1 and peer_ws is not None:
                peer_ws.merge(local, o, "bf16")
            elif d.world > 1:
                merge_nccl()
            else:
                runtime.decode_combine(local, o, rows=rows, D=c["D"], n_splits=1, row_stride=c["D"] + 2,
                                       split_stride=c["D"] + 2, out_dtype="bf16")

        # the whole of it as ONE launch per rank (split-K, local combine, push to the peers, wait, merge)
        fused_ws = torch.zeros(lib.nb200_decode_sharded_workspace_bytes(c["Hq"], c["Hkv"], c["D"], c["S"]), dtype=torch.uint8, device=dev)
        fused_gen = [0]

        def fused_part():
            if d.world > 1:
                peer_ws.sharded_decode(q, k, v, fused_ws, o, Hq=c["Hq"], Hkv=c["Hkv"], L=Ll, D=c["D"], n_splits=c["S"], dtype="bf16",
                                       scale_log2=scale_log2, out_dtype="bf16")
            else:
                st = torch.cuda.current_stream(dev).cuda_stream
                native.check(lib.nb200_decode_sharded_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), fused_ws.data_ptr(), None, o.data_ptr(),
                                                          c["Hq"], c["Hkv"], Ll, c["D"], c["S"], 1, scale_log2, 1, 0, 0, 1, 0,
                                                          runtime.status_buffer(dev).data_ptr(), st), "decode_sharded_fwd")

        use_fused = d.world == 1 or peer_ws is not None
        ms_stream = timed_steps(stream_part, steps, warm, flush, d)
        ms_merge_nccl = timed_steps(merge_nccl, steps, warm, flush, d) if (d.world > 1 and peer_ws is not None) else None
        ms_merge = timed_steps(merge_part, steps, warm, flush, d)
        ms_unfused = timed_steps(lambda: (stream_part(), merge_part()), steps, warm, flush, d)
        ms_both = timed_steps(fused_part, steps, warm, flush, d) if use_fused else ms_unfused
        runtime.check_status(dev)
        total = 2 * c["Hkv"] * c["L"] * c["D"] * 2 + 2 * c["Hq"] * c["D"] * 2
        entry = record("decode_single_sequence", ms_both, total,
                       {"config": f"B=1 L=262144 KV sharded along L over ranks, {c['S']} splits per rank (configs[2] variant)",
                        "launches_per_step": 1 if use_fused else 4,
                        "how": ("nb200_decode_sharded_fwd: one launch per rank (split-K, local combine, push, bounded wait, merge)" if use_fused
                                else "split-K + combine + NCCL all-gather + combine"),
                        "unfused_ms": ms_unfused, "stream_ms": ms_stream,
                        "merge_ms": ms_merge, "merge_bytes_per_rank": rows * (c["D"] + 2) * 4,
                        "collective": ("none" if d.world == 1 else
                                       "nb200_decode_merge_peer: one kernel, stores into peer-mapped buffers + flags (no NCCL on the data path)"
                                       if peer_ws is not None else "ncclAllGather inside nb200_decode_merge_nccl"),
                        "merge_ms_nccl_for_comparison": ms_merge_nccl, "peer_merge_unavailable": peer_note})
        # parity of the merged result at every rank count: each rank reduces its own KV slice with plain torch in
        # fp32 (scores, maximum, sums), the per-rank partials are gathered with torch.distributed and merged in
        # torch; the kernels' merged output must agree with that
        if not args.skip_parity:
            G = c["Hq"] // c["Hkv"]
            qf = q[0].float().view(c["Hkv"], G, c["D"])
            m = torch.full((c["Hkv"], G), float("-inf"), device=dev)
            l = torch.zeros((c["Hkv"], G), device=dev)
            acc = torch.zeros((c["Hkv"], G, c["D"]), device=dev)
            for t0_ in range(0, Ll, 16384):
                kc, vc = k[0, :, t0_:t0_ + 16384].float(), v[0, :, t0_:t0_ + 16384].float()
                x = torch.matmul(qf, kc.transpose(-1, -2)) / math.sqrt(c["D"])
                m_new = torch.maximum(m, x.amax(dim=-1))
                p = torch.exp(x - m_new[..., None])
                a = torch.exp(m - m_new)
                l = l * a + p.sum(dim=-1)
                acc = acc * a[..., None] + torch.matmul(p, vc)
                m = m_new
            packed = torch.cat([acc.view(rows, c["D"]), m.view(rows, 1), l.view(rows, 1)], dim=1).contiguous()
            if d.world > 1:
                allp = torch.empty((d.world * rows, c["D"] + 2), device=dev)
                dist.all_gather_into_tensor(allp, packed)
                allp = allp.view(d.world, rows, c["D"] + 2)
            else:
                allp = packed[None]
            M = allp[..., c["D"]].amax(dim=0)
            w = torch.exp(allp[..., c["D"]] - M[None])
            ref = (w[..., None] * allp[..., :c["D"]]).sum(0) / (w * allp[..., c["D"] + 1]).sum(0)[..., None]
            err = d.max((o.float() - ref).abs().max().item())
            entry["parity"] = {"max_abs_err": err, "tolerance": BF16_ATOL,
                               "sample": f"the whole sequence on {d.world} rank(s) after the merge, against an fp32 torch evaluation "
                                         "of each rank's slice merged through torch.distributed (max over ranks)"}
        if peer_ws is not None:
            torch.cuda.synchronize(dev)
            d.barrier()
            peer_ws.close()
        if comm is not None:
            torch.cuda.synchronize(dev)
            comm.destroy()
        del q, k, v, part, local, o, gathered
        torch.cuda.empty_cache()

    # -- Mamba-1 selective scan, (batch x channel) rows sharded as whole sequences when possible, else channels
    def run_scan():
        c = dict(SCAN, B=args.scan_batch) if args.scan_batch else dict(SCAN)
        if c["B"] % d.world == 0:
            Bl, Dl = c["B"] // d.world, c["Dm"]
        else:
            Bl, Dl = c["B"], c["Dm"] // d.world
        fn = load_callable(programs.selective_scan_decl("scan", Bl, Dl, c["L"], c["N"]), "scan")
        u, z = rnd((Bl, Dl, c["L"])), rnd((Bl, Dl, c["L"]))
        # delta = softplus(N(0,1) + dt_bias), dt_bias = inverse soft-plus of dt0 ~ logU(1e-3, 1e-1) per channel:
        # the same construction as the parity tests' inputs, drawn on the device
        dt0 = torch.exp(torch.rand((Dl,), device=dev, generator=gen) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
        dt_bias = dt0 + torch.log(-torch.expm1(-dt0))
        delta = torch.nn.functional.softplus(rnd((Bl, Dl, c["L"]), torch.float32) + dt_bias[None, :, None]).to(bf)
        A = -torch.exp(torch.rand((Dl, c["N"]), device=dev, generator=gen) * math.log(16.0))
        Bm, Cm = rnd((Bl, c["N"], c["L"])), rnd((Bl, c["N"], c["L"]))
        Dk = rnd((Dl,), torch.float32)
        o = torch.empty_like(u)
        with ClockSampler(dev.index) as clocks:
            ms = timed_steps(lambda: fn(u, delta, A, Bm, Cm, Dk, z, o), steps, warm, flush, d)
        total = 4 * c["B"] * c["Dm"] * c["L"] * 2 + 2 * c["B"] * c["N"] * c["L"] * 2 + c["Dm"] * c["N"] * 4 + c["Dm"] * 4
        updates = c["B"] * c["Dm"] * c["L"] * c["N"]
        clk = (clocks.summary()["sm_mhz"] or pk.get("sm_max_mhz", 1965.0)) * 1e6
        # two more floors of this kernel, per GPU: one ex2 per state update (plus one special-function result per
        # output element for the gate) at 16 results per clock per SM; and the issue slots, 4 per clock per SM
        mufu_s = (updates + c["B"] * c["Dm"] * c["L"]) / d.world / (16 * sm_count * clk)
        issue_s = updates * SCAN_WARP_INSTR_PER_UPDATE / d.world / (4 * sm_count * clk)
        entry = record("selective_scan", ms, total, {
            "config": "B=8 D=4096 L=4096 N=16 (configs[3])", "launches_per_step": 1,
            "state_updates_per_s": updates / (ms * 1e-3),
            "roofline_mufu": {"bound": "special-function unit (one ex2 per state update, 16 results/clk/SM)", "floor_ms": mufu_s * 1e3,
                              "frac": mufu_s * 1e3 / ms, "sm_mhz": clk / 1e6},
            "roofline_issue": {"bound": "issue slots (4 warp instructions/clk/SM)", "floor_ms": issue_s * 1e3, "frac": issue_s * 1e3 / ms,
                               "warp_instr_per_update": SCAN_WARP_INSTR_PER_UPDATE,
                               "source": "smsp__inst_executed.sum of one profiled launch of the 8-states-per-thread kernel"}})
        if not args.skip_e2e:
            hin = tuple(pinned(t) for t in (u, delta, Bm, Cm, z))
            ho = torch.empty(o.shape, dtype=o.dtype).pin_memory()
            add_e2e(entry, total, e2e_steps(lambda: fn(u, delta, A, Bm, Cm, Dk, z, o), hin, (u, delta, Bm, Cm, z), o, ho, flush, d))
            del hin
        del u, z, delta, A, Bm, Cm, Dk, o
        torch.cuda.empty_cache()
        if do_parity:
            from oracle import inputs, selective_scan as oscan
            ns_d = 2048
            sargs = inputs.selective_scan_inputs(B=1, Dm=ns_d, L=c["L"], N=c["N"])
            fn_s = load_callable(programs.selective_scan_decl("scan_sample", 1, ns_d, c["L"], c["N"]), "scan_sample")
            os_ = torch.full((1, ns_d, c["L"]), float("nan"), dtype=bf, device=dev)
            fn_s(*(a.to(dev) for a in sargs), os_)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ref = oscan.selective_scan_reference(*sargs)
            secs = time.perf_counter() - t0
            sample = f"1 of {c['B']} sequences x {ns_d} of {c['Dm']} channels, full L, against the CPU oracle (sequential recurrence)"
            entry["parity"] = bracket_stats(os_, ref, BF16_ATOL) | {
                "tolerance": "2e-2, or one bf16 unit in the last place at the exact value's magnitude", "sample": sample}
            if do_cpu:
                entry["cpu_baseline"] = cpu_entry(secs, total * ns_d / (c["B"] * c["Dm"]), sample)

    # -- Mamba-2 SSD, heads sharded over ranks
    def run_ssd():
        c = dict(SSD, B=args.ssd_batch) if args.ssd_batch else dict(SSD)
        lo, hi = shard_range(c["H"], d.rank, d.world)
        Hl = hi - lo
        ws_bytes = runtime.ssd_workspace_bytes(c["B"], c["L"], Hl, c["P"], c["N"], c["G"], c["chunk"])
        fn = load_callable(programs.ssd_chunk_scan_decl("ssd", c["B"], c["L"], Hl, c["P"], c["N"], c["G"], c["chunk"], ws_bytes), "ssd")
        x = rnd((c["B"], c["L"], Hl, c["P"]))
        dt = torch.nn.functional.softplus(rnd((c["B"], c["L"], Hl), torch.float32))
        A = -torch.exp(torch.rand((Hl,), device=dev, generator=gen) * math.log(16.0))
        Bm, Cm = rnd((c["B"], c["L"], c["G"], c["N"])), rnd((c["B"], c["L"], c["G"], c["N"]))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        y = torch.empty_like(x)
        ms = timed_steps(lambda: fn(x, dt, A, Bm, Cm, ws, y), steps, warm, flush, d)
        runtime.check_workspace_status(ws)
        total = 2 * c["B"] * c["L"] * c["H"] * c["P"] * 2 + c["B"] * c["L"] * c["H"] * 4 + 2 * c["B"] * c["L"] * c["G"] * c["N"] * 2 + c["H"] * 4
        entry = record("ssd_chunk_scan", ms, total, {"config": "B=4 L=8192 H=64 P=64 N=128 chunk=256 (configs[4])"})
        if not args.skip_e2e:
            hin = tuple(pinned(t) for t in (x, dt, Bm, Cm))
            ho = torch.empty(y.shape, dtype=y.dtype).pin_memory()
            add_e2e(entry, total, e2e_steps(lambda: fn(x, dt, A, Bm, Cm, ws, y), hin, (x, dt, Bm, Cm), y, ho, flush, d))
            del hin
        if args.third_party and d.rank == 0:
            # FlashInfer's Blackwell SSD kernel on the same tensors, same harness: a yardstick, not a product path
            try:
                from flashinfer.mamba import SSDCombined
                op = SSDCombined(chunk_size=128, nheads=Hl, headdim=c["P"], dstate=c["N"], ngroups=c["G"], has_d=False)
                op.run(x, dt, A, Bm, Cm)
                ms_fi = timed_steps(lambda: op.run(x, dt, A, Bm, Cm), steps, warm, flush, d)
                entry["third_party"] = {"flashinfer_SSDCombined_ms": ms_fi}
            except Exception as exc:  # noqa: BLE001
                entry["third_party"] = {"flashinfer_SSDCombined": f"unavailable: {type(exc).__name__}: {str(exc)[:160]}"}
        del x, dt, A, Bm, Cm, ws, y
        torch.cuda.empty_cache()
        if do_parity:
            from oracle import inputs, ssd as ossd
            hs = 16
            sargs = inputs.ssd_inputs(B=1, L=c["L"], H=hs, P=c["P"], N=c["N"], G=c["G"])
            wsb = runtime.ssd_workspace_bytes(1, c["L"], hs, c["P"], c["N"], c["G"], c["chunk"])
            fn_s = load_callable(programs.ssd_chunk_scan_decl("ssd_sample", 1, c["L"], hs, c["P"], c["N"], c["G"], c["chunk"], wsb), "ssd_sample")
            wss = torch.empty(wsb, dtype=torch.uint8, device=dev)
            ys = torch.full((1, c["L"], hs, c["P"]), float("nan"), dtype=bf, device=dev)
            fn_s(*(a.to(dev) for a in sargs), wss, ys)
            torch.cuda.synchronize()
            runtime.check_workspace_status(wss)
            t0 = time.perf_counter()
            ref = ossd.ssd_reference(*sargs)
            secs = time.perf_counter() - t0
            sample = f"1 of {c['B']} batches x {hs} of {c['H']} heads, full L, against the CPU oracle (sequential recurrence)"
            entry["parity"] = bracket_stats(ys, ref, BF16_ATOL) | {
                "tolerance": "rms error <= 2^-8 rms(ref); with bf16 tensor-core operands 2e-2 absolute is unreachable at |y| of several hundred",
                "sample": sample}
            if do_cpu:
                sample_bytes = 2 * c["L"] * hs * c["P"] * 2 + c["L"] * hs * 4 + 2 * c["L"] * c["G"] * c["N"] * 2
                entry["cpu_baseline"] = cpu_entry(secs, sample_bytes, sample)

    for name, fn_ in (("attn1", run_attn1), ("decode", run_decode), ("decode1", run_decode1), ("scan", run_scan), ("ssd", run_ssd)):
        if name in want:
            fn_()
            torch.cuda.empty_cache()
            d.barrier()
    return out


def bench_reference_shape(args, d: Dist, dev, flush, pk) -> dict:
    """The reference's own problem (non-causal f16 1x32x4096x128) through this build's kernel and through the
    kernels that the reference's Triton, TileLang and cuTile translators emit for the same HTile program
    (stored as text under tests/golden/reference_emitted/, launched the way the reference's tests launch them).
    Same inputs, same L2 flush and CUDA-event harness; each reference kernel's output is compared with this
    build's.  Runs on rank 0 of a 1-GPU run."""
    from neptune_mlir import runtime

    c = REF_SHAPE
    shape = (c["B"], c["H"], c["S"], c["D"])
    flops = 4.0 * c["B"] * c["H"] * c["S"] * c["S"] * c["D"]
    gen = torch.Generator(device=dev).manual_seed(0)
    q, k, v = (torch.randn(shape, dtype=torch.float16, device=dev, generator=gen) for _ in range(3))
    steps, warm = max(3, min(args.steps, 10)), 3
    res: dict = {"config": "non-causal f16 B=1 H=32 S=4096 D=128: the reference's own HTile program and shape",
                 "flop_count": "4*B*H*S*S*D", "arms": {}}

    text = (ROOT / "tests" / "data" / "attention_f16_1x32x4096x128.mlir").read_text()
    fn = load_callable(text, "attention_f16")
    out = torch.full(shape, float("nan"), dtype=torch.float16, device=dev)
    ms = timed_steps(lambda: fn(q, k, v, out), steps, warm, flush, d)
    runtime.check_status(dev)
    res["arms"]["nb200"] = {"ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                            "frac_of_peak": flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"]}

    emitted = ROOT / "tests" / "golden" / "reference_emitted"

    def load_emitted(name):
        path = emitted / f"attention_f16_1x32x4096x128_{name}.py"
        spec = importlib.util.spec_from_file_location(f"reference_emitted_{name}", path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod
        spec.loader.exec_module(mod)
        return mod.attention_f16

    grid = (c["S"] // 128, c["H"], c["B"])

    def arm_triton():
        kern = load_emitted("triton")
        o = torch.empty_like(out)
        kern[grid](q, k, v, o)
        return (lambda: kern[grid](q, k, v, o)), (lambda: o)

    def arm_tilelang():
        import tilelang
        kern = tilelang.compile(load_emitted("tilelang"), out_idx=[3], execution_backend="tvm_ffi", target="cuda")
        holder = {}

        def run():
            r = kern(q, k, v)
            holder["o"] = r[0] if isinstance(r, (list, tuple)) else r
        run()
        return run, (lambda: holder["o"])

    def arm_cutile():
        import cuda.tile as ct
        kern = load_emitted("cutile")
        o = torch.empty_like(out)

        def run():
            stream = torch.cuda.current_stream()
            try:
                ct.launch(stream, grid, kern, (q, k, v, o))
            except TypeError:
                ct.launch(stream, grid, kern, q, k, v, o)
        run()
        return run, (lambda: o)

    for name, make in (("reference_triton", arm_triton), ("reference_tilelang", arm_tilelang), ("reference_cutile", arm_cutile)):
        t0 = time.perf_counter()
        try:
            run, get = make()
            torch.cuda.synchronize()
            jit_s = time.perf_counter() - t0
            ms_r = timed_steps(run, steps, warm, flush, d)
            diff = (get().float() - out.float()).abs().max().item()
            res["arms"][name] = {"ms_per_step": ms_r, "tflops": flops / (ms_r * 1e-3) / 1e12, "jit_seconds": jit_s,
                                 "max_abs_diff_vs_nb200": diff, "reference_tolerance": 1e-3}
        except Exception as exc:  # noqa: BLE001 - a JIT that cannot run here is reported, not fatal
            res["arms"][name] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    best = max((a["tflops"] for n, a in res["arms"].items() if n != "nb200" and "tflops" in a), default=None)
    res["nb200_over_best_reference_kernel"] = (res["arms"]["nb200"]["tflops"] / best) if best else None
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("native", "reference"), default="native")
    ap.add_argument("--skip-extra", action="store_true", help="attention only (skip decode and the scans)")
    ap.add_argument("--decode1-splits", type=int, default=0, help="splits of the single-sequence decode (0 = fill the SMs once)")
    ap.add_argument("--extra", default="attn1,decode,decode1,scan,ssd,refshape",
                    help="comma list of the secondary workloads to run (attn1, decode, decode1, scan, ssd, refshape)")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--skip-parity", action="store_true", help="skip the per-workload parity samples (profiler captures)")
    ap.add_argument("--skip-attention", action="store_true",
                    help="secondary workloads only (profiler captures of decode and the scans)")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer end-to-end legs")
    ap.add_argument("--merge", choices=("peer", "nccl"), default="peer",
                    help="merge of the sharded single-sequence decode at N > 1: the peer-memory kernel (default) or NCCL")
    ap.add_argument("--third-party", action="store_true", help="also time third-party kernels of the image as yardsticks")
    ap.add_argument("--decode-batch", type=int, default=0,
                    help="batch of the split-K decode workload (default: the full 64); reduced for profiler captures")
    ap.add_argument("--ssd-batch", type=int, default=0,
                    help="batch of the SSD workload (default: the full 4); reduced for profiler captures")
    ap.add_argument("--scan-batch", type=int, default=0,
                    help="batch of the selective-scan workload (default: the full 8); reduced for profiler captures")
    ap.add_argument("--attn-units", type=int, default=0,
                    help="number of (batch, head) units of the attention workload (default: the full 256); "
                         "a reduced count is for profiler captures only and is recorded in config")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup

    if args.impl == "reference":
        if args.steps == 200:
            args.steps = 5   # a CPU step takes seconds: keep the default run to well under a minute
        run_reference_arm(args)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py measures CUDA kernels; no CUDA device is visible (there is no CPU fallback)")
    d = Dist(args.gpus)
    dev = torch.device("cuda", d.local_rank)
    torch.cuda.set_device(dev)
    pk, pk_kind = peaks()
    flush = torch.empty(128 * 1024 * 1024, dtype=torch.float32, device=dev)  # 512 MB > L2

    cpu = None
    if d.rank == 0 and not args.skip_cpu and d.world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        heads = 128
        cpu_attention_sample(2)  # warm the thread pool
        secs, tf = cpu_attention_sample(heads)
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "seconds": secs,
               "sample": f"{heads} of {ATTN['B'] * ATTN['H']} (batch, head) units of the configuration, full S, "
                         "oracle attention_reference (the reference's check math plus the causal mask) on CPU tensors"}
    d.barrier()

    if args.skip_attention:
        attn = {"value": None, "ms": None, "roofline": None, "e2e": None, "gpu_launches": 0, "clocks": None}
    else:
        attn = bench_attention(args, d, dev, flush, pk, pk_kind)
    extra = {} if args.skip_extra else bench_extra(args, d, dev, flush, pk, pk_kind)
    if not args.skip_extra and "refshape" in args.extra.split(",") and d.world == 1:
        extra["reference_shape"] = bench_reference_shape(args, d, dev, flush, pk)

    if d.rank == 0:
        line = {
            "metric": "attn_prefill_tflops", "value": attn["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": attn["ms"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": attn_config(args.gpus) | ({"reduced_units": args.attn_units} if args.attn_units else {}),
            "roofline": attn["roofline"], "cpu_baseline": cpu, "e2e": attn["e2e"],
            "gpu_launches": attn["gpu_launches"], "clocks": attn["clocks"], "parity": attn.get("parity"),
            "workloads": extra,
        }
        print(json.dumps(line))
    if d.world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
