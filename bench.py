#!/usr/bin/env python3
"""Benchmark of the quantized Pi0.5 decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (seeded synthetic, stands in for real checkpoints): the NVFP4 weight-only GEMV
(M = 1) over the 54 MLP matrices of the Gemma-300M action expert -- 18 layers x
(gate 1024->4096, up 1024->4096, down 4096->1024), e2m1 codes uniform over the 16 codes,
2 per byte, E4M3 scale per 16 K-elements = blockamax/6 of an N(0, 0.02) matrix over an fp32
global scale, bf16 activations N(0,1), bf16 outputs.  A step is one pass over all 54
matrices.  Four independent weight sets (4 x 128 MB) are rotated from step to step, so
every step streams its weights from HBM, never from the 126 MB L2.

`value` times the pass with inputs resident in HBM (one grouped launch per step);
`e2e` times the same pass through the Python API with HOST activations and results
(pinned H2D / D2H copies inside the timed region).  N > 1 runs one independent replica per
GPU (no collective on the data path); the barrier and max-over-ranks use NCCL.

Besides the headline the JSON line carries `config1_int4_gemv` (the reference's own benchmark shape),
`pi05_latency_ms` (1 / 3 / 10 denoise steps, host to host) and `serving` (a batch of independent requests
split over the replicas), and `extras` with per-shape figures next to cuBLAS bf16 on the same shapes.

`--case NAME` runs one bounded kernel case instead (what the ncu commands in profiles/ execute):
gemm | gemm-nvfp4 | rowop | attention | pi05, with --iters launches inside cudaProfilerStart/Stop.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYERS = 18
HIDDEN, INTER = 1024, 4096
SHAPES = [(INTER, HIDDEN), (INTER, HIDDEN), (HIDDEN, INTER)]      # (N, K): gate, up, down
BLOCK = 16
NSETS = 4
# dram__bytes_read.sum + dram__bytes_write.sum of one grouped launch over this workload, from ncu captures of
# the two kernels (CUDA-core: 127.46 MB read + 3.97 MB written; tensor-core: 127.69 MB + 4.20 MB)
NCU_TRAFFIC_BYTES_PER_LAUNCH = {"cuda": 131436544, "tc": 130795264}
METRIC = "nvfp4_gemv_hbm_gbps"
UNIT = "GB/s"


def algorithmic_bytes(N, K, M=1):
    """codes + E4M3 block scales + fp32 global scale + bf16 activations + bf16 outputs."""
    return N * K // 2 + N * K // BLOCK + 4 + M * K * 2 + M * N * 2


STEP_BYTES = LAYERS * sum(algorithmic_bytes(n, k) for n, k in SHAPES)


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------ synthetic weights
def make_weight_set(seed, device):
    """54 problems: packed codes, E4M3 scale bytes, global scale -- generated on the device."""
    g = torch.Generator(device=device).manual_seed(seed)
    mats = []
    for layer in range(LAYERS):
        for (N, K) in SHAPES:
            base = torch.randn(N, K, generator=g, device=device) * 0.02
            gs = float(base.abs().max() / (6.0 * 448.0))
            bmax = base.reshape(N, K // BLOCK, BLOCK).abs().amax(dim=2)
            scales = (bmax / 6.0 / gs).clamp(max=448.0).to(torch.float8_e4m3fn).view(torch.uint8)
            packed = torch.randint(0, 256, (N, K // 2), generator=g, device=device, dtype=torch.uint8)
            mats.append((packed, scales, gs, N, K))
    return mats


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU, sampled in the background."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for (t, r) in self.rows if t0 - 0.05 <= t <= t1 + 0.15] or [r for (_, r) in self.rows]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------ our arm
def run_ours(args):
    from turbopi_b200 import _lib, ops
    from turbopi_b200.replicas import ReplicaGroup
    group = ReplicaGroup.from_env("nccl")
    rank, world, local, device = group.rank, group.world, group.local_rank, group.device
    _lib.load()

    x = {K: torch.randn(1, K, device=device, generator=torch.Generator(device=device).manual_seed(7)).to(torch.bfloat16)
         for K in (HIDDEN, INTER)}
    sets, groups, outs = [], [], []
    for s in range(NSETS):
        mats = make_weight_set(100 + s, device)
        o = [torch.empty((1, N), dtype=torch.bfloat16, device=device) for (_, _, _, N, _) in mats]
        probs = [dict(x=x[K], weight_packed=p, weight_scales=sc, out=oo, global_scale=gs)
                 for (p, sc, gs, N, K), oo in zip(mats, o)]
        sets.append(mats)
        outs.append(o)
        groups.append(ops.GroupedGemv(probs, BLOCK))
    stream = torch.cuda.current_stream(device)
    tcs = None
    if args.path == "tc":
        # tensor-core GEMV: a step = re-quantise the two activation vectors into residual pieces
        # (1 small launch) + ONE grouped GEMV launch over the 54 matrices, chained by programmatic
        # dependent launch (the GEMV requests its first weight blocks while the quantiser runs)
        tcs = []
        for s in range(NSETS):
            probs = [dict(x=x[K], weight_packed=p, weight_scales=sc, global_scale=gs, out=oo)
                     for (p, sc, gs, N, K), oo in zip(sets[s], outs[s])]
            tcs.append(ops.TcGemv(probs, pieces=3, pdl=not args.no_pdl, fused=not args.no_fuse))

    def launch_step(i):
        if tcs is not None:
            tcs[i % NSETS].launch()
        else:
            groups[i % NSETS].launch()

    step_graphs = None
    timed_graph = None
    if not args.no_graph:
        # one CUDA graph per weight set: a step is a single graph launch on the host side
        side = torch.cuda.Stream(device=device)
        with torch.cuda.stream(side):
            for s in range(NSETS):
                launch_step(s)
        torch.cuda.synchronize()
        step_graphs = []
        for s in range(NSETS):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                launch_step(s)
            step_graphs.append(g)
        # the timed region is ONE graph holding all `steps` passes (weight sets rotating), so that the
        # device, not the host's replay loop, paces it
        timed_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(timed_graph, stream=side):
            for i in range(args.steps):
                launch_step(i)

    def step(i):
        if step_graphs is not None:
            step_graphs[i % NSETS].replay()
        else:
            launch_step(i)

    sampler = ClockSampler(local) if rank == 0 else None
    t_wall0 = time.time()
    # warm-up: W steps, extended to ~0.4 s of GPU work so the clock sampler sees the kernel under load
    w = 0
    t_w = time.time()
    while w < args.warmup or (not args.no_clock_warmup and (time.time() - t_w) < 0.4):
        step(w)
        w += 1
        if w % 64 == 0:
            torch.cuda.synchronize()
    group.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()       # `ncu --profile-from-start off` captures the timed region only
    e0.record(stream)
    if timed_graph is not None:
        timed_graph.replay()
    else:
        for i in range(args.steps):
            step(i)
    e1.record(stream)
    group.barrier()
    torch.cuda.profiler.stop()
    ms = group.max_over_ranks(e0.elapsed_time(e1))
    launches = args.steps * (2 if (tcs is not None and args.no_fuse) else 1)
    per_launch_s = (e0.elapsed_time(e1) / 1e3) / args.steps   # the GEMV launch; the quantisers ride in its shadow

    # ---- end to end: host activations in, host results out, through the Python API --------------------
    hx = {K: x[K].cpu().pin_memory() for K in x}
    out_flat = [torch.cat([o.reshape(-1) for o in outs[s]]) for s in range(NSETS)]   # contiguous result buffers
    # re-point the problems at slices of one result buffer per set so the step's result is one D2H copy
    e2e_groups = []
    for s in range(NSETS):
        off, probs = 0, []
        for (p, sc, gs, N, K) in sets[s]:
            probs.append(dict(x=x[K], weight_packed=p, weight_scales=sc, out=out_flat[s][off:off + N].view(1, N),
                              global_scale=gs))
            off += N
        e2e_groups.append(ops.GroupedGemv(probs, BLOCK) if tcs is None else ops.TcGemv(probs, pieces=3, pdl=not args.no_pdl, fused=not args.no_fuse))
    h_out = torch.empty_like(out_flat[0], device="cpu").pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in hx.values())
    d2h = h_out.numel() * h_out.element_size()

    def e2e_body(sidx):
        for K in x:
            x[K].copy_(hx[K], non_blocking=True)          # pinned host -> device
        e2e_groups[sidx].launch()
        h_out.copy_(out_flat[sidx], non_blocking=True)    # device -> pinned host

    # a caller that repeats the step captures it once (copies included) and replays it
    e2e_graphs = None
    if not args.no_graph:
        side2 = torch.cuda.Stream(device=device)
        with torch.cuda.stream(side2):
            for sidx in range(NSETS):
                e2e_body(sidx)
        torch.cuda.synchronize()
        e2e_graphs = []
        for sidx in range(NSETS):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side2):
                e2e_body(sidx)
            e2e_graphs.append(g)

    def e2e_step(i):
        if e2e_graphs is not None:
            e2e_graphs[i % NSETS].replay()
        else:
            e2e_body(i % NSETS)
        stream.synchronize()                      # the caller has its result on the host

    for i in range(max(3, min(args.warmup, 20))):
        e2e_step(i)
    group.barrier()
    e2e_steps = args.steps
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for i in range(e2e_steps):
        e2e_step(i)
    f1.record(stream)
    group.barrier()
    e2e_ms = group.max_over_ranks(f0.elapsed_time(f1))
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    extras = {}
    if rank == 0 and not args.no_extras:
        extras = run_extras(device, sets, x)
    serving = None
    if not args.no_extras and not args.no_serving:
        try:
            serving = run_serving(group, device)          # every rank takes part; rank 0 gets the figures
        except Exception as e:                            # the headline must not depend on the side measurement
            serving = {"error": f"{type(e).__name__}: {e}"}
    dev_err = _lib.load().tpb200_device_error(0)

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        total_bytes = STEP_BYTES * args.steps * world
        value = total_bytes / (ms / 1e3) / 1e9
        achieved = STEP_BYTES / per_launch_s / 1e9
        traffic = NCU_TRAFFIC_BYTES_PER_LAUNCH[args.path]
        cpu = cpu_baseline_sample() if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": ("f16 products / f32 accumulate" if tcs is None else
                      "e2m1 x e2m1 block-scaled tensor-core products / f32 accumulate (bf16 activations as 3 e2m1 pieces)"),
            "data": "synthetic",
            "config": {"workload": "NVFP4 weight-only GEMV, M=1, Gemma-300M action-expert MLP, 18 layers x "
                                   "(gate,up 1024->4096; down 4096->1024) = 54 matrices per step, E4M3 block-16 "
                                   "scales + fp32 global scale, bf16 in/out",
                       "launch": ("one grouped launch per step (tpb200_nvfp4_gemv_grouped)" if tcs is None else
                                  ("activation-piece quantiser + one grouped tensor-core launch per step "
                                   "(tpb200_nvfp4_quantize_acts_tc, tpb200_nvfp4_gemv_tc)" if args.no_fuse else
                                   "ONE grouped tensor-core launch per step, activations quantised inside it "
                                   "(tpb200_nvfp4_gemv_tc_fused)") +
                                  ("" if args.no_pdl else ", steps chained by programmatic dependent launch")),
                       "l2": f"{NSETS} weight sets of {STEP_BYTES / 1e6:.1f} MB rotated per step (> 126 MB L2)",
                       "graph": ("the timed region is one CUDA graph of all steps (device-paced)" if timed_graph is not None
                                 else "direct launches"),
                       "parallelism": f"{world} independent replica(s), no collective",
                       "warmup_note": "warm-up extended to >= 0.4 s so clocks are sampled under load"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_kind": f"of {peak_kind}",
                         "algorithmic_bytes_per_launch": STEP_BYTES, "nominal_peak": 8000.0,
                         "frac_of_nominal": achieved / 8000.0},
            "cpu_baseline": cpu,
            "e2e": {"value": STEP_BYTES * e2e_steps * world / (e2e_ms / 1e3) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "device_error": dev_err,
            "config1_int4_gemv": extras.get("w4a16_int4_rowmajor_g128_16384x2048"),
            "pi05_latency_ms": {k.split("_")[2]: v["ms_median"] for k, v in extras.items()
                                if k.startswith("pi05_e2e_") and isinstance(v, dict)} or None,
            "serving": serving,
            "extras": extras,
        }
        print(json.dumps(line))
    group.close()


def time_launches(fn, iters, warm=20):
    """Seconds per launch of fn(i) with the launches captured in ONE CUDA graph (rotating through
    `iters` argument sets), so the figure is device time per launch, not Python call overhead."""
    stream = torch.cuda.current_stream()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(min(warm, iters)):
            fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for i in range(iters):
            fn(i)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    reps = 5
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(reps):
        g.replay()
    b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (iters * reps) * 1e-3


def time_replays(fn, iters):
    stream = torch.cuda.current_stream()
    for i in range(8):
        fn(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for i in range(iters):
        fn(i)
    b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def run_extras(device, sets, x):
    """Per-configuration figures that explain the headline: single launches per shape and M,
    the dependent chain under programmatic dependent launch in a CUDA graph, and the INT4
    W4A16 GEMV of the reference's own benchmark shape."""
    from turbopi_b200 import ops
    ex = {}
    # (a) one launch per matrix, rotating through all 216 matrices (> L2), M in {1, 4, 16}
    flat = [m for s in sets for m in s]
    for M in (1, 4, 16):
        xm = {K: torch.randn(M, K, device=device).to(torch.bfloat16) for K in (HIDDEN, INTER)}
        om = {N: torch.empty((M, N), dtype=torch.bfloat16, device=device) for N in (HIDDEN, INTER)}
        for (Nsel, Ksel, name) in ((INTER, HIDDEN, "gateup_1024x4096"), (HIDDEN, INTER, "down_4096x1024")):
            ms_ = [m for m in flat if m[3] == Nsel]

            def fn(i, ms_=ms_, xm=xm, om=om, Nsel=Nsel, Ksel=Ksel):
                p, sc, gs, N, K = ms_[i % len(ms_)]
                ops.nvfp4_gemv_out(xm[Ksel], p, sc, om[Nsel], block_size=BLOCK, global_scale=gs)
            t = time_launches(fn, 216)
            ex[f"single_launch_M{M}_{name}"] = {"us": t * 1e6, "gbps": algorithmic_bytes(Nsel, Ksel, M) / t / 1e9}
    # (b) the 54 GEMVs as 54 launches with programmatic dependent launch, captured in one CUDA graph per set
    graphs = []
    side = torch.cuda.Stream(device=device)
    outs = [torch.empty((1, N), dtype=torch.bfloat16, device=device) for (_, _, _, N, _) in sets[0]]
    for pdl in (False, True):
        gl = []
        for s in range(NSETS):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                for (p, sc, gs, N, K), o in zip(sets[s], outs):     # warm the launch path on the side stream
                    ops.nvfp4_gemv_out(x[K], p, sc, o, block_size=BLOCK, global_scale=gs, pdl=pdl)
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=side):
                for (p, sc, gs, N, K), o in zip(sets[s], outs):
                    ops.nvfp4_gemv_out(x[K], p, sc, o, block_size=BLOCK, global_scale=gs, pdl=pdl)
            gl.append(g)
        t = time_replays(lambda i, gl=gl: gl[i % NSETS].replay(), 200)
        ex["graph_54_launches_pdl" if pdl else "graph_54_launches"] = {
            "us_per_step": t * 1e6, "gbps": STEP_BYTES / t / 1e9, "us_per_launch": t * 1e6 / 54}
        graphs.append(gl)
    # (c) W4A16 INT4 GEMV, N=16384 K=2048 g=128 row-major, bf16; 16 rotating weight buffers (277 MB)
    N, K, G = 16384, 2048, 128
    ws = [torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), device=device, dtype=torch.int32) for _ in range(16)]
    sc = [(torch.rand(N, K // G, device=device) * 0.015 + 0.005).to(torch.float16) for _ in range(16)]
    xi = torch.randn(1, K, device=device).to(torch.bfloat16)
    oi = torch.empty((1, N), dtype=torch.bfloat16, device=device)
    nbytes = N * K // 2 + N * (K // G) * 2 + K * 2 + N * 2
    t = time_launches(lambda i: ops.w4a16_gemv_out(xi, ws[i % 16], sc[i % 16], oi, group_size=G, layout=1, pdl=True), 64)
    t_plain = time_launches(lambda i: ops.w4a16_gemv_out(xi, ws[i % 16], sc[i % 16], oi, group_size=G, layout=1), 64)
    ex["w4a16_int4_rowmajor_g128_16384x2048"] = {"us": t * 1e6, "gbps": nbytes / t / 1e9, "bytes": nbytes,
                                                 "launch": "64 launches in one graph, chained by programmatic dependent launch "
                                                           "(as the headline's steps are)",
                                                 "us_without_pdl": t_plain * 1e6}
    # reference layout (K/32, N, 4) g=32, fp16 in / fp32 out
    wk = [torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 32, N, 4), device=device, dtype=torch.int32) for _ in range(16)]
    sk = [(torch.rand(K // 32, N, device=device) * 0.015 + 0.005).to(torch.float16) for _ in range(16)]
    xh = torch.randn(1, K, device=device).to(torch.float16)
    of = torch.empty((1, N), dtype=torch.float32, device=device)
    nbytes = N * K // 2 + N * (K // 32) * 2 + K * 2 + N * 4
    t = time_launches(lambda i: ops.w4a16_gemv_out(xh, wk[i % 16], sk[i % 16], of, group_size=32, layout=0), 64)
    ex["w4a16_int4_kblock_g32_16384x2048"] = {"us": t * 1e6, "gbps": nbytes / t / 1e9, "bytes": nbytes}
    # (d) NVFP4 GEMV at the Gemma-2B shapes (18.9 MB each), 12 rotating buffers
    for (N, K, name) in ((16384, 2048, "gemma2b_gateup_2048x16384"), (2048, 16384, "gemma2b_down_16384x2048")):
        wp = [torch.randint(0, 256, (N, K // 2), device=device, dtype=torch.uint8) for _ in range(12)]
        sp = [torch.randint(40, 120, (N, K // 16), device=device, dtype=torch.uint8) for _ in range(12)]
        xb = torch.randn(1, K, device=device).to(torch.bfloat16)
        ob = torch.empty((1, N), dtype=torch.bfloat16, device=device)
        t = time_launches(lambda i: ops.nvfp4_gemv_out(xb, wp[i % 12], sp[i % 12], ob, block_size=16,
                                                       global_scale=1e-3), 48)
        ex[f"nvfp4_single_launch_{name}"] = {"us": t * 1e6, "gbps": algorithmic_bytes(N, K) / t / 1e9}
    # (f) the same 54-matrix pass on the tensor-core GEMV (activation pieces + one grouped launch)
    tcs = []
    for sidx in range(NSETS):
        probs = [dict(x=x[K], weight_packed=p, weight_scales=sc, global_scale=gs,
                      out=torch.empty((1, N), dtype=torch.bfloat16, device=device)) for (p, sc, gs, N, K) in sets[sidx]]
        tcs.append(ops.TcGemv(probs, pieces=3, fused=False))
    t = time_launches(lambda i: tcs[i % NSETS].launch(), 64)
    ex["tc_grouped_54_quantiser_launch_plus_gemv"] = {"us_per_step": t * 1e6, "gbps": STEP_BYTES / t / 1e9}
    t = time_launches(lambda i: tcs[i % NSETS].gemv(), 64)
    ex["tc_grouped_54_gemv_on_pretiled_activations"] = {"us_per_step": t * 1e6, "gbps": STEP_BYTES / t / 1e9}
    for (Nsel, Ksel, name) in ((INTER, HIDDEN, "gateup_1024x4096"), (HIDDEN, INTER, "down_4096x1024")):
        ms_ = [m for m in flat if m[3] == Nsel][:24]
        for M in (1, 4, 16):
            xm = torch.randn(M, Ksel, device=device).to(torch.bfloat16)
            singles = [ops.TcGemv([dict(x=xm, weight_packed=p, weight_scales=sc, global_scale=gs,
                                        out=torch.empty((M, N), dtype=torch.bfloat16, device=device))], pieces=3,
                                  fused=M <= 4)          # the library's own rule: more than 4 tokens -> quantiser launch + GEMV
                       for (p, sc, gs, N, K) in ms_]
            for pdl in (False, True):
                for sg in singles:
                    sg.flags = ops.FLAG_PDL if pdl else ops.FLAG_NONE
                t = time_launches(lambda i: singles[i % len(singles)].launch(), 48)
                ex[f"tc_single_launch_M{M}_{name}" + ("_pdl" if pdl else "")] = {
                    "us": t * 1e6, "gbps": algorithmic_bytes(Nsel, Ksel, M) / t / 1e9}
            del singles
    del tcs
    # (e) prefix NVFP4 x NVFP4 GEMMs on tcgen05 (e2m1 activations and weights, UE4M3 block-16 scales)
    for (M, N, K, name) in ((712, 16384, 2048, "gemma2b_gateup_M712"), (712, 2048, 16384, "gemma2b_down_M712"),
                            (512, 4304, 1152, "siglip_fc1_M512"), (512, 1152, 4304, "siglip_fc2_M512")):
        pitch = ops.packed_pitch(K)
        nb = 4
        a = torch.randint(0, 256, (M, pitch), device=device, dtype=torch.uint8)
        a_sf = torch.randint(40, 120, (ops.nvfp4_sf_bytes(M, K),), device=device, dtype=torch.uint8)
        bs = [torch.randint(0, 256, (N, pitch), device=device, dtype=torch.uint8) for _ in range(nb)]
        b_sf = [torch.randint(40, 120, (ops.nvfp4_sf_bytes(N, K),), device=device, dtype=torch.uint8) for _ in range(nb)]
        o = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        t = time_launches(lambda i: ops.nvfp4_gemm(a, a_sf, bs[i % nb], b_sf[i % nb], M, N, K, alpha=1e-4, out=o), 16)
        flops = 2.0 * M * N * K
        bytes_ = M * K // 2 + M * K // 16 + N * K // 2 + N * K // 16 + M * N * 2
        xb_ = torch.randn(M, K, device=device).to(torch.bfloat16)
        wb_ = [(torch.randn(N, K, device=device) * 0.02).to(torch.bfloat16) for _ in range(2)]
        tb = time_launches(lambda i: torch.nn.functional.linear(xb_, wb_[i % 2]), 16)
        ex[f"nvfp4_gemm_{name}"] = {"us": t * 1e6, "tflops": flops / t / 1e12, "gbps": bytes_ / t / 1e9,
                                    "cublas_bf16_us": tb * 1e6, "cublas_bf16_tflops": flops / tb / 1e12}
        del wb_
        xq = torch.randn(M, K, device=device).to(torch.bfloat16)
        pk, sf = ops.nvfp4_quantize_act(xq)
        t = time_launches(lambda i: ops.nvfp4_quantize_act(xq, pk, sf), 16)
        ex[f"nvfp4_quantize_act_{M}x{K}"] = {"us": t * 1e6, "gbps": (M * K * 2 + M * K // 2 + M * K // 16) / t / 1e9}
    # (g) the model's linears as they run in the pipeline: bf16 activations -> 3 residual e2m1 pieces (row
    # kernel), NVFP4 weights; the two large prefix MLP matrices on the tiled images (128 x 256 output tiles), the
    # other shapes in the row-major operand form (128 x 128 tiles), chained by programmatic dependent launch as
    # in the pipeline (benchmark config 4 with weight-only semantics; `tflops` counts the useful 2 M N K once,
    # not the 3 pieces; `tiled_gemm_us`: the same shape on the tiled images)
    from turbopi_b200 import _lib as tlib
    from turbopi_b200.pi05 import TcLinear
    gemm_ws = ops.gemm_workspace(device)
    for (M, N, K, name) in ((712, 32768, 2048, "gemma2b_gate_up_M712"), (712, 2048, 16384, "gemma2b_down_M712"),
                            (712, 2560, 2048, "gemma2b_qkv_M712"), (512, 4304, 1152, "siglip_fc1_M512"),
                            (512, 1152, 4304, "siglip_fc2_M512"), (50, 8192, 1024, "expert_gate_up_M50"),
                            (50, 1024, 4096, "expert_down_M50")):
        rowmajor = N * K < (1 << 25)            # the pipeline's rule: everything but the prefix gate_up / down
        xq = torch.randn(M, K, device=device).to(torch.bfloat16)
        o = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        weights_ = [torch.randn(N, K, device=device) * 0.02 for _ in range(2)]
        times = {}
        for form in ((False, True) if rowmajor else (False,)):
            q = ops.QuantBuf(M, K, 3, device, tiled=not form)
            lins = [TcLinear.from_weight(w_, rowmajor=form) for w_ in weights_]
            for l_ in lins:
                l_.ws = gemm_ws
            ops.rowop(tlib.ROW_NONE, xq, K, q)
            with ops.launch_flags(ops.FLAG_PDL):
                times[form] = (time_launches(lambda i: lins[i % 2](q, o), 16),
                               time_launches(lambda i: ops.rowop(tlib.ROW_NONE, xq, K, q), 16))
            del lins
        del weights_
        t, tq = times[rowmajor]
        # the library comparator on the same shape: torch F.linear in bf16 (cuBLAS), weights rotating too
        wb = [(torch.randn(N, K, device=device) * 0.02).to(torch.bfloat16) for _ in range(2)]
        tb = time_launches(lambda i: torch.nn.functional.linear(xq, wb[i % 2]), 16)
        ex[f"w4a16_tc_linear_{name}"] = {"gemm_us": t * 1e6, "quantise_us": tq * 1e6,
                                         "form": "row-major operands, 128x128 tiles" if rowmajor else "tiled images, 128x256 tiles",
                                         "tflops": 2.0 * M * N * K / t / 1e12,
                                         "tensor_tflops": 3 * 2.0 * M * N * K / t / 1e12,
                                         "cublas_bf16_us": tb * 1e6, "cublas_bf16_tflops": 2.0 * M * N * K / tb / 1e12}
        if rowmajor:
            ex[f"w4a16_tc_linear_{name}"]["tiled_gemm_us"] = times[False][0] * 1e6
        del wb
    # (e2) the same NVFP4 x NVFP4 products on the tiled operand images (one e2m1 activation piece, 128 x 256 tiles):
    # the form the prefix would run with e2m1 activations
    for (M, N, K, name) in ((712, 16384, 2048, "gemma2b_gateup_M712"), (712, 2048, 16384, "gemma2b_down_M712")):
        q1 = ops.QuantBuf(M, K, 1, device)
        xq = torch.randn(M, K, device=device).to(torch.bfloat16)
        lins = [TcLinear.from_weight(torch.randn(N, K, device=device) * 0.02) for _ in range(2)]
        for l_ in lins:
            l_.ws = gemm_ws
        o = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        ops.rowop(tlib.ROW_NONE, xq, K, q1)
        t = time_launches(lambda i: lins[i % 2](q1, o), 16)
        ex[f"nvfp4_gemm_tiled_1piece_{name}"] = {"us": t * 1e6, "tflops": 2.0 * M * N * K / t / 1e12}
        del lins
    # (g0) this GPU's own e2m1 block-scaled MMA rate: back-to-back 128 x 256 x 64 MMAs on resident operands, one
    # CTA per SM -- the measured denominator for the GEMM rates above (the nominal dense FP4 figure is 9 PFLOP/s)
    lib = tlib.load()
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    stream_h = torch.cuda.current_stream(device).cuda_stream
    for mmas in (2000, 20000):
        tlib.check(lib.tpb200_measure_fp4_mma_rate(mmas, stream_h), "fp4 mma rate")     # the first call also warms up
    torch.cuda.synchronize()
    rates = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        tlib.check(lib.tpb200_measure_fp4_mma_rate(20000, stream_h), "fp4 mma rate")
        b.record()
        torch.cuda.synchronize()
        rates.append(sms * 20000 * 4194304.0 / (a.elapsed_time(b) * 1e-3) / 1e12)
    rates.sort()
    ex["fp4_mma_rate_measured"] = {"tflops": rates[len(rates) // 2], "mma": "tcgen05.mma kind::mxf4nvf4 128x256x64, no loads",
                                   "nominal_tflops": 9000.0}
    # (g1) INT4 x bf16 GEMM on the tensor cores (w4a16GemmForward's operands) at the prefix shape, next to cuBLAS bf16
    for (M, N, K, name) in ((712, 16384, 2048, "gemma2b_gateup_M712"), (712, 2048, 16384, "gemma2b_down_M712"),
                            (64, 16384, 2048, "gemma2b_gateup_M64")):
        xq = torch.randn(M, K, device=device).to(torch.bfloat16)
        wq = [torch.randint(-128, 128, (N, K // 2), device=device, dtype=torch.int8) for _ in range(2)]
        sq = (torch.rand(N, K // 128, device=device) * 0.01 + 0.002).to(torch.bfloat16)
        o = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        t = time_launches(lambda i: ops.w4a16_gemm(xq, wq[i % 2], sq, None, None, o, tlib.INT4_PLUGIN), 16)
        wb = [(torch.randn(N, K, device=device) * 0.02).to(torch.bfloat16) for _ in range(2)]
        tb = time_launches(lambda i: torch.nn.functional.linear(xq, wb[i % 2]), 16)
        ex[f"w4a16_int4_tc_gemm_{name}"] = {"us": t * 1e6, "tflops": 2.0 * M * N * K / t / 1e12, "cublas_bf16_us": tb * 1e6,
                                            "cublas_bf16_tflops": 2.0 * M * N * K / tb / 1e12}
        del wq, wb
    # (g2) attention on the tensor cores next to torch's scaled_dot_product_attention (library kernels)
    import torch.nn.functional as F
    for (rows, keys, name) in ((712 * 8, 712, "prefix_712x8_on_712"), (50 * 8, 762, "expert_50x8_on_762")):
        qm = torch.randn(rows, 256, device=device).to(torch.bfloat16)
        km = torch.randn(keys, 256, device=device).to(torch.bfloat16)
        vm = torch.randn(keys, 256, device=device).to(torch.bfloat16)
        om = torch.empty_like(qm)
        ws = ops.attention_workspace(rows, keys, 256, 1, device)
        t = time_launches(lambda i: ops.attention(qm, km, vm, om, 1 / 16, None, ws), 16)
        q4 = qm.view(rows // 8, 8, 256).transpose(0, 1)[None]
        ts = time_launches(lambda i: F.scaled_dot_product_attention(q4, km[None, None], vm[None, None], enable_gqa=True), 16)
        ex[f"attention_{name}"] = {"us": t * 1e6, "torch_sdpa_us": ts * 1e6,
                                   "tflops": 4.0 * rows * keys * 256 / t / 1e12}
    # (g3) the drop-in module surface: NVFP4PackedMLP.forward on Gemma-2B's MLP, decode and prefix token counts
    from turbopi_b200.nvfp4_packed import NVFP4PackedMLP

    class _Mlp(torch.nn.Module):
        def __init__(self, h, i):
            super().__init__()
            self.gate_proj = torch.nn.Linear(h, i, bias=False)
            self.up_proj = torch.nn.Linear(h, i, bias=False)
            self.down_proj = torch.nn.Linear(i, h, bias=False)

    src = _Mlp(2048, 16384).to(device)
    for prm in src.parameters():
        prm.data.normal_(0, 0.02)
    mlp = NVFP4PackedMLP.from_gemma_mlp(src, gate_activation="gelu", fmt="nvfp4")
    del src
    for T in (1, 712):
        xm = torch.randn(T, 2048, device=device).to(torch.bfloat16)
        with torch.no_grad():
            t = time_launches(lambda i: mlp(xm), 8)
        ex[f"nvfp4_packed_mlp_forward_gemma2b_M{T}"] = {"us": t * 1e6, "weight_bytes": 3 * 2048 * 16384 * 9 // 16,
                                                        "gbps": 3 * 2048 * 16384 * 9 / 16 / t / 1e9}
    del mlp
    # (h) the whole Pi0.5-shaped inference (SigLIP-So400m/14 on 2 images, 712-token Gemma-2B prefix with the
    # fused QKV + RoPE + KV-cache append, Gemma-300M action expert, Euler steps) as ONE CUDA graph:
    # pinned host images / tokens / noise in, actions back on the host, random-init weights
    from turbopi_b200.pi05 import Pi05, Pi05Config
    cfg = Pi05Config()
    model = Pi05(cfg, device, seed=0)
    gen = torch.Generator().manual_seed(1)
    images = torch.randint(0, 256, (cfg.num_images, cfg.image_size, cfg.image_size, 3), generator=gen,
                           dtype=torch.uint8).pin_memory()
    tokens = torch.randint(0, cfg.vocab, (cfg.text_len,), generator=gen).pin_memory()
    noise = torch.randn(cfg.action_horizon, cfg.action_dim, generator=gen).pin_memory()
    host_out = torch.empty(cfg.action_horizon, cfg.action_dim).pin_memory()
    for steps in (1, 3, 10):
        with torch.no_grad():
            model.infer(images, tokens, noise, steps)          # captures the graph for this step count
            torch.cuda.synchronize()
            ts = []
            for _ in range(10):
                t0 = time.perf_counter()
                host_out.copy_(model.infer(images, tokens, noise, steps), non_blocking=True)
                torch.cuda.synchronize()
                ts.append((time.perf_counter() - t0) * 1e3)
        ts.sort()
        ex[f"pi05_e2e_{steps}_steps"] = {"ms_median": ts[len(ts) // 2], "ms_best": ts[0], "hz": 1e3 / ts[len(ts) // 2],
                                         "finite": bool(torch.isfinite(host_out).all())}
    ex["pi05_e2e_note"] = ("host wall clock around H2D inputs + one graph replay + D2H actions; reference on Jetson Thor "
                           "(its published figures, other hardware): 83.5 ms / 1 step, 102.8 ms / 3 steps, 171.4 ms / 10 steps")
    del model
    return ex


# ------------------------------------------------------------------------------------------ serving
def run_serving(group, device, steps=10):
    """Batches of 8 and 64 independent Pi0.5 requests split over the replicas (contiguous chunks, one
    captured graph per GPU, results gathered on the host of rank 0; no collective on the data path):
    requests/s and p50 / p99 request latency."""
    from turbopi_b200.pi05 import Pi05, Pi05Config
    from turbopi_b200.policy import Pi05Policy
    from turbopi_b200.replicas import RequestDispatcher
    cfg = Pi05Config()
    # four pipelines over ONE set of weights per replica, each with buffers, KV cache and scratch of its own: an
    # inference is a chain of ~600 short dependent launches that leaves most SMs idle, four chains side by side
    # (one host thread + one stream each) fill them.  `one_in_flight` is the same batch through one pipeline.
    # one spinning host thread per pipeline: no more of them than the host has cores for all replicas
    lanes = max(1, min(4, (os.cpu_count() or 1) // max(1, group.world)))
    first = Pi05(cfg, device, seed=0)
    policies = [Pi05Policy(first if k == 0 else Pi05.sharing_weights(first), None, None, num_denoising_steps=steps)
                for k in range(lanes)]
    policy = policies[0]
    rng = np.random.default_rng(3)

    def request(i):
        return {"observation/image": rng.integers(0, 256, (cfg.image_size, cfg.image_size, 3), dtype=np.uint8),
                "observation/wrist_image": rng.integers(0, 256, (cfg.image_size, cfg.image_size, 3), dtype=np.uint8),
                "observation/state": rng.normal(size=8).astype(np.float32),
                "prompt": [2] + rng.integers(3, cfg.vocab, 12 + i % 20).tolist(), "noise": None}

    for p_ in policies:
        p_.warmup(2)
    infer_fns = [(lambda r, p_=p_: p_.infer(r)["actions"]) for p_ in policies]
    disp = RequestDispatcher(group, infer_fns, timeout_s=120.0)
    single = RequestDispatcher(group, infer_fns[0], port=int(os.environ.get("MASTER_PORT", "29500")) + 18, timeout_s=120.0)
    out = {"denoise_steps": steps, "replicas": group.world, "pipelines_in_flight_per_replica": lanes}

    def run(d, batch):
        reqs = [request(i) for i in range(batch)]
        group.barrier()
        results, stats = d.serve(reqs)
        group.barrier()
        if group.rank != 0:
            return None
        return {"requests_per_s": stats["requests_per_s"], "p50_ms": stats["p50_ms"], "p99_ms": stats["p99_ms"],
                "wall_s": stats["wall_s"], "requeued": len(stats["requeued"]),
                "finite": bool(all(np.isfinite(r).all() for r in results))}

    run(disp, 2 * lanes * group.world)           # untimed: the first replay of a graph on a new stream uploads it
    run(single, group.world)
    for batch in (8, 64):
        out[f"batch_{batch}"] = run(disp, batch)
    out["one_in_flight"] = {"batch_64": run(single, 64)}
    del policies, policy
    return out if group.rank == 0 else None


# ------------------------------------------------------------------------------------------ profiling cases
def run_case(args):
    """One bounded kernel case for ncu (`--profile-from-start off` sees exactly the --iters launches)."""
    from turbopi_b200 import _lib as tlib, ops
    from turbopi_b200.pi05 import Pi05, Pi05Config, TcLinear
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)

    def timed(fn, iters, warm=2):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.profiler.start()
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return a.elapsed_time(b) / iters

    M, N, K = args.M, args.N, args.K
    if args.case == "gemm":            # weight-only linear: activation-piece quantiser + tiled tcgen05 GEMM
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        lin = TcLinear.from_weight(torch.randn(N, K, device=dev, generator=g) * 0.02, rowmajor=args.rowmajor)
        lin.ws = ops.gemm_workspace(dev)
        q = ops.QuantBuf(M, K, args.pieces, dev, tiled=not args.rowmajor)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)

        def step():
            ops.rowop(tlib.ROW_NONE, x, K, q)
            lin(q, out)
        ms = timed(step, args.iters)
        print(f"gemm M={M} N={N} K={K} pieces={args.pieces}: {ms * 1e3:.1f} us per quantise+GEMM, "
              f"{2.0 * M * N * K / (ms * 1e-3) / 1e12:.0f} TFLOP/s useful")
    elif args.case == "gemm-nvfp4":    # e2m1 x e2m1, row-major operands
        pitch = ops.packed_pitch(K)
        a = torch.randint(0, 256, (M, pitch), device=dev, dtype=torch.uint8)
        a_sf = torch.randint(40, 120, (ops.nvfp4_sf_bytes(M, K),), device=dev, dtype=torch.uint8)
        b = torch.randint(0, 256, (N, pitch), device=dev, dtype=torch.uint8)
        b_sf = torch.randint(40, 120, (ops.nvfp4_sf_bytes(N, K),), device=dev, dtype=torch.uint8)
        o = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.nvfp4_gemm(a, a_sf, b, b_sf, M, N, K, alpha=1e-4, out=o), args.iters)
        print(f"gemm-nvfp4 M={M} N={N} K={K}: {ms * 1e3:.1f} us, {2.0 * M * N * K / (ms * 1e-3) / 1e12:.0f} TFLOP/s")
    elif args.case == "rowop":
        x = torch.randn(M, 2 * K, device=dev, generator=g).to(torch.bfloat16)
        q = ops.QuantBuf(M, K, args.pieces, dev)
        ms = timed(lambda: ops.rowop(tlib.ROW_GELU_MUL, x, K, q), args.iters)
        print(f"rowop GELU*up + 3-piece quantiser M={M} K={K}: {ms * 1e3:.1f} us")
    elif args.case == "attention":
        rows, keys = args.M, args.N
        qm = torch.randn(rows, 256, device=dev, generator=g).to(torch.bfloat16)
        km = torch.randn(keys, 256, device=dev, generator=g).to(torch.bfloat16)
        vm = torch.randn(keys, 256, device=dev, generator=g).to(torch.bfloat16)
        o = torch.empty_like(qm)
        ws = ops.attention_workspace(rows, keys, 256, 1, dev)
        ms = timed(lambda: ops.attention(qm, km, vm, o, 1 / 16, None, ws), args.iters)
        print(f"attention rows={rows} keys={keys} d=256: {ms * 1e3:.1f} us per call (partial + combine)")
    elif args.case == "int4-gemm":     # bf16 x int4 (plugin layout, group 128) on the tensor cores
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        w = torch.randint(-128, 128, (N, K // 2), device=dev, dtype=torch.int8)
        sc = (torch.rand(N, K // 128, device=dev) * 0.01 + 0.002).to(torch.bfloat16)
        o = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.w4a16_gemm(x, w, sc, None, None, o, tlib.INT4_PLUGIN), args.iters)
        print(f"int4-gemm M={M} N={N} K={K}: {ms * 1e3:.1f} us, {2.0 * M * N * K / (ms * 1e-3) / 1e12:.0f} TFLOP/s")
    elif args.case == "int4-gemv":     # the reference's (K/32, N, 4) layout, one fp16 row
        x = torch.randn(1, K, device=dev, generator=g).to(torch.float16)
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 32, N, 4), device=dev, dtype=torch.int32)
        sc = (torch.rand(K // 32, N, device=dev) * 0.015 + 0.005).to(torch.float16)
        ms = timed(lambda: ops.w4a16_gemv(x, w, sc), args.iters)
        print(f"int4-gemv N={N} K={K} (k-block layout, group 32): {ms * 1e3:.1f} us per call")
    elif args.case == "int4-gemv-rowmajor":   # benchmark config 1: row-major [N, K/8] words, group 128, one bf16 row
        x = torch.randn(1, K, device=dev, generator=g).to(torch.bfloat16)
        ws = [torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), device=dev, dtype=torch.int32) for _ in range(8)]
        sc = (torch.rand(N, K // 128, device=dev) * 0.015 + 0.005).to(torch.float16)
        o = torch.empty((1, N), dtype=torch.bfloat16, device=dev)
        it = [0]

        def step():                    # eight weight matrices in turn: 8 x N x K / 2 bytes, more than the L2 holds at config 1
            it[0] += 1
            ops.w4a16_gemv_out(x, ws[it[0] % 8], sc, o, group_size=128, layout=1)
        ms = timed(step, args.iters)
        print(f"int4-gemv N={N} K={K} (row-major layout, group 128): {ms * 1e3:.1f} us per call")
    elif args.case == "quantize":      # bf16 activations -> e2m1 codes + swizzled UE4M3 scales
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        packed, sf = ops.nvfp4_quantize_act(x)
        ms = timed(lambda: ops.nvfp4_quantize_act(x, packed, sf), args.iters)
        print(f"quantize M={M} K={K}: {ms * 1e3:.1f} us per call")
    elif args.case == "pi05":
        cfg = Pi05Config()
        model = Pi05(cfg, dev, seed=0)
        gen = torch.Generator().manual_seed(1)
        images = torch.randint(0, 256, (cfg.num_images, cfg.image_size, cfg.image_size, 3), generator=gen, dtype=torch.uint8)
        tokens = torch.randint(0, cfg.vocab, (cfg.text_len,), generator=gen)
        noise = torch.randn(cfg.action_horizon, cfg.action_dim, generator=gen)
        with torch.no_grad():
            ms = timed(lambda: model.infer(images, tokens, noise, args.denoise_steps, use_graph=False), args.iters, warm=1)
        print(f"pi05 {args.denoise_steps} denoise step(s), eager launches: {ms:.2f} ms per inference")
    print("device_error", tlib.load().tpb200_device_error(0))


# ------------------------------------------------------------------------------------------ CPU arms
def _cpu_layer(seed):
    g = torch.Generator().manual_seed(seed)
    mats = []
    for (N, K) in SHAPES:
        base = torch.randn(N, K, generator=g) * 0.02
        gs = float(base.abs().max() / (6.0 * 448.0))
        bmax = base.reshape(N, K // BLOCK, BLOCK).abs().amax(dim=2)
        scales = (bmax / 6.0 / gs).to(torch.float8_e4m3fn).float() * gs          # pre-expanded to fp32
        packed = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
        mats.append((packed, scales, N, K))
    return mats


def cpu_time_layers(n_layers, reps):
    """Reference CPU path (dequantise every call + F.linear, fp32) over `n_layers` layers."""
    from oracle import cpu_baseline
    torch.set_num_threads(os.cpu_count() or 1)
    layers = [_cpu_layer(1000 + i) for i in range(n_layers)]
    xs = {K: torch.randn(1, K) for K in (HIDDEN, INTER)}
    times = []
    for r in range(reps):
        t0 = time.perf_counter()
        for mats in layers:
            for (p, s, N, K) in mats:
                cpu_baseline.nvfp4_forward_dequant_gemm(xs[K], p, s, BLOCK)
        times.append(time.perf_counter() - t0)
    return times


def cpu_baseline_sample():
    """~10-20 s of the reference CPU path on the host cores of this box: all 18 layers (the 54
    matrices of one step) per repetition."""
    n_layers = LAYERS
    cpu_time_layers(n_layers, 1)
    times = cpu_time_layers(n_layers, 8)
    t = float(np.median(times))
    bytes_ = n_layers * sum(algorithmic_bytes(n, k) for n, k in SHAPES)
    return {"value": bytes_ / t / 1e9, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
            "sample": f"{n_layers} of 18 layers ({3 * n_layers} matrices = one full step), median of 8 repetitions; torch CPU restatement of "
                      "NVFP4PackedLinear._forward_dequant_gemm (dequantise per call + F.linear, fp32), "
                      f"torch threads = {torch.get_num_threads()}",
            "seconds_per_sample": t}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_layers = LAYERS                 # the same 54 matrices per step as the GPU arm
    bytes_ = n_layers * sum(algorithmic_bytes(n, k) for n, k in SHAPES)
    cpu_time_layers(n_layers, max(1, min(args.warmup, 3)))
    steps = args.steps
    budget_s = 150.0
    times = []
    t_start = time.perf_counter()
    for i in range(steps):
        times += cpu_time_layers(n_layers, 1)
        if time.perf_counter() - t_start > budget_s:
            break
    done = len(times)
    total = float(sum(times))
    value = bytes_ * done / total / 1e9
    cpu = {"value": value, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
           "sample": f"each step = all {n_layers} layers (54 matrices) of the same workload, as many of the requested steps "
                     f"as fit {budget_s:.0f} s; torch CPU restatement of NVFP4PackedLinear._forward_dequant_gemm "
                     "(dequantise per call + F.linear, fp32), all host threads"}
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": int(args.gpus),
            "steps": done, "steps_requested": steps, "warmup": args.warmup, "ms_per_step": total / done * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "NVFP4 weight-only GEMV, M=1, Gemma-300M action-expert MLP, 18 layers x "
                                   "(gate,up 1024->4096; down 4096->1024) = 54 matrices per step, E4M3 block-16 "
                                   "scales + fp32 global scale", "parallelism": "host CPU, rank 0 only"},
            "cpu_baseline": cpu,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="tc", choices=["cuda", "tc"],
                    help="GEMV kernel: CUDA-core decode (cuda) or tensor-core (tc)")
    ap.add_argument("--no-graph", action="store_true", help="launch the step's kernels directly instead of one CUDA graph")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-configuration side measurements")
    ap.add_argument("--no-fuse", action="store_true",
                    help="--path tc: stand-alone activation quantiser launch + GEMV instead of the fused launch")
    ap.add_argument("--no-pdl", action="store_true",
                    help="--path tc: no programmatic dependent launch between quantiser and GEMV")
    ap.add_argument("--no-serving", action="store_true", help="skip the request-serving measurement (builds a full model)")
    ap.add_argument("--case", default=None, choices=["gemm", "gemm-nvfp4", "rowop", "attention", "pi05", "int4-gemm", "int4-gemv", "int4-gemv-rowmajor", "quantize"],
                    help="run one bounded kernel case (for ncu) instead of the benchmark")
    ap.add_argument("--M", type=int, default=712)
    ap.add_argument("--N", type=int, default=32768)
    ap.add_argument("--K", type=int, default=2048)
    ap.add_argument("--pieces", type=int, default=3)
    ap.add_argument("--rowmajor", action="store_true",
                    help="--case gemm: the row-major operand form (128 x 128 tiles) instead of the tiled images")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--denoise-steps", type=int, default=1)
    ap.add_argument("--no-clock-warmup", action="store_true",
                    help="do exactly W warm-up steps (profiling runs); by default warm-up lasts >= 0.4 s")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
        if args.case is not None:
            run_case(args)
        else:
            run_ours(args)


if __name__ == "__main__":
    main()
