#!/usr/bin/env python
"""Benchmark of the quantized GEMM micro-kernel path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c3|c4|c5]

Prints ONE JSON line.  Headline workload ("c3"): the W4A8 prefill GEMM of the Llama-3-8B MLP
up-projection shape (M=2048, K=4096, N=14336; bf16 activations dynamically quantised per row to
int8, per-channel int4 weights, bf16 output), metric int8 TOPS = 2*M*N*K / step time.  One step =
quantise+pack the activations, then run_gemm, through the C ABI.  The same line carries the decode
GEMV (M=1, K=N=4096, f32) as HBM GB/s under "decode_gemv".

Inputs are seeded synthetic data with the shapes and value distributions the configurations state
(there are no datasets or checkpoints involved).

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) the weight matrix is split
along N across the ranks (column-parallel, total work fixed: "strong" scaling); activations are
replicated; no collective is on the data path.  --gather additionally times an NCCL all-gather
of the output column shards and the fused form (peer stores from the GEMM epilogue), reported
separately under "gather", not part of "value".

--impl reference times the CPU implementation of the same path on the host cores (the oracle port
built from oracle/tqt_oracle.c; the reference's W4A8 code lives in a gtest translation unit that
cannot be compiled off RISC-V), on a bounded sample of rows.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (M, K, N, description)
    "c3": (2048, 4096, 14336, "gemm_1xnbias_clamp_bf16_qai8dxp_qsi4cxp prefill M=2048 K=4096 N=14336 (Llama-3-8B MLP up-proj)"),
    "c4": (4096, 4096, 4096, "gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp M=K=N=4096 (static W8A8, int8 out)"),
    "c5": (8192, 8192, 28672, "gemm_1xnbias_clamp_f16_f16p_qsi4c2p M=8192 K=8192 N=28672 bl=32 (Llama-3-70B MLP)"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    PERIOD_MS = 50

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.PERIOD_MS)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------
# CPU arm
# ---------------------------------------------------------------------------------------------------
def cpu_w4a8_sample(M, K, N, budget_s=12.0, threads=None):
    """Times the oracle's W4A8 GEMM on the host cores for `rows` rows of the workload (all of N and K)
    chosen so that the run takes roughly budget_s.  Returns (tops, rows, seconds, threads)."""
    from oracle.tqo import TD_BF16, Oracle
    orc = Oracle(native=True)
    nthreads = threads or orc.max_threads()
    orc.set_threads(nthreads)
    rng = np.random.default_rng(1)
    nib = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    sb = rng.uniform(0.001, 0.01, N).astype(np.float32)

    def run(rows):
        q = rng.integers(-128, 128, (rows, K), dtype=np.int8)
        sa = rng.uniform(0.01, 0.05, rows).astype(np.float32)
        zp = rng.integers(-20, 20, rows).astype(np.int32)
        t0 = time.perf_counter()
        orc.gemm_w4a8(q, nib, sa, zp, sb, TD_BF16, None, None, (-65504.0, 65504.0))
        return time.perf_counter() - t0

    probe_rows = max(nthreads, 16)
    t_probe = run(probe_rows)
    rows = int(min(M, max(probe_rows, probe_rows * budget_s / max(t_probe, 1e-6))))
    rows = max(nthreads, rows - rows % nthreads)
    t = run(rows)
    return 2.0 * rows * N * K / t / 1e12, rows, t, nthreads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M, K, N, desc = CONFIGS["c3"]
    per_step = []
    rows = 0
    nthreads = 0
    budget = max(0.5, min(8.0, 150.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        tops, rows, secs, nthreads = cpu_w4a8_sample(M, K, N, budget_s=budget if i >= args.warmup else 2.0)
        if i >= args.warmup:
            per_step.append((tops, secs))
    tops = float(np.mean([p[0] for p in per_step]))
    ms = float(np.mean([p[1] for p in per_step]) * 1e3)
    sample = f"{rows} of {M} rows x all N={N} x K={K} per step (int8 x int4 -> f32 epilogue -> bf16), {nthreads} OpenMP threads"
    line = {
        "impl": "reference", "metric": "w4a8_gemm_int8_tops", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": CONFIGS["c3"][3], "sample": sample},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": nthreads, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load, load_linear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        if args.gather:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only: no multicast binding
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    torch.cuda.set_device(local_rank)
    dev = torch.device(f"cuda:{local_rank}")
    pkg = load()
    lin = load_linear()
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cfg = args.config
    M, K, N, desc = CONFIGS[cfg]
    n_begin, n_local = pkg.shard_plan_n(N, world, rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)

    # ---- build R rotating weight sets for this rank's column shard -------------------------------
    R = args.rotate
    layers = []
    if cfg == "c3":
        for r in range(R):
            # int4 weights of W ~ N(0, 0.02) quantised per channel: nibble = clamp(round(w / (absmax/8)), -8, 7) + 8
            w = torch.randn((n_local, K), generator=gen, device=dev) * 0.02
            s = w.abs().amax(dim=1) / 8.0
            q = torch.clamp(torch.round(w / s[:, None]), -8, 7).to(torch.int16) + 8
            nib = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8)
            layers.append(lin.W4A8Linear(nib, s, K, "bf16", bias=torch.zeros(n_local, dtype=torch.bfloat16, device=dev)))
            del w, q, nib
        a_host = torch.randn((M, K), dtype=torch.float32).to(torch.bfloat16).pin_memory()
        a_dev = a_host.to(dev)
        in_bytes = M * K * 2
        out_bytes = M * n_local * 2

        def step_device(i):
            L = layers[i % R]
            L.quantize(a_dev)
            return L.gemm(M)

        def gemm_only(i):
            return layers[i % R].gemm(M)
        launches_per_step = 2
        dtype = "int8"
    elif cfg == "c4":
        for r in range(R):
            w = torch.randint(-127, 128, (n_local, K), generator=gen, device=dev, dtype=torch.int8)
            sb = torch.rand(n_local, generator=gen, device=dev) * 0.009 + 0.001
            bias = torch.randint(-1000, 1001, (n_local,), generator=gen, device=dev, dtype=torch.int32)
            fused = bias - 3 * w.to(torch.int32).sum(dim=1, dtype=torch.int32)
            layers.append(lin.W8A8RequantLinear(w, sb, 0.05, 3, 0.1, -5, fused))
            del w
        a_host = torch.randint(-128, 128, (M, K), dtype=torch.int8).pin_memory()
        a_dev = a_host.to(dev)
        in_bytes = M * K
        out_bytes = M * n_local

        def step_device(i):
            L = layers[i % R]
            L.pack(a_dev)
            return L.gemm(M)

        def gemm_only(i):
            return layers[i % R].gemm(M)
        launches_per_step = 2
        dtype = "int8"
    else:  # c5
        bl = 32
        for r in range(R):
            nib = torch.randint(0, 256, (n_local, K // 2), generator=gen, device=dev, dtype=torch.uint8)
            sc = (torch.rand((n_local, K // bl), generator=gen, device=dev) * 0.005 + 0.001).to(torch.float16)
            bias = (torch.randn(n_local, generator=gen, device=dev) * 0.1).to(torch.float16)
            layers.append(lin.W4A16Linear(nib, sc, K, bl, "f16", bias=bias))
            del nib
        a_host = torch.randn((M, K), dtype=torch.float32).to(torch.float16).pin_memory()
        a_dev = a_host.to(dev)
        in_bytes = M * K * 2
        out_bytes = M * n_local * 2

        def step_device(i):
            L = layers[i % R]
            L.pack(a_dev)
            return L.gemm(M)

        def gemm_only(i):
            return layers[i % R].gemm(M)
        launches_per_step = 2
        dtype = "f16"

    # The step's two launches replayed as one CUDA graph per weight set: the host then needs ~10 us per step
    # instead of ~100 us of Python argument marshalling, which otherwise bounds the column shards on 2-8 GPUs.
    eager_step, eager_gemm = step_device, gemm_only
    if not args.no_graphs:
        step_graphs = [L.captured(a_dev) for L in layers]
        gemm_graphs = [L.captured(a_dev, gemm_only=True) for L in layers]

        def step_device(i):   # noqa: F811
            return step_graphs[i % R]()

        def gemm_only(i):   # noqa: F811
            return gemm_graphs[i % R]()

    ops = 2.0 * M * N * K               # whole job (all ranks)
    ops_local = 2.0 * M * n_local * K
    unit = "TOPS" if cfg != "c5" else "TFLOP/s"

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_step = timed(step_device, args.steps, args.warmup)
    ms_gemm = timed(gemm_only, args.steps, args.warmup)
    # the timed region lasts milliseconds; keep the same step loop running for about a second and a half so that
    # the clock samples (and the sustained figure) describe the kernels under load, power cap included
    sustain_steps = int(min(20000, max(args.steps, math.ceil(args.sustain_s * 1e3 / ms_step)))) if args.sustain_s > 0 else 0
    ms_sustained = timed(step_device, sustain_steps, 0) if sustain_steps else None
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["note"] = (f"sampled every {ClockSampler.PERIOD_MS} ms from the start of the timed region to the end of a "
                          f"{sustain_steps}-step continuation of the same step loop")

    # ---- end to end: pinned host activations in, result back to the host, every step --------------
    out_host = torch.empty((M, n_local), dtype=layers[0].workspace(M)["out"].dtype).pin_memory()

    def step_e2e(i):
        layers[i % R].forward_host(a_host, out_host)
    # PCIe-bound and therefore sensitive to what else the host is doing: five batches, the median batch is reported
    e2e_steps = max(3, min(args.steps, 10))
    timed(step_e2e, 1, 3)
    e2e_batches = sorted(timed(step_e2e, e2e_steps, 0) for _ in range(5))
    ms_e2e = e2e_batches[len(e2e_batches) // 2]

    # ---- optional: the full output on every GPU -------------------------------------------------------
    # (a) the step followed by an NCCL all-gather of the column shards; (b) the fused form: the GEMM's epilogue
    # stores every tile into the peer-mapped output buffers of all ranks (tqt_cuda_set_output_replicas), no collective.
    gather = None
    if world > 1 and args.gather and cfg in ("c3", "c5"):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only: no multicast binding
        import torch.distributed._symmetric_memory as symm
        out_local = layers[0].workspace(M)["out"]
        staged = torch.empty((world * M, n_local), dtype=out_local.dtype, device=dev)
        full = symm.empty((M, N), dtype=out_local.dtype, device=dev)
        hdl = symm.rendezvous(full, dist.group.WORLD.group_name)
        peers = [int(hdl.buffer_ptrs[r]) for r in range(world) if r != rank]
        g_steps, g_warm = max(3, min(args.steps, 50)), 3

        def step_nccl(i):
            out = step_device(i)
            dist.all_gather_into_tensor(staged, out)

        def step_fused(i):
            L = layers[i % R]
            (L.quantize if cfg == "c3" else L.pack)(a_dev)
            pkg.set_output_replicas(full.data_ptr(), peers)
            try:
                L.gemm(M, out=full[:, n_begin:n_begin + n_local])
            finally:
                pkg.set_output_replicas(0, [])

        if not args.no_graphs:   # the fused step replayed as a graph too (the replica offsets are kernel arguments)
            eager_fused, fused_graphs = step_fused, []
            for li in range(R):
                eager_fused(li)
                torch.cuda.current_stream().synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    eager_fused(li)
                fused_graphs.append(gr)

            def step_fused(i):   # noqa: F811
                fused_graphs[i % R].replay()

        ms_nccl = timed(step_nccl, g_steps, g_warm)
        ms_fused = timed(step_fused, g_steps, g_warm)
        # the two forms must agree: run step 0 both ways and compare every rank's copy of the full output
        full.zero_()
        barrier()
        step_fused(0)
        barrier()
        step_nccl(0)
        barrier()
        same = all(torch.equal(full[:, r * n_local:(r + 1) * n_local], staged[r * M:(r + 1) * M]) for r in range(world))
        flag = torch.tensor([1 if same else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        gather = {"nccl_step_ms": ms_nccl, "fused_step_ms": ms_fused, "outputs_equal_on_all_ranks": bool(flag.item()),
                  "bytes_per_rank": M * n_local * out_local.element_size(),
                  "note": "nccl: step + all_gather_into_tensor of the column shards; fused: the GEMM epilogue stores "
                          "each tile into every rank's output buffer (peer stores over NVLink), no collective"}

    fault = pkg.read_device_fault()

    # ---- decode GEMV (M=1, K=N=4096, f32), captured in a CUDA graph over rotating weights ----------
    decode = None
    if cfg == "c3" and rank == 0 and not args.no_decode:
        decode = bench_decode(torch, lin, pkg, dev, peaks)
        decode["other_shapes"] = []
        for (K2, N2, c2) in ((4096, 14336, 16), (8192, 28672, 6)):   # the prefill configs' weight shapes at M=1
            d2 = bench_decode(torch, lin, pkg, dev, peaks, K=K2, N=N2, copies=c2)
            decode["other_shapes"].append({"workload": d2["workload"], "gbs": d2["value"], "us_per_gemv": d2["us_per_gemv"],
                                           "frac": d2["roofline"]["frac"], "read_ceiling_gbs": d2["read_ceiling"]["gbs"]})

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- CPU baseline on a bounded sample (rank 0, N=1 only) -------------------------------------------
    cpu = None
    if world == 1 and not args.no_cpu and cfg == "c3":
        tops, rows, secs, nthreads = cpu_w4a8_sample(M, K, N, budget_s=12.0)
        cpu = {"value": tops, "unit": "TOPS", "cores": nthreads, "kind": "port",
               "sample": f"{rows} of {M} rows x all N x K in {secs:.1f} s, oracle/tqt_oracle.c with {nthreads} OpenMP threads"}

    # dram__bytes_read.sum + dram__bytes_write.sum of one GEMM launch, from the ncu captures summarised under profiles/
    ncu_traffic = {"c3": 56.2e6, "c4": 33.9e6, "c5": 1419.1e6}[cfg] if world == 1 else None
    int8_peak = 2.0 * peaks["bf16_sustained"] if cfg != "c5" else peaks["bf16_sustained"]
    achieved = ops_local / (ms_gemm * 1e-3) / 1e12
    line = {
        "metric": "w4a8_gemm_int8_tops" if cfg == "c3" else ("w8a8_gemm_int8_tops" if cfg == "c4" else "w4a16_gemm_f16_tflops"),
        "value": ops / (ms_step * 1e-3) / 1e12, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype,
        "data": "synthetic",
        "config": {"workload": desc, "step": "activation quantise+pack (or pack) kernel + run_gemm, weights packed once outside" +
                           ("" if args.no_graphs else "; the two launches replayed as one CUDA graph"),
                   "parallelism": f"N-sharded x{world}, no collective" if world > 1 else "single GPU",
                   "n_per_gpu": n_local,
                   "l2": f"rotating {R} weight/output sets per rank ({R * (layers[0].b_packed.numel() + out_bytes) / 1e6:.0f} MB) > 126 MB L2"},
        "gemm_only_ms": ms_gemm,
        "sustained": None if ms_sustained is None else {"steps": sustain_steps, "ms_per_step": ms_sustained,
                                                        "value": ops / (ms_sustained * 1e-3) / 1e12, "unit": unit},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s",
                     "frac": achieved / int8_peak, "traffic": ncu_traffic,
                     "note": ("run_gemm kernel alone, per GPU; peak = 2 x bf16_tflops_sustained of " + peaks["source"] +
                              " (int8 tensor rate is twice the bf16 rate)") if cfg != "c5" else
                             "run_gemm kernel alone, per GPU; peak = bf16_tflops_sustained of " + peaks["source"]},
        "e2e": {"value": ops / (ms_e2e * 1e-3) / 1e12, "unit": unit, "h2d_bytes_per_step": in_bytes,
                "d2h_bytes_per_step": out_bytes, "ms_per_step": ms_e2e,
                "batches_ms": e2e_batches, "note": f"median of 5 batches of {e2e_steps} steps"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks, "device_fault": fault,
    }
    if gather is not None:
        line["gather"] = gather
    if cpu:
        line["cpu_baseline"] = cpu
    if decode:
        line["decode_gemv"] = decode
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _graph_time_us(torch, stream, launch_all, launches, reps):
    """Capture `launch_all` (which issues `launches` kernels) in a CUDA graph and return us per kernel."""
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        launch_all()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            launch_all()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * launches)


def bench_decode(torch, lin, pkg, dev, peaks, K=4096, N=4096, copies=48, reps=20):
    """GEMV M=1 f32: one CUDA graph replays `copies` GEMVs over distinct weight sets (together larger
    than L2), so every launch streams its weights from HBM.  `read_ceiling` is a kernel with the same
    launch shape that only reads the same number of bytes from the same buffers, timed the same way."""
    import ctypes
    nbytes = N * K // 2 + 3 * 4 * N + K + 8   # weights + scale_b, bias, D + int8 row + (scale, zp)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    layers = []
    for _ in range(copies):
        nib = torch.randint(0, 256, (N, K // 2), generator=gen, device=dev, dtype=torch.uint8)
        sb = torch.rand(N, generator=gen, device=dev) * 0.01
        layers.append(lin.W4A8Linear(nib, sb, K, "f32", bias=torch.randn(N, generator=gen, device=dev) * 0.1))
    a = torch.randn((1, K), generator=gen, device=dev)
    for L in layers:
        L.quantize(a)
        L.gemm(1)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()

    def gemvs():
        for L in layers:
            L.gemm(1)

    us = _graph_time_us(torch, stream, gemvs, copies, reps)
    lib = pkg.lib()
    lib.tqt_cuda_debug_stream_read.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    lib.tqt_cuda_debug_stream_read.restype = None
    rd = nbytes // 16 * 16

    def reads():
        pkg.set_stream(torch.cuda.current_stream().cuda_stream)
        for L in layers:
            lib.tqt_cuda_debug_stream_read(L.b_packed.data_ptr(), rd, None)

    us_read = _graph_time_us(torch, stream, reads, copies, reps)
    pkg.set_stream(torch.cuda.current_stream().cuda_stream)
    gbs = nbytes / (us * 1e-6) / 1e9
    return {"metric": "w4a8_gemv_hbm_gbs", "value": gbs, "unit": "GB/s", "us_per_gemv": us,
            "workload": f"gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp decode M=1 K={K} N={N}",
            "bytes_per_gemv": nbytes, "gpu_launches": reps * copies,
            "read_ceiling": {"gbs": rd / (us_read * 1e-6) / 1e9, "us": us_read,
                             "note": "a kernel with the GEMV's launch shape that only reads the same bytes, same graph"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm"], "traffic": 8.698e6 if (K, N) == (4096, 4096) else None,
                         "note": f"CUDA-graph replay of {copies} back-to-back GEMVs over distinct weights; peak = hbm_gbs of {peaks['source']}"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    ap.add_argument("--rotate", type=int, default=4, help="distinct weight/output sets cycled through (defeats L2 reuse)")
    ap.add_argument("--gather", action="store_true", help="N > 1: also time the step with the full output gathered on every GPU (NCCL, and fused peer stores)")
    ap.add_argument("--sustain-s", type=float, default=1.5, help="seconds of continued step loop for clock sampling (0 = off)")
    ap.add_argument("--no-graphs", action="store_true", help="issue the step's launches from Python instead of replaying CUDA graphs")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
