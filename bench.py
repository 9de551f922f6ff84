#!/usr/bin/env python
"""Benchmark of the quantized GEMM micro-kernel path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c3|c4|c5]

Prints ONE JSON line.  Headline workload ("c3"): the W4A8 prefill GEMM of the Llama-3-8B MLP
up-projection shape (M=2048, K=4096, N=14336; bf16 activations dynamically quantised per row to
int8, per-channel int4 weights, bf16 output), metric int8 TOPS = 2*M*N*K / step time.  One step =
quantise+pack the activations, then run_gemm, through the C ABI.  On one GPU the same line carries
the other two prefill configurations under "c4" (static W8A8 with int8 requantisation) and "c5"
(W4A16 block-quant), measured the same way with fewer steps, the decode GEMV (M=1, K=N=4096, f32) as
HBM GB/s under "decode_gemv" (with an M=16 row), and the layout kernels' HBM fractions under "layout".

Inputs are seeded synthetic data with the shapes and value distributions the configurations state
(there are no datasets or checkpoints involved).

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) the weight matrix is split
along N across the ranks (column-parallel, total work fixed: "strong" scaling); activations are
replicated; no collective is on the data path.  --gather additionally times an NCCL all-gather
of the output column shards and the fused form (peer stores from the GEMM epilogue), reported
separately under "gather", not part of "value".

--impl reference times the CPU implementation of the same path on the host cores, on a bounded sample
of rows: the reference's own w4a8_reference_fp32 (test/gemm/test_gemm_i8_i4_rvv.cpp:122-156, compiled
into oracle/_ref by oracle/Makefile; single-threaded code, run here on disjoint row slices from one
thread per core) when that library is present, else the oracle port built from oracle/tqt_oracle.c.
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
    """Times the CPU W4A8 GEMM on the host cores for `rows` rows of the workload (all of N and K) chosen
    so that the run takes roughly budget_s.  Returns (tops, rows, seconds, threads, kind): kind
    "reference" = the reference's own w4a8_reference_fp32 from oracle/_ref, one thread per core on
    disjoint row slices (the function itself is single-threaded); "port" = the oracle restatement with
    OpenMP."""
    from concurrent.futures import ThreadPoolExecutor

    from oracle.tqo import TD_BF16, Oracle, Reference
    orc = Oracle(native=True)
    nthreads = threads or orc.max_threads()
    orc.set_threads(nthreads)
    ref = Reference(native=True)
    kind = "reference" if ref.has_w4a8() else "port"
    rng = np.random.default_rng(1)
    nib = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    sb = rng.uniform(0.001, 0.01, N).astype(np.float32)
    pool = ThreadPoolExecutor(nthreads) if kind == "reference" else None

    def run(rows):
        q = rng.integers(-128, 128, (rows, K), dtype=np.int8)
        sa = rng.uniform(0.01, 0.05, rows).astype(np.float32)
        zp = rng.integers(-20, 20, rows).astype(np.int32)
        t0 = time.perf_counter()
        if kind == "reference":
            per = -(-rows // nthreads)
            parts = [(r0, min(rows, r0 + per)) for r0 in range(0, rows, per)]
            list(pool.map(lambda b: ref.w4a8_gemm(q[b[0]:b[1]], nib, sa[b[0]:b[1]], zp[b[0]:b[1]], sb, TD_BF16, None, None,
                                                  (-65504.0, 65504.0)), parts))
        else:
            orc.gemm_w4a8(q, nib, sa, zp, sb, TD_BF16, None, None, (-65504.0, 65504.0))
        return time.perf_counter() - t0

    probe_rows = max(nthreads, 16)
    t_probe = run(probe_rows)
    rows = int(min(M, max(probe_rows, probe_rows * budget_s / max(t_probe, 1e-6))))
    rows = max(nthreads, rows - rows % nthreads)
    t = run(rows)
    if pool is not None:
        pool.shutdown()
    return 2.0 * rows * N * K / t / 1e12, rows, t, nthreads, kind


def cpu_sample_text(rows, M, N, K, nthreads, kind, secs=None):
    what = ("the reference's w4a8_reference_fp32 (oracle/_ref), one thread per core on disjoint row slices" if kind == "reference"
            else "oracle/tqt_oracle.c with OpenMP")
    t = "" if secs is None else f" in {secs:.1f} s"
    return f"{rows} of {M} rows x all N={N} x K={K}{t} (int8 x int4 -> f32 epilogue -> bf16), {what}, {nthreads} threads"


def workload_config(cfg, world, n_local, R, set_bytes, graphs=True):
    """The `config` object of the JSON line; both arms (ours, reference) print the same one."""
    return {"workload": CONFIGS[cfg][3],
            "step": "activation quantise+pack (or pack) kernel + run_gemm, weights packed once outside" +
                    ("; launches replayed as CUDA graphs of several consecutive steps" if graphs else ""),
            "parallelism": f"N-sharded x{world}, no collective" if world > 1 else "single GPU",
            "n_per_gpu": n_local,
            "l2": f"rotating {R} weight/output sets per rank ({R * set_bytes / 1e6:.0f} MB) > 126 MB L2"}


def set_bytes_of(cfg, n_local):
    """Bytes of one rotating set on a rank: packed weights + output (what has to exceed L2 R times over)."""
    M, K, N, _ = CONFIGS[cfg]
    if cfg == "c3":
        return -(-n_local // 128) * (K // 128) * 8448 + M * n_local * 2
    if cfg == "c4":
        return n_local * K + M * n_local
    return n_local * K // 2 + M * n_local * 2


def rotation(cfg, n_local, requested):
    """Number of rotating weight/output sets: at least the requested count, and enough that together they are
    well above the 126 MB L2 at every shard size."""
    need = int(math.ceil(1.5 * 126e6 / set_bytes_of(cfg, n_local)))
    return max(requested, need)


def shard_plan(n, world, rank):
    """Same split as tqt_shard_plan_n (contiguous ranges of 128-column blocks), for the arm that does not load the library."""
    blocks = -(-n // 128)
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    nb = base + (1 if rank < extra else 0)
    return min(b0 * 128, n), min((b0 + nb) * 128, n) - min(b0 * 128, n)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    M, K, N, desc = CONFIGS["c3"]
    per_step = []
    rows = 0
    nthreads = 0
    kind = "port"
    budget = max(0.5, min(8.0, 150.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        tops, rows, secs, nthreads, kind = cpu_w4a8_sample(M, K, N, budget_s=budget if i >= args.warmup else 2.0)
        if i >= args.warmup:
            per_step.append((tops, secs))
    tops = float(np.mean([p[0] for p in per_step]))
    ms = float(np.mean([p[1] for p in per_step]) * 1e3)
    sample = cpu_sample_text(rows, M, N, K, nthreads, kind) + " per step"
    _, n_local = shard_plan(N, world, 0)
    R = rotation("c3", n_local, args.rotate)
    line = {
        "impl": "reference", "metric": "w4a8_gemm_int8_tops", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config("c3", world, n_local, R, set_bytes_of("c3", n_local), graphs=not args.no_graphs),
        "note": "CPU arm: the config names the workload of both arms; this arm runs its rows on the host cores, no GPU, no graphs",
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": nthreads, "kind": kind, "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
# Rate at which tcgen05.mma actually issues on this part (measured with a loop of MMAs on static operands:
# kind::i8 M128 x N192 x K32 every 102.5 cycles per SM, 148 SMs, 1965 MHz); kind::f16 runs at half of it.
ISSUE_RATE_INT8_TOPS = 2.0 * 128 * 192 * 32 / 102.5 * 148 * 1.965e9 / 1e12   # 4.46e3
# dram__bytes_read.sum + dram__bytes_write.sum of ONE run_gemm launch from the ncu captures summarised under
# profiles/ (file named beside each figure): taken under ncu on an earlier run of the same kernels, NOT measured by
# the run that prints the line.
NCU_TRAFFIC = {"c3": (55.7e6, "profiles/gemm_ts_pair_w4a8_c3.txt"), "c4": (33.7e6, "profiles/gemm_pair_i8_c4.txt"),
               "c5": (1438.5e6, "profiles/gemm_ts_pair_w4a16_c5.txt")}


def algorithmic_bytes(cfg, n_local):
    """Bytes one run_gemm launch must move: packed A + packed B (+ scales, bias) in, D out."""
    M, K, N, _ = CONFIGS[cfg]
    if cfg == "c3":
        return M * K + -(-n_local // 128) * (K // 128) * 8448 + 8 * M + 4 * n_local + 2 * n_local + 2 * M * n_local
    if cfg == "c4":
        return M * K + n_local * K + 4 * n_local + 4 * n_local + M * n_local
    return 2 * M * K + n_local * K // 2 + 2 * n_local * (K // 32) + 2 * n_local + 2 * M * n_local


def build_layers(torch, lin, cfg, n_local, R, dev, gen):
    """R rotating weight sets of this rank's column shard + the activations; returns the pieces of one step."""
    M, K, N, _ = CONFIGS[cfg]
    layers = []
    if cfg == "c3":
        for r in range(R):
            # int4 weights of W ~ N(0, 0.02) quantised per channel: nibble = clamp(round(w / (absmax/8)), -8, 7) + 8
            w = torch.randn((n_local, K), generator=gen, device=dev) * 0.02
            sc = w.abs().amax(dim=1) / 8.0
            q = torch.clamp(torch.round(w / sc[:, None]), -8, 7).to(torch.int16) + 8
            nib = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8)
            layers.append(lin.W4A8Linear(nib, sc, K, "bf16", bias=torch.zeros(n_local, dtype=torch.bfloat16, device=dev),
                                         clamp=(-65504.0, 65504.0)))
            del w, q, nib
        a_host = torch.randn((M, K), dtype=torch.float32).to(torch.bfloat16).pin_memory()
        prepare, in_bytes, out_bytes, dtype = "quantize", M * K * 2, M * n_local * 2, "int8"
    elif cfg == "c4":
        for r in range(R):
            w = torch.randint(-127, 128, (n_local, K), generator=gen, device=dev, dtype=torch.int8)
            sb = torch.rand(n_local, generator=gen, device=dev) * 0.009 + 0.001
            bias = torch.randint(-1000, 1001, (n_local,), generator=gen, device=dev, dtype=torch.int32)
            fused = bias - 3 * w.to(torch.int32).sum(dim=1, dtype=torch.int32)
            layers.append(lin.W8A8RequantLinear(w, sb, 0.05, 3, 0.1, -5, fused))
            del w
        a_host = torch.randint(-128, 128, (M, K), dtype=torch.int8).pin_memory()
        prepare, in_bytes, out_bytes, dtype = "pack", M * K, M * n_local, "int8"
    else:  # c5
        bl = 32
        for r in range(R):
            nib = torch.randint(0, 256, (n_local, K // 2), generator=gen, device=dev, dtype=torch.uint8)
            sc = (torch.rand((n_local, K // bl), generator=gen, device=dev) * 0.005 + 0.001).to(torch.float16)
            bias = (torch.randn(n_local, generator=gen, device=dev) * 0.1).to(torch.float16)
            layers.append(lin.W4A16Linear(nib, sc, K, bl, "f16", bias=bias))
            del nib
        a_host = torch.randn((M, K), dtype=torch.float32).to(torch.float16).pin_memory()
        prepare, in_bytes, out_bytes, dtype = "pack", M * K * 2, M * n_local * 2, "f16"
    return layers, a_host, prepare, in_bytes, out_bytes, dtype


def roofline_of(cfg, peaks, ops_local, ms_gemm, ms_sustained_step, n_local, world):
    """Tensor roofline of the run_gemm kernel: the burst loop (milliseconds) against the burst peak, the sustained
    step loop (seconds, power cap included) against the sustained peak, and against the MMA issue rate."""
    mult = 2.0 if cfg != "c5" else 1.0      # the int8 tensor rate is twice the bf16 rate (the file has no int8 figure)
    peak_burst, peak_sust = mult * peaks["bf16"], mult * peaks["bf16_sustained"]
    achieved = ops_local / (ms_gemm * 1e-3) / 1e12
    issue = ISSUE_RATE_INT8_TOPS * (1.0 if cfg != "c5" else 0.5)
    r = {"bound": "tensor", "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s", "frac": achieved / peak_burst,
         "frac_of_issue_rate": achieved / issue, "issue_rate": issue,
         "algorithmic_bytes": algorithmic_bytes(cfg, n_local),
         "traffic": NCU_TRAFFIC[cfg][0] if world == 1 else None,
         "traffic_source": (f"ncu capture of an earlier run summarised in {NCU_TRAFFIC[cfg][1]} (one launch, dram read + write); "
                            "not measured by this run") if world == 1 else None,
         "note": (f"run_gemm kernel alone (a loop of milliseconds), per GPU; peak = {mult:g} x bf16_tflops (burst) of {peaks['source']}"
                  + ("; the int8 tensor rate is twice the bf16 rate" if cfg != "c5" else "")
                  + "; frac_of_issue_rate = achieved / the rate tcgen05.mma issues at (what ncu's tensor-pipe counter shows)")}
    if ms_sustained_step:
        a_s = ops_local / (ms_sustained_step * 1e-3) / 1e12
        r["sustained"] = {"achieved": a_s, "peak": peak_sust, "frac": a_s / peak_sust,
                          "note": f"whole step (prepare + run_gemm) continued for seconds; peak = {mult:g} x bf16_tflops_sustained of {peaks['source']}"}
    return r


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

    def timed(fn, steps, warmup, block=None):
        """Time exactly `steps` steps.  block = (U, graph): the timed steps are issued as steps / U replays of one CUDA graph
        that holds U consecutive steps (the sets rotate inside it), so that the host's launch cost per step does not bound
        steps of a few tens of microseconds (column shards on 4-8 GPUs); the warm-up steps are single-step launches."""
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if block is None:
            for i in range(steps):
                fn(warmup + i)
        else:
            U, graph = block
            assert steps % U == 0
            for _ in range(steps // U):
                graph.replay()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    def block_size(steps, R):
        """Steps per block graph: the smallest divisor of `steps` that holds every rotating set and at least 8 steps."""
        want = max(R, 8)
        for u in range(want, steps + 1):
            if steps % u == 0:
                return u
        return steps

    def measure(cfg, steps, warmup, sustain_s, with_e2e, with_gather):
        """One prefill configuration on this rank's column shard: device-timed step, run_gemm alone, sustained loop
        with clock samples, optionally the host-to-host step and the gathered-output variants."""
        M, K, N, desc = CONFIGS[cfg]
        n_begin, n_local = pkg.shard_plan_n(N, world, rank)
        R = rotation(cfg, n_local, args.rotate)
        gen = torch.Generator(device=dev)
        gen.manual_seed(1234 + rank)
        layers, a_host, prepare, in_bytes, out_bytes, dtype = build_layers(torch, lin, cfg, n_local, R, dev, gen)
        a_dev = a_host.to(dev)

        def step_device(i):
            L = layers[i % R]
            getattr(L, prepare)(a_dev)
            return L.gemm(M)

        def gemm_only(i):
            return layers[i % R].gemm(M)

        # The step's two launches replayed as one CUDA graph per weight set: the host then needs ~10 us per step
        # instead of ~100 us of Python argument marshalling, which otherwise bounds the column shards on 2-8 GPUs.
        eager_step = step_device
        if not args.no_graphs:
            step_graphs = [L.captured(a_dev) for L in layers]
            gemm_graphs = [L.captured(a_dev, gemm_only=True) for L in layers]

            def step_device(i):   # noqa: F811
                return step_graphs[i % R]()

            def gemm_only(i):   # noqa: F811
                return gemm_graphs[i % R]()

            U = block_size(steps, R)

            def block_graph(eager):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for j in range(U):
                        eager(j)
                return g

            step_block = (U, block_graph(lambda j: layers[j % R].step(a_dev)))
            gemm_block = (U, block_graph(lambda j: layers[j % R].gemm(M)))
        else:
            U, step_block, gemm_block = 1, None, None

        ops = 2.0 * M * N * K               # whole job (all ranks)
        ops_local = 2.0 * M * n_local * K
        unit = "TOPS" if cfg != "c5" else "TFLOP/s"
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        ms_step = timed(step_device, steps, warmup, step_block)
        ms_gemm = timed(gemm_only, steps, warmup, gemm_block)
        # the timed region lasts milliseconds; keep the same step loop running for a second or so, so that the clock
        # samples (and the sustained figure) describe the kernels under load, power cap included
        sustain_steps = int(min(20000, max(steps, math.ceil(sustain_s * 1e3 / ms_step)))) if sustain_s > 0 else 0
        sustain_steps = -(-sustain_steps // U) * U
        ms_sustained = timed(step_device, sustain_steps, 0, step_block) if sustain_steps else None
        clocks = sampler.stop() if rank == 0 else None
        if clocks is not None:
            clocks["note"] = (f"sampled every {ClockSampler.PERIOD_MS} ms from the start of the timed region to the end of a "
                              f"{sustain_steps}-step continuation of the same step loop")
        rec = {
            "metric": {"c3": "w4a8_gemm_int8_tops", "c4": "w8a8_gemm_int8_tops", "c5": "w4a16_gemm_f16_tflops"}[cfg],
            "value": ops / (ms_step * 1e-3) / 1e12, "unit": unit, "ms_per_step": ms_step, "dtype": dtype,
            "config": workload_config(cfg, world, n_local, R, set_bytes_of(cfg, n_local), graphs=not args.no_graphs),
            "gemm_only_ms": ms_gemm,
            "sustained": None if ms_sustained is None else {"steps": sustain_steps, "ms_per_step": ms_sustained,
                                                            "value": ops / (ms_sustained * 1e-3) / 1e12, "unit": unit},
            "roofline": roofline_of(cfg, peaks, ops_local, ms_gemm, ms_sustained, n_local, world),
            "gpu_launches": 2 * steps, "clocks": clocks,
        }

        if with_e2e:
            # ---- end to end: pinned host activations in, result back to the host, every step --------------
            out_host = torch.empty((M, n_local), dtype=layers[0].workspace(M)["out"].dtype).pin_memory()

            def step_e2e(i):
                layers[i % R].forward_host(a_host, out_host)
            # PCIe-bound and therefore sensitive to what else the host is doing: five batches, the median batch is reported
            e2e_steps = max(3, min(steps, 10))
            timed(step_e2e, 1, 3)
            e2e_batches = sorted(timed(step_e2e, e2e_steps, 0) for _ in range(5))
            ms_e2e = e2e_batches[len(e2e_batches) // 2]
            # the same bytes over the same three streams with no kernel in between: what PCIe alone allows
            floor = pcie_floor(torch, layers[0], a_host, out_host, timed, e2e_steps)
            rec["e2e"] = {"value": ops / (ms_e2e * 1e-3) / 1e12, "unit": unit, "h2d_bytes_per_step": in_bytes,
                          "d2h_bytes_per_step": out_bytes, "ms_per_step": ms_e2e, "batches_ms": e2e_batches,
                          "pcie_floor_ms": floor,
                          "note": f"median of 5 batches of {e2e_steps} steps; pcie_floor_ms = the step's host-to-device and "
                                  "device-to-host copies alone (same chunks, same streams, no kernels), median of 5 batches"}

        # ---- optional: the full output on every GPU -------------------------------------------------------
        # (a) the step followed by an NCCL all-gather of the column shards; (b) the fused form: the GEMM's epilogue
        # stores every tile into the peer-mapped output buffers of all ranks (tqt_cuda_set_output_replicas), no collective.
        if with_gather and world > 1 and cfg in ("c3", "c5"):
            import torch.distributed._symmetric_memory as symm
            out_local = layers[0].workspace(M)["out"]
            staged = torch.empty((world * M, n_local), dtype=out_local.dtype, device=dev)
            full = symm.empty((M, N), dtype=out_local.dtype, device=dev)
            hdl = symm.rendezvous(full, dist.group.WORLD.group_name)
            peers = [int(hdl.buffer_ptrs[r]) for r in range(world) if r != rank]
            done = torch.zeros(1, dtype=torch.int32, device=dev)
            g_steps, g_warm = max(3, min(steps, 50)), 3

            def step_nccl(i):
                out = step_device(i)
                dist.all_gather_into_tensor(staged, out)

            def fused_kernels(i):
                L = layers[i % R]
                getattr(L, prepare)(a_dev)
                with pkg.output_replicas(full.data_ptr(), full.numel() * full.element_size(), peers):
                    L.gemm(M, out=full[:, n_begin:n_begin + n_local])

            if not args.no_graphs:   # the fused step replayed as a graph too (the replica offsets are kernel arguments)
                eager_fused, fused_graphs = fused_kernels, []
                for li in range(R):
                    eager_fused(li)
                    torch.cuda.current_stream().synchronize()
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr):
                        eager_fused(li)
                    fused_graphs.append(gr)

                def fused_kernels(i):   # noqa: F811
                    fused_graphs[i % R].replay()

            def step_fused(i):
                # peers may read the full output only when every rank's kernel has completed: the cross-rank completion
                # signal (a one-int all-reduce) is part of the timed step, as the all-gather's own synchronisation is
                fused_kernels(i)
                dist.all_reduce(done)

            ms_nccl = timed(step_nccl, g_steps, g_warm)
            ms_fused = timed(step_fused, g_steps, g_warm)
            ms_fused_kernels = timed(fused_kernels, g_steps, g_warm)
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
            rec["gather"] = {"nccl_step_ms": ms_nccl, "fused_step_ms": ms_fused, "fused_kernels_only_ms": ms_fused_kernels,
                             "outputs_equal_on_all_ranks": bool(flag.item()),
                             "bytes_per_rank": M * n_local * out_local.element_size(),
                             "note": "nccl: step + all_gather_into_tensor of the column shards; fused: the GEMM epilogue stores "
                                     "each tile into every rank's output buffer (peer stores over NVLink) + a one-int all-reduce "
                                     "as the cross-rank completion signal; fused_kernels_only_ms leaves that signal out"}
        del layers
        torch.cuda.empty_cache()
        return rec

    cfg = args.config
    M, K, N, desc = CONFIGS[cfg]
    head = measure(cfg, args.steps, args.warmup, args.sustain_s, with_e2e=True, with_gather=args.gather)
    fault = pkg.read_device_fault()

    # ---- the other two prefill configurations, the decode GEMV and the layout kernels (one GPU, headline run) ---
    extra = {}
    if cfg == "c3" and world == 1 and not args.no_extra:
        for c in ("c4", "c5"):
            extra[c] = measure(c, max(3, min(args.steps, 20)), 3, min(args.sustain_s, 0.7), with_e2e=False, with_gather=False)
        extra["layout"] = bench_layout(torch, pkg, dev, peaks)
    decode = None
    if cfg == "c3" and rank == 0 and not args.no_decode:
        decode = bench_decode(torch, lin, pkg, dev, peaks)
        d16 = bench_decode(torch, lin, pkg, dev, peaks, M=16)
        decode["m16"] = {k: d16[k] for k in ("workload", "value", "unit", "us_per_gemv", "bytes_per_gemv", "read_ceiling", "roofline")}
        decode["other_shapes"] = []
        for (K2, N2, c2) in ((4096, 14336, 16), (8192, 28672, 6)):   # the prefill configs' weight shapes at M=1
            d2 = bench_decode(torch, lin, pkg, dev, peaks, K=K2, N=N2, copies=c2)
            decode["other_shapes"].append({"workload": d2["workload"], "gbs": d2["value"], "us_per_gemv": d2["us_per_gemv"],
                                           "frac": d2["roofline"]["frac"], "read_ceiling_gbs": d2["read_ceiling"]["gbs"]})
    fault = fault or pkg.read_device_fault()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- CPU baseline on a bounded sample (rank 0, N=1 only) -------------------------------------------
    cpu = None
    if world == 1 and not args.no_cpu and cfg == "c3":
        tops, rows, secs, nthreads, kind = cpu_w4a8_sample(M, K, N, budget_s=12.0)
        cpu = {"value": tops, "unit": "TOPS", "cores": nthreads, "kind": kind,
               "sample": cpu_sample_text(rows, M, N, K, nthreads, kind, secs)}

    line = {
        "metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic", "config": head["config"],
        "gemm_only_ms": head["gemm_only_ms"], "sustained": head["sustained"], "roofline": head["roofline"],
        "e2e": head["e2e"], "gpu_launches": head["gpu_launches"], "clocks": head["clocks"], "device_fault": fault,
    }
    if "gather" in head:
        line["gather"] = head["gather"]
    if cpu:
        line["cpu_baseline"] = cpu
    for c in ("c4", "c5", "layout"):
        if c in extra:
            line[c] = extra[c]
    if decode:
        line["decode_gemv"] = decode
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def pcie_floor(torch, layer, a_host, out_host, timed, steps):
    """The host<->device copies of one forward_host call and nothing else: the same row chunks on the same copy
    streams, a chunk's result copy ordered after its input copy as in the real step, no kernel."""
    m = a_host.shape[0]
    st = layer._pipe(m, 4, a_host.dtype)
    evs = [torch.cuda.Event() for _ in st["bounds"]]

    def copies(i):
        cur = torch.cuda.current_stream()
        st["s_in"].wait_stream(cur)
        st["s_out"].wait_stream(cur)
        for c, (r0, r1) in enumerate(st["bounds"]):
            with torch.cuda.stream(st["s_in"]):
                st["a_dev"][r0:r1].copy_(a_host[r0:r1], non_blocking=True)
                evs[c].record()
            with torch.cuda.stream(st["s_out"]):
                st["s_out"].wait_event(evs[c])
                out_host[r0:r1].copy_(st["out_dev"][r0:r1], non_blocking=True)
        cur.wait_stream(st["s_in"])
        cur.wait_stream(st["s_out"])

    timed(copies, 1, 2)
    batches = sorted(timed(copies, steps, 0) for _ in range(5))
    return batches[len(batches) // 2]


def bench_layout(torch, pkg, dev, peaks):
    """The layout kernels of the C3 shapes as HBM GB/s: the one-time RHS pack (nibbles [14336, 2048 bytes] ->
    packed blocks with row sums) and the per-step activation quantise+pack (bf16 [2048, 4096] -> int8 blocks + scale,
    zero point).  Each is timed over rotating buffer sets larger than L2, CUDA events on the current stream."""
    M, K, N, _ = CONFIGS["c3"]
    uk = pkg.GemmW4A8("bf16")
    pkg.use_current_torch_stream()
    out = {}

    def time_us(fn, sets, reps=3):
        """us per launch of fn(i), i over the rotating sets, replayed as one CUDA graph (no host launch cost in the figure)."""
        stream = torch.cuda.Stream()

        def all_sets():
            pkg.use_current_torch_stream()
            for i in range(sets):
                fn(i)

        us = _graph_time_us(torch, stream, all_sets, sets, max(reps, 3))
        pkg.use_current_torch_stream()
        return us

    sets = 6
    nibs = [torch.randint(0, 256, (N, K // 2), device=dev, dtype=torch.uint8) for _ in range(sets)]
    packed = [torch.empty(uk.get_b_packed_size(N, K), dtype=torch.uint8, device=dev) for _ in range(sets)]
    us = time_us(lambda i: uk.run_bt_pack(N, K, K, K, 0, nibs[i], packed[i]), sets)
    nbytes = N * K // 2 + packed[0].numel()
    out["rhs_pack_qsi4cxp"] = {"workload": f"run_bt_pack qsi4cx N={N} K={K}", "us": us, "bytes": nbytes,
                               "gbs": nbytes / (us * 1e-6) / 1e9, "frac": nbytes / (us * 1e-6) / 1e9 / peaks["hbm"]}
    del nibs, packed
    sets = 8
    acts = [torch.randn((M, K), device=dev).to(torch.bfloat16) for _ in range(sets)]
    ap = [torch.empty(uk.get_a_packed_size(M, K), dtype=torch.uint8, device=dev) for _ in range(sets)]
    sa = torch.empty(M, dtype=torch.float32, device=dev)
    zp = torch.empty(M, dtype=torch.int32, device=dev)
    us = time_us(lambda i: pkg.quant_pack_qai8dxp(acts[i], ap[i], sa, zp), sets, reps=6)
    nbytes = M * K * 3 + 8 * M
    out["quant_pack_qai8dxp_bf16"] = {"workload": f"tqt_run_quant_pack_qai8dxp_bf16 M={M} K={K}", "us": us, "bytes": nbytes,
                                      "gbs": nbytes / (us * 1e-6) / 1e9, "frac": nbytes / (us * 1e-6) / 1e9 / peaks["hbm"]}
    out["note"] = f"bytes in + bytes out per launch / CUDA-event time over rotating buffer sets (> 126 MB); frac of hbm_gbs of {peaks['source']}"
    del acts, ap
    out.update(bench_unpacked_and_conv(torch, pkg, dev, peaks, time_us))
    return out


def bench_unpacked_and_conv(torch, pkg, dev, peaks, time_us):
    """C1's kernel type on row-major operands (tiled TMA loads into the tcgen05 CTA-pair kernel): the reference's own
    CPU-runnable case (M=64, K=512, N=256) as a latency, and M=K=N=4096 as int8 TOPS; and one layer-sized int8
    convolution through the packed channel-last wrapper (fused im2col + pack, then the requantising GEMM)."""
    out = {}
    uk = pkg.GemmClampI32I8I8()
    for (M, K, N, sets, reps) in ((64, 512, 256, 8, 20), (4096, 4096, 4096, 6, 3)):
        A = [torch.randint(-128, 128, (M, K), device=dev, dtype=torch.int8) for _ in range(sets)]
        B = [torch.randint(-128, 128, (K, N), device=dev, dtype=torch.int8) for _ in range(sets)]
        D = [torch.empty((M, N), device=dev, dtype=torch.int32) for _ in range(sets)]
        us = time_us(lambda i: uk.run_gemm(M, N, K, A[i], K, 0, B[i], N, 0, None, N, D[i], N, -2**31, 2**31 - 1), sets, reps=reps)
        rec = {"workload": f"gemm_clamp_i32_i8_i8 M={M} K={K} N={N}, row-major operands (A [m,k], B [k,n]) through tensor maps",
               "us": us, "tops": 2.0 * M * N * K / (us * 1e-6) / 1e12, "kernel_family": pkg.debug_last_kernel()}
        if M == 4096:
            rec["frac"] = rec["tops"] / (2.0 * peaks["bf16"])
            rec["note"] = "frac of 2 x bf16_tflops (burst); sets rotate through 302 MB"
        else:
            rec["note"] = "launch-latency bound: one tile on one CTA pair"
        out["c1_i32_unpacked" if M == 64 else "i32_unpacked_4096"] = rec
        del A, B, D
    # unquantised bf16 GEMM (packed operands) at 4096^3: kind::f16 MMAs, f32 accumulators, bf16 output
    fk = pkg.FloatGemm("gemm_1xnbias_clamp_bf16_bf16p_bf16p")
    Mf = Kf = Nf = 4096
    sets = 6
    ap = [torch.empty(fk.get_a_packed_size(Mf, Kf), dtype=torch.uint8, device=dev) for _ in range(sets)]
    bp = [torch.empty(fk.get_b_packed_size(Nf, Kf), dtype=torch.uint8, device=dev) for _ in range(sets)]
    for i in range(sets):
        fk.run_a_pack(Mf, Kf, Kf, Kf, 0, torch.randn((Mf, Kf), device=dev).to(torch.bfloat16), ap[i])
        fk.run_bt_pack(Nf, Kf, Kf, Kf, 0, torch.randn((Nf, Kf), device=dev).to(torch.bfloat16), bp[i])
    D = [torch.empty((Mf, Nf), device=dev, dtype=torch.bfloat16) for _ in range(sets)]
    us = time_us(lambda i: fk.run_gemm(Mf, Nf, Kf, ap[i], Kf, 0, bp[i], Kf, 0, None, Nf, D[i], Nf, None, -3.0e38, 3.0e38), sets)
    tf = 2.0 * Mf * Nf * Kf / (us * 1e-6) / 1e12
    out["bf16_gemm_4096"] = {"workload": "gemm_1xnbias_clamp_bf16_bf16p_bf16p M=K=N=4096 (unquantised, packed operands)", "us": us,
                             "tflops": tf, "frac": tf / peaks["bf16"], "kernel_family": pkg.debug_last_kernel(),
                             "note": "frac of bf16_tflops (burst); sets rotate through 600 MB"}
    del ap, bp, D
    # the W4A8 prefill shape with both operands left in the caller's layouts (A int8 [m, k], B nibbles [n, k / 2]): tiled TMA
    # loads into the tensor-memory kernel, converters decode the reference's unpacked nibble order
    M, K, N, _ = CONFIGS["c3"]
    us_w = pkg.SiblingGemm("gemm_1xnbias_clamp_bf16_qai8dx_qsi4cxt")
    sets = 5
    A = [torch.randint(-128, 128, (M, K), device=dev, dtype=torch.int8) for _ in range(sets)]
    B = [torch.randint(0, 256, (N, K // 2), device=dev, dtype=torch.uint8) for _ in range(sets)]
    D = [torch.empty((M, N), device=dev, dtype=torch.bfloat16) for _ in range(sets)]
    sa = torch.full((M,), 0.02, device=dev, dtype=torch.float32)
    zp = torch.zeros(M, device=dev, dtype=torch.int32)
    sb = torch.full((N,), 0.004, device=dev, dtype=torch.float32)
    wp = pkg.QaI8DxQsI4CxParams(sa.data_ptr(), zp.data_ptr(), sb.data_ptr())
    us = time_us(lambda i: us_w.run_gemm(M, N, K, A[i], K, 0, B[i], K, 0, None, N, D[i], N, None, -65504.0, 65504.0, wp), sets)
    out["w4a8_unpacked_c3"] = {"workload": f"gemm_1xnbias_clamp_bf16_qai8dx_qsi4cxt M={M} K={K} N={N}, row-major operands through tensor maps",
                               "us": us, "tops": 2.0 * M * N * K / (us * 1e-6) / 1e12, "kernel_family": pkg.debug_last_kernel(),
                               "frac": 2.0 * M * N * K / (us * 1e-6) / 1e12 / (2.0 * peaks["bf16"]),
                               "note": "frac of 2 x bf16_tflops (burst); sets rotate through 480 MB"}
    del A, B, D
    # 56 x 56 x 256 -> 256 channels, 3 x 3, pad 1 (M = 3136, K = 2304, N = 256), batch of 8 images as 8 groups of rows
    ck = pkg.ConvI8(pkg.CONV_TYPES[0])
    IC = OC = 256
    cp = pkg.ConvParams.make(IC, OC, 1, (8, 56, 56), (1, 3, 3), pad=(0, 1, 1))
    Mc, Kc = 8 * 56 * 56, 9 * IC
    sets = 6
    acts = [torch.randint(-128, 128, (8 * 56 * 56 * IC,), device=dev, dtype=torch.int8) for _ in range(sets)]
    W = torch.randint(-127, 128, (OC, Kc), device=dev, dtype=torch.int8)
    wp = torch.empty(ck.get_b_packed_size(OC, Kc), dtype=torch.uint8, device=dev)
    ck.run_bt_pack(OC, Kc, Kc, Kc, 0, W, wp)
    ap = [torch.empty(ck.get_a_im2colpack_size(Mc, Kc), dtype=torch.uint8, device=dev) for _ in range(sets)]
    D = [torch.empty((Mc, OC), device=dev, dtype=torch.int8) for _ in range(sets)]
    sb = torch.full((OC,), 0.004, device=dev, dtype=torch.float32)
    bias = torch.zeros(OC, device=dev, dtype=torch.int32)
    qp = pkg.QaI8QaI8QsI8CxParams(0.05, 0, sb.data_ptr(), OC, 2.0, 0)
    us_col = time_us(lambda i: ck.run_im2colpack(0, acts[i], Kc, 0, ap[i], cp), sets)
    us_all = time_us(lambda i: (ck.run_im2colpack(0, acts[i], Kc, 0, ap[i], cp),
                                ck.run_conv(Mc, OC, Kc, ap[i], Kc, 0, wp, Kc, 0, None, OC, D[i], OC, bias, -128, 127, qp)), sets)
    nbytes = acts[0].numel() + ap[0].numel()
    out["conv_i8_channel_last_packed"] = {
        "workload": "convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp: 8 x 56 x 56 x 256 -> 256 channels, 3 x 3, pad 1 (M=25088, K=2304, N=256)",
        "im2colpack_us": us_col, "im2colpack_gbs": nbytes / (us_col * 1e-6) / 1e9, "im2colpack_frac": nbytes / (us_col * 1e-6) / 1e9 / peaks["hbm"],
        "conv_us": us_all, "tops": 2.0 * Mc * OC * Kc / (us_all * 1e-6) / 1e12,
        "note": "im2colpack bytes = input tensor + packed matrix; conv = im2colpack + run_conv, int8 TOPS of the whole convolution"}
    return out


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


def bench_decode(torch, lin, pkg, dev, peaks, K=4096, N=4096, copies=48, reps=20, M=1):
    """GEMV, M rows (decode batch), f32: one CUDA graph replays `copies` GEMVs over distinct weight sets (together
    larger than L2), so every launch streams its weights from HBM.  `read_ceiling` is a kernel with the same
    launch shape that only reads the same number of bytes from the same buffers, timed the same way."""
    import ctypes
    nbytes = N * K // 2 + 2 * 4 * N + M * (4 * N + K + 8)   # weights + scale_b, bias + per row: D, int8 row, (scale, zp)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    layers = []
    for _ in range(copies):
        nib = torch.randint(0, 256, (N, K // 2), generator=gen, device=dev, dtype=torch.uint8)
        sb = torch.rand(N, generator=gen, device=dev) * 0.01
        layers.append(lin.W4A8Linear(nib, sb, K, "f32", bias=torch.randn(N, generator=gen, device=dev) * 0.1))
    a = torch.randn((M, K), generator=gen, device=dev)
    for L in layers:
        L.quantize(a)
        L.gemm(M)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()

    def gemvs():
        for L in layers:
            L.gemm(M)

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
    phases = None
    if M == 1:
        # clock64 phase stamps of the dp4a GEMV (thread 0 of every CTA), one buffer per launch of the same chain: where a
        # GEMV's time goes when its predecessor is still running (the stamped graph is not the timed one).  The stamps exist
        # in library builds with -DTQT_B200_DIAG only; otherwise the buffers stay zero and `phases` is null.
        lib.tqt_cuda_debug_set_timing_buffer.argtypes = [ctypes.c_void_p]
        bufs = [torch.zeros(148 * 16, dtype=torch.int64, device=dev) for _ in layers]

        def stamped():
            for L, b in zip(layers, bufs):
                lib.tqt_cuda_debug_set_timing_buffer(b.data_ptr())
                L.gemm(M)
            lib.tqt_cuda_debug_set_timing_buffer(None)

        _graph_time_us(torch, stream, stamped, copies, 2)
        pkg.set_stream(torch.cuda.current_stream().cuda_stream)
        rows = []
        for b in bufs[8:]:
            t = b.cpu().numpy().reshape(148, 16)[:, :6].astype("float64")
            t = t[t[:, 5] > 0]
            if len(t):
                rows.append((t[:, 1:] - t[:, :-1]).mean(0))
        if rows:
            import numpy as _np
            d = _np.median(_np.array(rows), axis=0)
            phases = {"unit": "SM cycles, mean over the CTAs of a launch, median over launches 9..48 of the chain",
                      "entry_to_loads_issued": d[0], "griddepcontrol_wait": d[1], "k_loop_after_wait": d[2], "combine": d[3],
                      "epilogue_store": d[4], "total": float(d.sum())}
    return {"metric": "w4a8_gemv_hbm_gbs", "value": gbs, "unit": "GB/s", "us_per_gemv": us, "phases": phases,
            "workload": f"gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp decode M={M} K={K} N={N}",
            "bytes_per_gemv": nbytes, "gpu_launches": reps * copies,
            "read_ceiling": {"gbs": rd / (us_read * 1e-6) / 1e9, "us": us_read,
                             "note": "a kernel with the GEMV's launch shape that only reads the same bytes, same graph"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm"], "algorithmic_bytes": nbytes,
                         "traffic": 8.702e6 if (K, N, M) == (4096, 4096, 1) else None,
                         "traffic_source": ("ncu capture of an earlier run summarised in profiles/gemv_w4a8_c2.txt (one launch, dram "
                                            "read + write); not measured by this run") if (K, N, M) == (4096, 4096, 1) else None,
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
    ap.add_argument("--no-extra", action="store_true", help="headline configuration only: skip the c4 / c5 / layout sub-records")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
