#!/usr/bin/env python
"""Benchmark of the hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload: the large fp16 GEMM M=16384, N=16384, K=8192 (fp32
accumulate, U[-1,1] inputs), N-sharded over the ranks — one step is one pass of
that GEMM; `value` is whole-job TFLOP/s with inputs resident in HBM.  `e2e` is
the same metric through the C-ABI kernel entry point with pinned HOST buffers
(copies inside the timed region).  `extra` carries the other configs (1024^3
and 4096^3 GEMM, softmax GB/s, w8a16 GB/s, MLP tokens/s).  `--impl reference`
times the CPU restatement of the reference's lowering on the host cores on a
bounded sample of the same workload.

Inputs come from one counter-based generator (Philox4x32-10) implemented in the
library (device), in the oracle's C++ and in numpy: A is seed 4, B seed 5, both
U[-1,1); the CPU legs draw the same bytes, and `parity_sample` compares 64
random 128x128 tiles of the timed GEMM's own output with the oracle.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

M, N, K = 16384, 16384, 8192
WORKLOAD = f"gemm_f16_{M}x{N}x{K}"
FLOPS = 2.0 * M * N * K
SEED_A, SEED_B = 4, 5
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) from a thread while the
    timed region runs; a 2 ms period resolves regions of a few tens of milliseconds."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
               "sw_power_cap": 0x4}

    def __init__(self, index: int):
        self.index = index
        self.sm, self.reason_bits, self.max_mhz = [], 0, None
        self._stop = threading.Event()
        self._thread = None
        self._h = None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        except Exception:
            self._h = None
        return self

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
            except Exception:
                pass
            time.sleep(0.002)

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        reasons = sorted(n for n, bit in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                "sm_min_mhz": min(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.sm)}


# ---- the reference arm / CPU baseline: the oracle on host cores -----------------------------

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch, by (variant, M, N, K): each entry comes
# from an ncu capture whose summary is committed under profiles/ (file and capture date beside the
# number).  A run whose variant or shape has no capture reports traffic null.
DRAM_TRAFFIC_CAPTURES = {
    ("tc256x256x64_2cta_s6", 16384, 16384, 8192): {
        "bytes": 8.371e9 + 0.532e9, "profile": "profiles/bench_gemm_16384x16384x8192_launches.md", "captured": "2026-11-25"},
    ("tc256x256x64_2cta_streamk", 16384, 16384, 8192): {
        "bytes": 6.417e9 + 0.545e9, "profile": "profiles/bench_gemm_16384x16384x8192_launches.md (stream-K section)",
        "captured": "2026-11-25"},
}


def operand_rows(r0, rows):
    """Rows [r0, r0+rows) of A as the device holds them (same generator, same seed)."""
    import oracle
    return oracle.random_rows(r0, rows, K, np.float16, SEED_A, oracle.UNIFORM, -1.0, 1.0)


def operand_cols(c0, cols):
    """Columns [c0, c0+cols) of the whole B [K, N]."""
    import oracle
    return oracle.random_cols(c0, cols, K, N, np.float16, SEED_B, oracle.UNIFORM, -1.0, 1.0)


def cpu_gemm_sample(target_s: float = 4.0):
    """The CPU restatement on a slab of M rows (full N, K) sized to about target_s per pass; the
    operands are the bytes the GPU arm multiplies."""
    import oracle
    threads = oracle.hw_threads()
    b = oracle.fill_random((K, N), np.float16, SEED_B, oracle.UNIFORM, -1.0, 1.0)

    def once(rows):
        a = operand_rows(0, rows)
        t0 = time.perf_counter()
        oracle.gemm_f16(a, b, threads=threads)
        return time.perf_counter() - t0
    once(threads)  # page in
    # every call widens B to fp32 once (fixed cost); the slope between two slab sizes is the per-row cost
    t_small, t_large = once(threads), once(3 * threads)
    per_row = max((t_large - t_small) / (2 * threads), 1e-6)
    fixed = max(t_small - per_row * threads, 0.0)
    rows = int(max(threads, min(4096, (target_s - fixed) / per_row)))
    rows -= rows % threads
    a = operand_rows(0, max(rows, threads))
    return a, b, a.shape[0], threads


def cpu_time_once(a, b, threads):
    import oracle
    t0 = time.perf_counter()
    c = oracle.gemm_f16(a, b, threads=threads)
    return time.perf_counter() - t0, c


def cpu_baseline(target_s: float = 4.0):
    """One warm pass, then three timed ones; the median is reported (the harness protocol of the
    reference: repetitions and quantiles, backend/hmx_search.py:1109-1171)."""
    a, b, rows, threads = cpu_gemm_sample(target_s)
    cpu_time_once(a, b, threads)
    times = sorted(cpu_time_once(a, b, threads)[0] for _ in range(3))
    dt = times[1]
    tflops = 2.0 * rows * N * K / dt / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"rows 0..{rows} of {M} of A (full N={N}, K={K}), one warm pass + 3 timed, median {dt:.2f} s "
                      f"(min {times[0]:.2f}, max {times[2]:.2f}); whole problem extrapolates linearly to {dt * M / rows:.0f} s"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    a, b, rows, threads = cpu_gemm_sample(target_s=max(min(2.0, args.reference_seconds),
                                                       args.reference_seconds / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_time_once(a, b, threads)
    times = [cpu_time_once(a, b, threads)[0] for _ in range(args.steps)]
    dt = sum(times) / len(times)
    tflops = 2.0 * rows * N * K / dt / 1e12
    sample = (f"rows 0..{rows} of {M} of A per step (full N={N}, K={K}), the GPU arm's own operand bytes; "
              "CPU restatement of the reference lowering")
    line = {
        "impl": "reference", "metric": "gemm_f16_tflops", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ---- the product arm ----------------------------------------------------------------------------

def timed(torch, fn, steps, warmup, dist=None):
    """warmup untimed calls, then `steps` calls between CUDA events on the current stream;
    barrier + synchronize on both sides; max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms / steps


def graph_timed(torch, fn, reps, inner):
    """Launch-bound kernels: capture `inner` calls in a CUDA graph, replay `reps` times."""
    fn()
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        fn()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            for _ in range(inner):
                fn()
    torch.cuda.synchronize()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * inner)


def extras_single_gpu(torch, hm, peaks, only=None):
    """The other configs of the metric, one GPU.  Each entry: algorithmic work / device time.
    `only` restricts the run to the cases whose name starts with it (profiling captures)."""
    out = {}
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)

    def want(name):
        return only is None or name.startswith(only) or only.startswith(name)

    def rand_h(shape, lo=-1.0, hi=1.0):
        return (torch.rand(shape, generator=g, device=dev) * (hi - lo) + lo).half()

    for n in (512, 1024, 2048, 4096, 8192):  # the square sweep of the large-GEMM config
        kloop_only = only is not None and only.startswith("kloop")  # profiling captures of the K-looped form alone
        if not want(f"gemm_f16_{n}") and not (kloop_only and n == 4096):
            continue
        # rotate over enough operand sets to exceed L2 between launches
        sets = max(2, int(np.ceil(3 * 126e6 / (3 * n * n * 2))))
        sets = min(sets, 24)
        A = [rand_h((n, n)) for _ in range(sets)]
        B = [rand_h((n, n)) for _ in range(sets)]
        C = [torch.empty((n, n), dtype=torch.float16, device=dev) for _ in range(sets)]
        state = {"i": 0}

        def fn():
            i = state["i"] % sets
            state["i"] += 1
            hm.matmul[(1,)](A[i], B[i], C[i])
        # (launches of a few microseconds are replayed from a CUDA graph: issued from Python they are host-bound)
        if not kloop_only:
            ms = graph_timed(torch, fn, reps=5, inner=sets * 2) if n <= 2048 else timed(torch, fn, 40 if n <= 4096 else 10, 5)
            tf = 2.0 * n ** 3 / (ms * 1e-3) / 1e12
            out[f"gemm_f16_{n}^3"] = {"us": ms * 1e3, "tflops": tf, "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"],
                                      "variant": hm.gemm_explain(n, n, n)["name"]}
        if only is None:
            # what the on-device search (enumerate, verify, measure, gate, canary) picks for the shape
            hm.autotune_cache_clear()
            rep = hm.gemm_autotune(n, n, n)
            names = {v["variant"]: v["name"] for v in hm.gemm_variants()}
            out[f"gemm_f16_{n}^3"]["search"] = {"verdict": rep.get("round_verdict"),
                                               "champion": names.get(rep.get("champion_variant"), None)}
            hm.autotune_cache_clear()
        if n == 4096:
            # the K-looped form (fp16 read-out per 64-deep segment, fp32 running sum in the read-out warps)
            def fk():
                i = state["i"] % sets
                state["i"] += 1
                hm.klooped_matmul[(1,)](A[i], B[i], C[i], BLOCK_K=64)
            ms = timed(torch, fk, 20, 3)
            tf = 2.0 * n ** 3 / (ms * 1e-3) / 1e12
            out[f"gemm_f16_kloop64_{n}^3"] = {"us": ms * 1e3, "tflops": tf,
                                              "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"]}

            # the same form with the reference test's own segment (test_matmul_kloop.py: BLOCK_K = 256)
            def fk256():
                i = state["i"] % sets
                state["i"] += 1
                hm.klooped_matmul[(1,)](A[i], B[i], C[i], BLOCK_K=256)
            ms = timed(torch, fk256, 20, 3)
            tf = 2.0 * n ** 3 / (ms * 1e-3) / 1e12
            out[f"gemm_f16_kloop256_{n}^3"] = {"us": ms * 1e3, "tflops": tf,
                                               "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"]}
        del A, B, C
    if want("softmax"):
        # C2 softmax [4096,1024]: 16 MiB in + out per launch; 12 buffer pairs (201 MB) rotate past L2
        sets = 12
        X = [(torch.randn((4096, 1024), generator=g, device=dev) * 3).half() for _ in range(sets)]
        Y = [torch.empty_like(X[0]) for _ in range(sets)]
        state = {"i": 0}

        def sm():
            i = state["i"] % sets
            state["i"] += 1
            hm.softmax_kernel[(1,)](X[i], Y[i])
        ms = graph_timed(torch, sm, reps=10, inner=sets * 2)
        gbs = 2 * 4096 * 1024 * 2 / (ms * 1e-3) / 1e9
        # yardstick: a plain device copy of the same buffers, timed the same way (launch and first-byte
        # latency weigh on a 16 MiB launch whatever it computes; the HBM peak is a large copy's)
        state["i"] = 0

        def cp():
            i = state["i"] % sets
            state["i"] += 1
            Y[i].copy_(X[i])
        cms = graph_timed(torch, cp, reps=10, inner=sets * 2)
        out["softmax_f16_4096x1024"] = {"us": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                        "same_size_copy_us": cms * 1e3, "frac_of_same_size_copy": cms / ms}
        del X, Y
        # the same kernel where the launch and the first-byte latency no longer dominate: 8x the rows
        X = [(torch.randn((32768, 1024), generator=g, device=dev) * 3).half() for _ in range(3)]
        Y = [torch.empty_like(X[0]) for _ in range(3)]
        state = {"i": 0}

        def sm_big():
            i = state["i"] % 3
            state["i"] += 1
            hm.softmax_kernel[(1,)](X[i], Y[i])
        ms = graph_timed(torch, sm_big, reps=10, inner=6)
        gbs = 2 * 32768 * 1024 * 2 / (ms * 1e-3) / 1e9
        out["softmax_f16_32768x1024"] = {"us": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}
        del X, Y
    if want("rmsnorm"):
        # RMSNorm / SwiGLU at the MLP's shapes
        x = torch.randn((2048, 4096), generator=g, device=dev).half()
        xs = [x.clone() for _ in range(8)]
        ys = [torch.empty_like(x) for _ in range(8)]
        w = torch.ones(4096, dtype=torch.float16, device=dev)
        state = {"i": 0}

        def rn():
            i = state["i"] % 8
            state["i"] += 1
            hm.rms_norm_fwd_kernel[(1,)](xs[i], ys[i], w, EPSILON=1e-6)
        ms = graph_timed(torch, rn, reps=10, inner=16)
        gbs = (2 * 2048 * 4096 * 2 + 4096 * 2) / (ms * 1e-3) / 1e9
        state["i"] = 0

        def rcp():
            i = state["i"] % 8
            state["i"] += 1
            ys[i].copy_(xs[i])
        cms = graph_timed(torch, rcp, reps=10, inner=16)
        out["rmsnorm_f16_2048x4096"] = {"us": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                        "same_size_copy_us": cms * 1e3, "frac_of_same_size_copy": cms / ms}
        del xs, ys
    if want("swiglu"):
        nel = 2048 * 11008
        gs = [torch.randn(nel, generator=g, device=dev).half() for _ in range(3)]
        us = [torch.randn(nel, generator=g, device=dev).half() for _ in range(3)]
        os_ = [torch.empty(nel, dtype=torch.float16, device=dev) for _ in range(3)]
        state = {"i": 0}

        def sw():
            i = state["i"] % 3
            state["i"] += 1
            hm.swiglu_kernel[(1,)](gs[i], us[i], os_[i])
        ms = graph_timed(torch, sw, reps=10, inner=6)
        gbs = 3 * nel * 2 / (ms * 1e-3) / 1e9
        out["swiglu_f16_2048x11008"] = {"us": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}
        del gs, us, os_
    if want("w8a16"):
        # C3 w8a16: four distinct resident weights (180 MB) rotate past L2 = cold-L2 number;
        # one weight re-used = L2-resident number
        k, n = 4096, 11008
        Wq = [torch.randint(-127, 128, (k, n), generator=g, device=dev, dtype=torch.int8) for _ in range(4)]
        S = (torch.rand(n, generator=g, device=dev) * 0.019 + 0.001).half()
        for mrows in (1, 16, 256):
            if not want(f"w8a16_m{mrows}_"):
                continue
            a = torch.randn((mrows, k), generator=g, device=dev).half()
            c = torch.empty((mrows, n), dtype=torch.float16, device=dev)
            state = {"i": 0}

            def wf():
                i = state["i"] % 4
                state["i"] += 1
                hm.w8a16_matmul[(1,)](a, Wq[i], S, c)

            def wf_same():
                hm.w8a16_matmul[(1,)](a, Wq[0], S, c)
            for _ in range(4):
                wf()
            ms = graph_timed(torch, wf, reps=10, inner=8)
            ms_hot = graph_timed(torch, wf_same, reps=10, inner=8)
            # the same weight under an L2 persistence window (registered with l2_persist: the decode
            # case of weight residency); other traffic (an 80 MB copy between launches) competes for L2
            hm.unregister_w8a16_weight(Wq[0])
            hm.register_w8a16_weight(Wq[0], S, l2_persist=True)
            noise_src = torch.empty(40 << 20, dtype=torch.uint8, device=dev)
            noise_dst = torch.empty_like(noise_src)

            def wf_noise():
                noise_dst.copy_(noise_src)
                hm.w8a16_matmul[(1,)](a, Wq[0], S, c)

            def noise_only():
                noise_dst.copy_(noise_src)
            ms_persist = graph_timed(torch, wf_noise, reps=10, inner=8) - graph_timed(torch, noise_only, reps=10, inner=8)
            hm.unregister_w8a16_weight(Wq[0])
            hm.register_w8a16_weight(Wq[0], S, l2_persist=False)
            ms_plain_noise = graph_timed(torch, wf_noise, reps=10, inner=8) - graph_timed(torch, noise_only, reps=10, inner=8)
            del noise_src, noise_dst
            bytes_ = k * n + 2 * n + 2 * mrows * k + 2 * mrows * n
            gbs = bytes_ / (ms * 1e-3) / 1e9
            out[f"w8a16_m{mrows}_4096x11008"] = {
                "us": ms * 1e3, "us_cold": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                "us_weight_in_l2": ms_hot * 1e3,
                "us_persisting_l2": ms_persist * 1e3, "us_no_window_same_traffic": ms_plain_noise * 1e3,
                "persisting_note": "one weight re-used with an 80 MB copy between launches; with and without the L2 "
                                   "persistence window; the copy's own time subtracted",
                "tflops": 2.0 * mrows * k * n / (ms * 1e-3) / 1e12}
        for wq_ in Wq:
            hm.unregister_w8a16_weight(wq_)
        del Wq
        if only is not None and not "w8a16_m1_4096x32000".startswith(only):
            return out
        # the same kernel on a wider weight (a vocabulary projection): twice the bytes per CTA per launch,
        # so the ~6 us a launch costs before and after its streaming phase weigh half as much
        k, n = 4096, 32000
        Wq = [torch.randint(-127, 128, (k, n), generator=g, device=dev, dtype=torch.int8) for _ in range(2)]
        S = (torch.rand(n, generator=g, device=dev) * 0.019 + 0.001).half()
        a = torch.randn((1, k), generator=g, device=dev).half()
        c = torch.empty((1, n), dtype=torch.float16, device=dev)
        state = {"i": 0}

        def wide():
            i = state["i"] % 2
            state["i"] += 1
            hm.w8a16_matmul[(1,)](a, Wq[i], S, c)
        for _ in range(2):
            wide()
        ms = graph_timed(torch, wide, reps=10, inner=4)
        bytes_ = k * n + 2 * n + 2 * k + 2 * n
        out["w8a16_m1_4096x32000"] = {"us": ms * 1e3, "gbs": bytes_ / (ms * 1e-3) / 1e9,
                                      "frac_of_measured_hbm": bytes_ / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        for wq_ in Wq:
            hm.unregister_w8a16_weight(wq_)
        del Wq
    if want("gemm_i8_4096"):
        n = 4096
        a8 = [torch.randint(-128, 128, (n, n), generator=g, device=dev, dtype=torch.int8) for _ in range(4)]
        b8 = [torch.randint(-128, 128, (n, n), generator=g, device=dev, dtype=torch.int8) for _ in range(4)]
        c32 = torch.empty((n, n), dtype=torch.int32, device=dev)
        state = {"i": 0}

        def i8():
            i = state["i"] % 4
            state["i"] += 1
            hm.matmul_i8[(1,)](a8[i], b8[i], c32)
        ms = graph_timed(torch, i8, reps=5, inner=8)
        out["gemm_i8_4096^3"] = {"us": ms * 1e3, "tops": 2.0 * n ** 3 / (ms * 1e-3) / 1e12,
                                 "note": "int32 sums, exact; includes the transpose of B"}
        del a8, b8, c32
    # attention block: the reference's own case (one head of 1024 x 64, fp32 tensors, sm_scale 0.5:
    # test/python/triton/test_flash_attention.py:17,37) and head counts / lengths that fill the device
    for name, (z, h, n, d, f32) in {"attention_f32_1x1x1024x64": (1, 1, 1024, 64, True),
                                    "attention_f16_4x16x4096x64": (4, 16, 4096, 64, False),
                                    "attention_f16_4x16x4096x128": (4, 16, 4096, 128, False),
                                    "attention_f16_causal_4x16x4096x128": (4, 16, 4096, 128, False)}.items():
        if not want(name):
            continue
        dt = torch.float32 if f32 else torch.float16
        sets = 2 if z * h > 1 else 8  # 4 x 16 x 4096 x 128: 67 MB per tensor, two sets exceed L2
        Q, K, V = ([torch.rand((z, h, n, d), generator=g, device=dev).to(dt) for _ in range(sets)] for _ in range(3))
        O = [torch.empty_like(Q[0]) for _ in range(sets)]
        state = {"i": 0}
        scale = 0.5 if f32 else d ** -0.5

        def att():
            i = state["i"] % sets
            state["i"] += 1
            hm.attention(Q[i], K[i], V[i], O[i], scale, causal="causal" in name)
        ms = graph_timed(torch, att, reps=5, inner=sets * (1 if z * h > 1 else 4))
        flops = 4.0 * z * h * n * n * d * (0.5 if "causal" in name else 1.0)
        out[name] = {"us": ms * 1e3, "tflops": flops / (ms * 1e-3) / 1e12,
                     "frac_of_measured_bf16_burst": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
        del Q, K, V, O
    return out


def mlp_extra(torch, hm, dist, rank, world):
    """C4: Llama MLP block, 2048 tokens x 4096, ffn 11008, tensor-parallel over the ranks.  Every N is
    timed the same way: the whole step (kernels and, at N > 1, the all-reduce — one call into the
    library) replayed from a CUDA graph.  `phases_us` is a separate, eager run with events between
    the block's phases."""
    from hexagon_mlir_b200 import tp
    t, d, f = 2048, 4096, 11008
    x = torch.empty((t, d), dtype=torch.float16, device="cuda")
    hm.fill_random(x, 3, hm.NORMAL, 0.0, 1.0)
    gain = torch.ones(d, dtype=torch.float16, device="cuda")
    lo, hi = tp.shard_bounds(f, rank, world)

    def shard(seed, shape, rows=None, cols=None):
        full = torch.empty(shape, dtype=torch.float16, device="cuda")
        hm.fill_random(full, seed, hm.NORMAL, 0.0, 0.02)
        part = full[:, lo:hi] if cols else full[lo:hi]
        return part.contiguous()
    wg, wu, wd = shard(31, (d, f), cols=True), shard(32, (d, f), cols=True), shard(33, (f, d), rows=True)
    out = torch.empty_like(x)
    group = dist.group.WORLD if world > 1 else None
    block = tp.TensorParallelMLP(gain, wg, wu, wd, eps=1e-6, group=group)
    block.captured(x, out)
    ms = timed(torch, lambda: block.captured(x, out), 20, 5, dist if world > 1 else None)
    mode = "cuda-graph"
    # per-phase times (eager, events inside the call)
    hm.set_option("mlpPhaseTiming", 1)
    for _ in range(3):
        block(x, out)
    phases = {k: round(v, 2) for k, v in hm.mlp_phase_times().items()}
    hm.set_option("mlpPhaseTiming", 0)
    torch.cuda.synchronize()
    flops = 6.0 * t * d * f
    reduction = "ncclAllReduce inside mlp_block_tp_float16 (C++)" if world > 1 else "none"
    forms = {}
    if world > 1:
        forms["nccl_all_reduce_ms"] = ms
        # two token chunks: the all-reduce of chunk 0 under the kernels of chunk 1
        try:
            b2 = tp.TensorParallelMLP(gain, wg, wu, wd, eps=1e-6, group=group, chunks=2)
            b2.captured(x, out)
            forms["nccl_two_chunks_ms"] = timed(torch, lambda: b2.captured(x, out), 20, 5, dist)
            b2.release()
            if forms["nccl_two_chunks_ms"] < ms:
                ms, reduction = forms["nccl_two_chunks_ms"], reduction + ", two token chunks overlapped"
        except Exception as exc:  # noqa: BLE001
            forms["nccl_two_chunks_ms"] = f"unavailable ({type(exc).__name__})"
        # the same block with the reduction fused into the kernels (peer stores over NVLink)
        try:
            fused = tp.FusedTensorParallelMLP(gain, wg, wu, wd, tokens=t, eps=1e-6, group=dist.group.WORLD)
            fused.captured(x)
            fms = timed(torch, lambda: fused.captured(x), 20, 5, dist)
            fused.release()
            forms["fused_peer_store_ms"] = fms
            if fms < ms:
                ms, reduction = fms, "fused: read-out pushes partial rows to their owners"
        except Exception as exc:  # symmetric memory is a property of the box, not of this code
            forms["fused_peer_store_ms"] = f"unavailable ({type(exc).__name__})"
        # the all-reduce by this library's own kernel over NVSwitch multicast (multimem.ld_reduce / multimem.st):
        # with barrier kernels around the launch, and with both rendezvous inside the launch
        for key, rdv, ch, what in (
                ("multicast_all_reduce_ms", "barriers", 1, "barrier kernels around it"),
                ("multicast_own_barriers_ms", "own_barriers", 1, "the whole block one C++ call, the library's barrier launches around its all-reduce"),
                ("multicast_in_kernel_rendezvous_ms", "kernel", 1, "both rendezvous inside the launch"),
                ("multicast_entry_rendezvous_ms", "entry", 1, "the wait for the partials inside the launch, a barrier kernel after it"),
                ("multicast_two_chunks_overlapped_ms", "kernel", 2,
                 "one call, each token chunk's all-reduce beside the next chunk's down GEMM")):
            try:
                mc = tp.MulticastTensorParallelMLP(gain, wg, wu, wd, tokens=t, eps=1e-6, group=dist.group.WORLD,
                                                   rendezvous=rdv, chunks=ch)
                if mc.available():
                    mc.captured(x)
                    mms = timed(torch, lambda: mc.captured(x), 20, 5, dist)
                    mc.release()
                    forms[key] = mms
                    if hm.device_status() != 0:
                        forms[key] = "a bounded wait ran out"
                    elif mms < ms:
                        ms, reduction = mms, f"own kernel over NVSwitch multicast (multimem.ld_reduce + multimem.st), {what}"
                else:
                    forms[key] = "unavailable (no multicast mapping)"
            except Exception as exc:  # noqa: BLE001
                forms[key] = f"unavailable ({type(exc).__name__}: {exc})"[:200]
    block.release()  # the captured graph holds NCCL work: drop it before the process group goes
    return {"ms": ms, "reduction": reduction, **forms, "tokens_per_s": t / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
            "parallelism": f"tp{world}", "allreduce_bytes": t * d * 2 if world > 1 else 0, "launch": mode,
            "phases_us": phases}


def mlp_shard_compute(torch, hm):
    """The compute side of the tensor-parallel MLP on ONE GPU: rank 0's shard of 2, 4 and 8 ranks
    (F / ways columns of Wg and Wu, rows of Wd), no collective, replayed from a CUDA graph, with
    the phase times of an eager run.  What a step at N ranks takes beyond this is the exchange."""
    from hexagon_mlir_b200 import tp
    t, d, f = 2048, 4096, 11008
    x = torch.empty((t, d), dtype=torch.float16, device="cuda")
    hm.fill_random(x, 3, hm.NORMAL, 0.0, 1.0)
    gain = torch.ones(d, dtype=torch.float16, device="cuda")
    out = torch.empty_like(x)
    res = {}
    for ways in (2, 4, 8):
        lo, hi = tp.shard_bounds(f, 0, ways)
        w = []
        for seed, shape, cols in ((31, (d, f), True), (32, (d, f), True), (33, (f, d), False)):
            full = torch.empty(shape, dtype=torch.float16, device="cuda")
            hm.fill_random(full, seed, hm.NORMAL, 0.0, 0.02)
            w.append((full[:, lo:hi] if cols else full[lo:hi]).contiguous())
            del full
        block = tp.TensorParallelMLP(gain, w[0], w[1], w[2], eps=1e-6, group=None)
        block.captured(x, out)
        ms = timed(torch, lambda: block.captured(x, out), 20, 5, None)
        hm.set_option("mlpPhaseTiming", 1)
        for _ in range(3):
            block(x, out)
        phases = {k: round(v, 2) for k, v in hm.mlp_phase_times().items()}
        hm.set_option("mlpPhaseTiming", 0)
        torch.cuda.synchronize()
        block.release()
        res[f"tp{ways}_shard"] = {"ms": ms, "ffn_columns": hi - lo, "phases_us": phases,
                                  "tflops": 6.0 * t * d * (hi - lo) / (ms * 1e-3) / 1e12}
    return res


def parity_sample(torch, hm, c, n_lo, tiles=64, tile=128):
    """`tiles` random tile x tile blocks of the timed GEMM's output against the oracle (full K);
    the operand rows and columns are drawn on the CPU from the generator that filled the device."""
    import oracle
    rng = np.random.Generator(np.random.Philox(1234))
    picks = set()
    while len(picks) < tiles:
        picks.add((int(rng.integers(c.shape[0] // tile)), int(rng.integers(c.shape[1] // tile))))
    worst, rows_cache = 0.0, {}
    for tm, tn in sorted(picks):
        if tm not in rows_cache:
            rows_cache[tm] = operand_rows(tm * tile, tile)
        want = oracle.gemm_f16(rows_cache[tm], operand_cols(n_lo + tn * tile, tile)).astype(np.float32)
        got = c[tm * tile:(tm + 1) * tile, tn * tile:(tn + 1) * tile].cpu().numpy().astype(np.float32)
        worst = max(worst, float(np.abs(got - want).max() / max(float(np.abs(want).max()), 1e-30)))
    return {"tiles": len(picks), "tile": tile, "max_abs_rel": worst, "against": "oracle.gemm_f16, full K"}


def run_product_arm(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # Libraries (NCCL's version banner, for one) print to stdout; the contract is ONE JSON line
    # there, so everything else goes to stderr and the line is written to the saved descriptor.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world != args.gpus and world > 1:
        args.gpus = world
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local)
    import hexagon_mlir_b200 as hm
    hm.init(local)
    multi = world > 1
    if multi:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks, peak_kind = load_peaks()
    if args.case:
        # one small case of `extra` alone (what the ncu captures under profiles/ run)
        if args.case == "mlp":
            result = {"mlp_block_2048x4096x11008": mlp_extra(torch, hm, dist, rank, world)}
        elif args.case == "mlp_shards":
            result = {"mlp_shard_compute_one_gpu": mlp_shard_compute(torch, hm)}
        else:
            result = extras_single_gpu(torch, hm, peaks, only=args.case)
        line = json.dumps({"case": args.case, "result": result})
        os.write(json_fd, (line + "\n").encode())
        return 0

    # inputs resident in HBM: A replicated, this rank's column block of B and C; the bytes are the
    # generator's (A seed 4, the whole B seed 5), so every rank and the CPU legs see the same operands
    n_lo, n_hi = rank * N // world, (rank + 1) * N // world
    n_loc = n_hi - n_lo
    a = torch.empty((M, K), dtype=torch.float16, device="cuda")
    hm.fill_random(a, SEED_A, hm.UNIFORM, -1.0, 1.0)
    b_full = torch.empty((K, N), dtype=torch.float16, device="cuda")
    hm.fill_random(b_full, SEED_B, hm.UNIFORM, -1.0, 1.0)
    b = b_full[:, n_lo:n_hi].contiguous() if world > 1 else b_full
    del b_full
    c = torch.empty((M, n_loc), dtype=torch.float16, device="cuda")

    def step():
        hm.matmul[(1,)](a, b, c)

    step()
    torch.cuda.synchronize()
    if hm.device_status() != 0:
        raise SystemExit("bench.py: device status word set after the first GEMM")
    hm.reset_launch_count()
    with ClockSampler(local) as clk:
        ms = timed(torch, step, args.steps, args.warmup, dist if multi else None)
    launches = hm.launch_count() - args.warmup
    clocks = clk.summary()
    tflops = FLOPS / (ms * 1e-3) / 1e12
    kernel_tflops = (2.0 * M * n_loc * K) / (ms * 1e-3) / 1e12  # this rank's kernel
    plan = hm.gemm_explain(M, n_loc, K)

    # The device-timed value exists from here on.  Everything after it (long run, parity sample, the
    # host-buffer calls, the extra kernels and the multi-rank MLP forms) is reported in the same
    # line; should one of those stages fail or stall on some rank, the line is still written, with
    # what was measured and the stage named in "incomplete".
    peak = peaks["bf16_tflops"]
    capture = DRAM_TRAFFIC_CAPTURES.get((plan["name"], M, n_loc, K))
    line = {
        "metric": "gemm_f16_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sharding": f"N split over {world} rank(s), A replicated, no collective",
                   "l2": "inputs larger than L2 (A 268 MB per rank)", "variant": plan["name"],
                   "inputs": f"Philox4x32-10, A seed {SEED_A}, B seed {SEED_B}, U[-1,1)",
                   "accumulate": "fp32 in TMEM, one fp16 rounding"},
        "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": peak, "unit": "TFLOP/s",
                     "frac": kernel_tflops / peak,
                     "traffic": (capture or {}).get("bytes"), "traffic_source": capture,
                     "peak_source": f"{peak_kind} cuBLAS bf16 burst; sustained {peaks.get('bf16_tflops_sustained')}",
                     "frac_of_sustained": kernel_tflops / peaks.get("bf16_tflops_sustained", peak),
                     "frac_of_nominal_2250": kernel_tflops / 2250.0,
                     "algorithmic_flops_per_launch": 2.0 * M * n_loc * K},
        "cpu_baseline": None, "e2e": None, "parity_sample": None, "long_run": None,
        "gpu_launches": int(launches), "clocks": clocks, "extra": {},
    }
    stage = {"name": "long_run", "written": False}
    write_lock = threading.Lock()

    def write_line(incomplete=None):
        with write_lock:
            if stage["written"]:
                return
            stage["written"] = True
            if incomplete:
                line["incomplete"] = incomplete
            if rank == 0:
                sys.stdout.flush()
                os.write(json_fd, (json.dumps(line) + "\n").encode())

    def stalled():
        write_line(f"stage '{stage['name']}' did not finish within {args.stage_limit:.0f} s on some rank")
        os._exit(0)
    watchdog = threading.Timer(args.stage_limit, stalled)
    watchdog.daemon = True
    watchdog.start()

    # the same loop kept running for --min-time seconds: the chip settles at the clock its power
    # limit allows, and time x median SM MHz lets runs at different N be compared at equal clocks
    long_run = None
    if args.min_time > 0:
        per_round = max(1, int(0.25 / (ms * 1e-3)))
        total_ms, total_steps = 0.0, 0
        with ClockSampler(local) as lclk:
            t_wall = time.perf_counter()
            while time.perf_counter() - t_wall < args.min_time:
                total_ms += timed(torch, step, per_round, 0, dist if multi else None) * per_round
                total_steps += per_round
        lsum = lclk.summary()
        lms = total_ms / total_steps
        long_run = {"seconds": round(time.perf_counter() - t_wall, 2), "steps": total_steps, "ms_per_step": lms,
                    "value": FLOPS / (lms * 1e-3) / 1e12, "sm_mhz_median": lsum["sm_mhz"], "reasons": lsum["reasons"],
                    "ms_x_mhz": lms * lsum["sm_mhz"] if lsum["sm_mhz"] else None}

    line["long_run"] = long_run

    # parity of the timed result itself (untimed): sampled tiles against the oracle
    stage["name"] = "parity_sample"
    parity = parity_sample(torch, hm, c, n_lo) if rank == 0 else None
    if parity is not None and not parity["max_abs_rel"] <= 1e-2:
        raise SystemExit(f"bench.py: the timed GEMM disagrees with the oracle: {parity}")
    line["parity_sample"] = parity
    stage["name"] = "e2e"

    def measure_e2e():
        # e2e: same GEMM through the kernel entry point with pinned host buffers.  At N > 1 every rank's
        # host holds the same A: each rank sends up its 1/N row slab over its own PCIe link and the
        # slabs are exchanged GPU to GPU inside the call (option replicatedOperandA; needs the library's
        # own communicator, which tp.init_group creates).
        e2e_steps = max(1, min(3, args.steps))
        ha = torch.empty((M, K), dtype=torch.float16).pin_memory()
        hb = torch.empty((K, n_loc), dtype=torch.float16).pin_memory()
        hc = torch.empty((M, n_loc), dtype=torch.float16).pin_memory()
        ha.copy_(a)
        hb.copy_(b)
        torch.cuda.synchronize()
        npa, npb, npc = ha.numpy(), hb.numpy(), hc.numpy()
        sharded_upload = False
        if multi:
            from hexagon_mlir_b200 import tp
            tp.init_group(dist.group.WORLD)
            hm.set_option("replicatedOperandA", 1)
            sharded_upload = True

        # what the host side gives at this moment, all ranks copying at once: one direction at a time,
        # then both at once.  The GPUs of a box share one host (and the host is shared with other
        # tenants), so the aggregate — not the per-GPU link — bounds the host-buffer call at N > 1.
        def link_rate(up, down):
            s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
            if multi:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            if up:
                with torch.cuda.stream(s1):
                    c2.copy_(hc, non_blocking=True)
            if down:
                with torch.cuda.stream(s2):
                    hc2.copy_(c, non_blocking=True)
            torch.cuda.synchronize()
            gbs = hc.numel() * 2 / (time.perf_counter() - t0) / 1e9
            if multi:
                t = torch.tensor([gbs], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
                gbs = float(t.item())
            return gbs
        c2, hc2 = torch.empty_like(c), torch.empty_like(hc).pin_memory()
        link_rate(True, True)
        host_link = {"h2d_gbs_per_gpu": round(link_rate(True, False), 1), "d2h_gbs_per_gpu": round(link_rate(False, True), 1),
                     "both_ways_gbs_each_per_gpu": round(link_rate(True, True), 1), "ranks_copying_at_once": world,
                     "rate": "slowest rank"}
        bytes_rank = (M * K // world + K * n_loc + M * n_loc) * 2
        host_link["floor_ms"] = round(bytes_rank / 2 / (host_link["both_ways_gbs_each_per_gpu"] * 1e9) * 1e3, 2)
        del c2, hc2

        def e2e_step():
            hm.matmul[(1,)](npa, npb, npc)  # H2D A and B, GEMM, D2H C, wait — all inside the call
        e2e_step()
        e2e_each = [timed(torch, e2e_step, 1, 0, dist if multi else None) for _ in range(e2e_steps)]
        e2e_ms = sum(e2e_each) / len(e2e_each)
        hm.set_option("replicatedOperandA", 0)
        slab_mode = hm.tp_slab_exchange_mode() if multi else "none"
        e2e_tflops = FLOPS / (e2e_ms * 1e-3) / 1e12
        # the strips of the host path and the whole-problem device run may take different variants
        # (fp32 sums associated differently): agreement is stated as an error, not as byte equality
        sl = slice(0, 256)
        dref = c[sl].float()
        e2e_err = float((hc[sl].cuda().float() - dref).abs().max() / dref.abs().max())
        h2d_step = (M * K // (world if sharded_upload else 1) + K * n_loc) * 2 * world
        # ... and as byte equality with every launch on ONE whole-tile variant (same fp32 sums in the same order)
        hm.set_option("gemmVariant", 3)
        if sharded_upload:
            hm.set_option("replicatedOperandA", 1)
        try:
            e2e_step()
            c_one = torch.empty_like(c)
            hm.matmul[(1,)](a, b, c_one)
            torch.cuda.synchronize()
            e2e_bytes_equal = bool(torch.equal(hc.cuda(), c_one))
            del c_one
        finally:
            hm.set_option("gemmVariant", -1)
            hm.set_option("replicatedOperandA", 0)
        del ha, hb, hc
        return {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d_step,
                "d2h_bytes_per_step": M * n_loc * 2 * world, "steps": e2e_steps,
                "ms_each_step": [round(x, 3) for x in e2e_each], "host_link": host_link,
                "a_upload": f"1/N row slab per rank, slabs exchanged over NVLink by {slab_mode}" if sharded_upload else "whole A",
                "max_abs_rel_vs_device_run": e2e_err, "bytes_equal_to_device_run_on_one_variant": e2e_bytes_equal}

    try:
        line["e2e"] = measure_e2e()
    except Exception as exc:  # noqa: BLE001  (the device-timed value is still reported)
        line["e2e"] = {"value": None, "unit": "TFLOP/s", "error": f"{type(exc).__name__}: {exc}"[:300]}

    stage["name"] = "extra"
    if not args.no_extras:
        try:
            if not multi:
                line["extra"].update(extras_single_gpu(torch, hm, peaks))
            line["extra"]["mlp_block_2048x4096x11008"] = mlp_extra(torch, hm, dist, rank, world)
            if not multi:
                line["extra"]["mlp_shard_compute_one_gpu"] = mlp_shard_compute(torch, hm)
        except Exception as exc:  # noqa: BLE001
            line["extra"]["error"] = f"{type(exc).__name__}: {exc}"[:300]

    stage["name"] = "cpu_baseline"
    if rank == 0 and not multi and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline()

    stage["name"] = "final barrier"
    if multi:
        dist.barrier()
    watchdog.cancel()
    write_line()
    if multi:
        # The line is out; tear down, but never let a stuck teardown hold the launcher.
        threading.Timer(60.0, lambda: os._exit(0)).start()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        os._exit(0)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--case", default="", help="run one case of `extra` only (profiling captures): gemm_f16_1024, "
                                               "gemm_f16_4096, gemm_f16_8192, kloop, gemm_i8, softmax, rmsnorm, swiglu, w8a16, attention_f16_4x16x4096x64, ...")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--reference-seconds", type=float, default=40.0,
                    help="--impl reference: CPU seconds to spend over all passes (the slab of A is sized to it)")
    ap.add_argument("--stage-limit", type=float, default=420.0,
                    help="seconds the stages after the device-timed loop may take together before the line is "
                         "written without the unfinished ones")
    ap.add_argument("--min-time", type=float, default=2.0,
                    help="seconds the timed GEMM loop is kept running for the long-run value (0: skip)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.gpus > 1 and "RANK" not in os.environ:
        raise SystemExit("bench.py --gpus N>1 must be launched with torch.distributed.run")
    return run_product_arm(args)


if __name__ == "__main__":
    sys.exit(main())
