#!/usr/bin/env python
"""Benchmark of the hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload: the large fp16 GEMM M=16384, N=16384, K=8192 (fp32
accumulate, U[-1,1] inputs, seed 4), N-sharded over the ranks — one step is one
pass of that GEMM; `value` is whole-job TFLOP/s with inputs resident in HBM.
`e2e` is the same metric through the C-ABI kernel entry point with pinned HOST
buffers (copies inside the timed region).  `extra` carries the other configs
(1024^3 and 4096^3 GEMM, softmax GB/s, w8a16 GB/s, MLP tokens/s).
`--impl reference` times the CPU restatement of the reference's lowering on the
host cores on a bounded sample of the same workload.
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

# dram__bytes_read.sum + dram__bytes_write.sum of the 16384x16384x8192 launch (one ncu capture)
HEADLINE_DRAM_BYTES_PER_LAUNCH = 8.371e9 + 0.532e9


def cpu_gemm_sample(target_s: float = 12.0):
    """Times the CPU restatement on a slab of M rows (full N, K) sized to about target_s."""
    import oracle
    threads = oracle.hw_threads()
    rng = np.random.Generator(np.random.Philox(4))
    b = rng.uniform(-1, 1, (K, N)).astype(np.float16)

    def once(rows):
        a = rng.uniform(-1, 1, (rows, K)).astype(np.float16)
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
    a = rng.uniform(-1, 1, (max(rows, threads), K)).astype(np.float16)
    return a, b, a.shape[0], threads


def cpu_time_once(a, b, threads):
    import oracle
    t0 = time.perf_counter()
    oracle.gemm_f16(a, b, threads=threads)
    return time.perf_counter() - t0


def cpu_baseline(target_s: float = 12.0):
    a, b, rows, threads = cpu_gemm_sample(target_s)
    dt = cpu_time_once(a, b, threads)
    tflops = 2.0 * rows * N * K / dt / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{rows} of {M} rows of A (full N={N}, K={K}), one pass, {dt:.2f} s; "
                      f"whole-problem time extrapolates linearly to {dt * M / rows:.0f} s"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    a, b, rows, threads = cpu_gemm_sample(target_s=max(2.0, 40.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_time_once(a, b, threads)
    times = [cpu_time_once(a, b, threads) for _ in range(args.steps)]
    dt = sum(times) / len(times)
    tflops = 2.0 * rows * N * K / dt / 1e12
    sample = f"{rows} of {M} rows of A per step (full N={N}, K={K}); CPU restatement of the reference lowering"
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
        return only is None or name.startswith(only)

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
        out["softmax_f16_4096x1024"] = {"us": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}
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
        out["rmsnorm_f16_2048x4096"] = {"us": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}
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
            bytes_ = k * n + 2 * n + 2 * mrows * k + 2 * mrows * n
            gbs = bytes_ / (ms * 1e-3) / 1e9
            out[f"w8a16_m{mrows}_4096x11008"] = {
                "us": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                "us_weight_in_l2": ms_hot * 1e3, "tflops": 2.0 * mrows * k * n / (ms * 1e-3) / 1e12}
        for wq_ in Wq:
            hm.unregister_w8a16_weight(wq_)
        del Wq
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
    """C4: Llama MLP block, 2048 tokens x 4096, ffn 11008, tensor-parallel over the ranks."""
    from hexagon_mlir_b200 import tp
    t, d, f = 2048, 4096, 11008
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((t, d), generator=g, device="cuda").half()
    gain = torch.ones(d, dtype=torch.float16, device="cuda")
    lo, hi = tp.shard_bounds(f, rank, world)
    g2 = torch.Generator(device="cuda").manual_seed(300 + rank)
    wg = (torch.randn((d, hi - lo), generator=g2, device="cuda") * 0.02).half()
    wu = (torch.randn((d, hi - lo), generator=g2, device="cuda") * 0.02).half()
    wd = (torch.randn((hi - lo, d), generator=g2, device="cuda") * 0.02).half()
    out = torch.empty_like(x)
    block = tp.TensorParallelMLP(gain, wg, wu, wd, eps=1e-6, group=dist.group.WORLD if world > 1 else None)

    def step():
        block(x, out)
    mode = "eager"
    if world > 1:
        try:
            block.captured(x, out)

            def step():
                block.captured(x, out)
            mode = "cuda-graph"
        except Exception as exc:  # capture of the collective is an optimisation, not a requirement
            mode = f"eager ({type(exc).__name__})"
    ms = timed(torch, step, 20, 5, dist if world > 1 else None)
    flops = 6.0 * t * d * f
    block.release()  # the captured graph holds NCCL work: drop it before the process group goes
    reduction = "nccl all-reduce" if world > 1 else "none"
    forms = {}
    if world > 1:
        # the same block with the reduction fused into the kernels (peer stores over NVLink)
        forms["nccl_all_reduce_ms"] = ms
        try:
            fused = tp.FusedTensorParallelMLP(gain, wg, wu, wd, tokens=t, eps=1e-6, group=dist.group.WORLD)
            fms = timed(torch, lambda: fused(x), 20, 5, dist)
            fmode = "eager"
            try:
                fused.captured(x)
                gms = timed(torch, lambda: fused.captured(x), 20, 5, dist)
                if gms < fms:
                    fms, fmode = gms, "cuda-graph"
            except Exception:  # capture of the symmetric-memory barriers is an optimisation only
                pass
            fused.release()
            forms["fused_peer_store_ms"] = fms
            forms["fused_launch"] = fmode
            if fms < ms:
                ms, reduction, mode = fms, "fused: read-out pushes partial rows to their owners", fmode
        except Exception as exc:  # symmetric memory is a property of the box, not of this code
            forms["fused_peer_store_ms"] = f"unavailable ({type(exc).__name__})"
    return {"ms": ms, "reduction": reduction, **forms, "tokens_per_s": t / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
            "parallelism": f"tp{world}", "allreduce_bytes": t * d * 2 if world > 1 else 0, "launch": mode}


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
        line = json.dumps({"case": args.case, "result": extras_single_gpu(torch, hm, peaks, only=args.case)})
        os.write(json_fd, (line + "\n").encode())
        return 0

    # inputs resident in HBM: A replicated, this rank's column block of B and C
    n_lo, n_hi = rank * N // world, (rank + 1) * N // world
    n_loc = n_hi - n_lo
    g = torch.Generator(device="cuda").manual_seed(4)
    a = (torch.rand((M, K), generator=g, device="cuda") * 2 - 1).half()
    gb = torch.Generator(device="cuda").manual_seed(40 + rank)
    b = (torch.rand((K, n_loc), generator=gb, device="cuda") * 2 - 1).half()
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

    # sampled parity of the timed result against the CUDA-core path on 64 random tiles is in
    # the test-suite; here only a checksum guard that the kernel wrote something sane
    if not bool(torch.isfinite(c[:256, :256].float()).all()):
        raise SystemExit("bench.py: non-finite output")

    # e2e: same GEMM through the kernel entry point with pinned host buffers
    e2e_steps = max(1, min(2, args.steps))
    ha = torch.empty((M, K), dtype=torch.float16).pin_memory()
    hb = torch.empty((K, n_loc), dtype=torch.float16).pin_memory()
    hc = torch.empty((M, n_loc), dtype=torch.float16).pin_memory()
    ha.copy_(a)
    hb.copy_(b)
    torch.cuda.synchronize()
    npa, npb, npc = ha.numpy(), hb.numpy(), hc.numpy()

    def e2e_step():
        hm.matmul[(1,)](npa, npb, npc)  # H2D A and B, GEMM, D2H C, wait — all inside the call
    e2e_ms = timed(torch, e2e_step, e2e_steps, 1, dist if multi else None)
    e2e_tflops = FLOPS / (e2e_ms * 1e-3) / 1e12
    e2e_ok = bool(torch.equal(hc[:128].cuda(), c[:128]))
    del ha, hb, hc

    extra = {}
    if not args.no_extras:
        if not multi:
            extra.update(extras_single_gpu(torch, hm, peaks))
        extra["mlp_block_2048x4096x11008"] = mlp_extra(torch, hm, dist, rank, world)

    cpu = None
    if rank == 0 and not multi and not args.no_cpu:
        cpu = cpu_baseline()

    if multi:
        dist.barrier()
    if rank == 0:
        peak = peaks["bf16_tflops"]
        line = {
            "metric": "gemm_f16_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sharding": f"N split over {world} rank(s), A replicated, no collective",
                       "l2": "inputs larger than L2 (A 268 MB per rank)", "variant": plan["name"],
                       "accumulate": "fp32 in TMEM, one fp16 rounding"},
            "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": peak, "unit": "TFLOP/s",
                         "frac": kernel_tflops / peak,
                         # DRAM read + write bytes of one whole-problem launch (ncu capture summarised in
                         # profiles/bench_gemm_16384x16384x8192_launches.md); not captured for the shards at N > 1
                         "traffic": HEADLINE_DRAM_BYTES_PER_LAUNCH if world == 1 else None,
                         "peak_source": f"{peak_kind} cuBLAS bf16 burst; sustained {peaks.get('bf16_tflops_sustained')}",
                         "frac_of_sustained": kernel_tflops / peaks.get("bf16_tflops_sustained", peak),
                         "frac_of_nominal_2250": kernel_tflops / 2250.0,
                         "algorithmic_flops_per_launch": 2.0 * M * n_loc * K},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": (M * K + K * n_loc) * 2 * world,
                    "d2h_bytes_per_step": M * n_loc * 2 * world, "steps": e2e_steps, "matches_device_run": e2e_ok},
            "gpu_launches": int(launches), "clocks": clocks, "extra": extra,
        }
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if multi:
        # The line is out; tear down, but never let a stuck teardown hold the launcher.
        import threading
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
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.gpus > 1 and "RANK" not in os.environ:
        raise SystemExit("bench.py --gpus N>1 must be launched with torch.distributed.run")
    return run_product_arm(args)


if __name__ == "__main__":
    sys.exit(main())
