"""Generates the committed golden fixtures from the reference itself.

Run where the reference checkout is available (its location: HEXMLIR_REFERENCE_ROOT):

    python tests/golden/make_golden.py

It (1) runs the reference's own layout leaves (HMXLayout.c, compiled by
oracle/Makefile target "ref") on seeded inputs and stores inputs + outputs, and
(2) imports the reference's stdlib-only backend/hmx_search.py and stores what
its search-loop functions return on scripted measurements, and (3) evaluates the
expected values of the reference's own device tests — the torch call each test
compares its kernel against, on that test's shapes — and stores inputs and
expectations.  The tests read the fixtures only; nothing at test time touches
the reference.  (4) runs the reference's flash-attention and online-softmax kernel
sources (test/python/triton/test_flash_attention.py, test_online_softmax.py) with
Triton's CPU interpreter on seeded inputs and stores inputs and outputs.
"""
import importlib.util
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("HEXMLIR_REFERENCE_ROOT") or sys.exit("set HEXMLIR_REFERENCE_ROOT to the reference checkout")

import oracle  # noqa: E402


def layout_fixture():
    oracle.build(with_ref=True)
    assert oracle.ref_lib() is not None, "reference layout leaves did not build"
    rng = np.random.Generator(np.random.Philox(1234))
    out = {}
    for name, (k, n) in {"w64x96": (64, 96), "w70x45": (70, 45), "w32x32": (32, 32),
                         "w1x33": (1, 33)}.items():
        w = rng.uniform(-4, 4, (k, n)).astype(np.float16)
        out[f"{name}_src"] = w.view(np.uint16)
        out[f"{name}_weight_image"] = oracle.ref_pack_weight_f16(w)
        out[f"{name}_act_image"] = oracle.ref_pack_act_f16(w)
        tiles = oracle.ref_pack_act_f16(w)
        out[f"{name}_unpacked"] = oracle.ref_unpack_acc_f16(tiles, k, n)
        res = rng.normal(0, 1, (k, n)).astype(np.float32)
        out[f"{name}_res"] = res
        out[f"{name}_unpacked_f32_res"] = oracle.ref_unpack_acc_f32(tiles, k, n, res)
    f = rng.normal(0, 100, (64, 64)).astype(np.float32)
    f[0, :8] = [-0.0, 0.0, 65504.0, 65520.0, 1e-8, -1e-8, 6.1e-5, 2049.0]
    out["f32_src"] = f
    with np.errstate(over="ignore"):
        out["f32_weight_image"] = oracle.ref_pack_weight_f32(f)
    np.savez_compressed(os.path.join(HERE, "layout_golden.npz"), **out)


def search_fixture():
    path = os.path.join(REF, "qcom_hexagon_backend", "backend", "hmx_search.py")
    spec = importlib.util.spec_from_file_location("ref_hmx_search", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_hmx_search"] = mod
    spec.loader.exec_module(mod)
    g = {}
    g["constants"] = dict(TILE_EDGE=mod.TILE_EDGE, MIN_ROWS=mod.MIN_ROWS,
                          CHAMPION_CV_FACTOR=mod.CHAMPION_CV_FACTOR,
                          CHAMPION_MARGIN_FLOOR=mod.CHAMPION_MARGIN_FLOOR)
    g["champion_gate"] = [[cv, mod.champion_gate(cv)] for cv in
                          [0.0, 0.01, 0.049, 0.05, 0.051, 0.1, 0.5, float("nan")]]
    g["quantile"] = [[s, q, mod._quantile(s, q)] for s in
                     ([1.0], [3.0, 1.0, 2.0], [10.0, 20.0, 40.0], [5.0, 7.0]) for q in (0.5, 0.2, 0.8)]
    g["calibration_iters"] = [[us, mod.calibration_iters(us)] for us in
                              [0.5, 1.0, 100.0, 2000.0, 1e6, 1e7]]
    g["tile_verdict"] = [[bm, bn, bk, mod.tile_verdict(bm, bn, bk)] for bm, bn, bk in
                         [(32, 32, 32), (4, 32, 32), (1, 32, 32), (64, 48, 32), (1024, 1024, 1024),
                          (2048, 1024, 1024), (1024, 1024, 2048), (512, 512, 512)]]
    g["span_count"] = [[m, n, k, list(t), mod.span_count(m, n, k, t)] for m, n, k, t in
                       [(1024, 1024, 1024, (128, 256, 64)), (1000, 1000, 1000, (128, 128, 64)),
                        (16384, 16384, 8192, (128, 256, 64))]]
    # canary verdicts
    def rec(q50, q20, q80):
        return {"q50_pcyc": q50, "q20_pcyc": q20, "q80_pcyc": q80}
    cases = {
        "missing": (None, None),
        "unmeasured": (rec(float("inf"), float("inf"), float("inf")), 100.0),
        "reference_established": (rec(100.0, 99.0, 101.0), None),
        "ok": (rec(105.0, 104.0, 106.0), 100.0),
        "drift": (rec(130.0, 129.0, 131.0), 100.0),
        "noisy_ok": (rec(130.0, 120.0, 140.0), 100.0),
    }
    g["canary"] = {}
    for name, (metrics, ref) in cases.items():
        v = mod.canary_verdict(metrics, ref)
        g["canary"][name] = {"metrics": metrics, "reference": ref, "status": v["status"],
                             "healthy": v["healthy"]}
    # champion rounds on scripted measurements; labels a/b/c stand for three
    # candidates visited in this order, "a" the control arm
    def rows(ts):
        return [dict(cfg=lbl, tiles=[i, 0, 0], q50_pcyc=t[0], q20_pcyc=t[1], q80_pcyc=t[2])
                for i, (lbl, t) in enumerate(zip("abc", ts))]
    rounds = {
        "control_keeps": [(100, 99, 101), (95, 94, 96), (90, 89, 91)],
        "clear_takeover": [(100, 99, 101), (80, 79, 81), (120, 119, 121)],
        "chain": [(100, 99, 101), (80, 79, 81), (60, 59, 61)],
        "noisy_blocks": [(100, 80, 120), (70, 69, 71), (200, 199, 201)],
        "exactly_on_gate": [(100, 100, 100), (85, 85, 85), (300, 300, 300)],
        "failed_candidate": [(100, 99, 101), (float("inf"),) * 3, (50, 49, 51)],
        "control_failed": [(float("inf"),) * 3, (80, 79, 81), (60, 59, 61)],
    }
    g["rounds"] = {}
    healthy = rec(100.0, 99.0, 101.0)
    for name, ts in rounds.items():
        r = mod.judge_champion_round(rows(ts), control="a", canary=healthy, canary_reference=100.0,
                                     iters=10)
        g["rounds"][name] = {
            "timings": [[None if x == float("inf") else x for x in t] for t in ts],
            "champion": r["champion"], "round_verdict": r["round_verdict"],
            "champion_significant": r["champion_significant"], "unmeasured": r["unmeasured"],
            "outcomes": [c["outcome"] for c in r["comparisons"]],
        }
    r = mod.judge_champion_round(rows(rounds["clear_takeover"]), control="a",
                                 canary=rec(150.0, 149.0, 151.0), canary_reference=100.0, iters=10)
    g["rounds"]["void_round"] = {
        "timings": [list(t) for t in rounds["clear_takeover"]], "champion": r["champion"],
        "round_verdict": r["round_verdict"], "champion_significant": r["champion_significant"],
        "unmeasured": r["unmeasured"], "outcomes": [c["outcome"] for c in r["comparisons"]],
        "canary": [150.0, 149.0, 151.0],
    }
    with open(os.path.join(HERE, "search_golden.json"), "w") as f:
        json.dump(g, f, indent=1, sort_keys=True)


def device_test_fixture():
    """What the reference's device tests expect of each kernel: same shapes and input
    distributions (torch.rand), the same torch call as the expected value.  The tolerance each
    test applies is recorded beside it.  Sources: test/python/triton/test_softmax.py:18-19,71,
    90-93; test_rms_norm.py:17-24,62-64,82-86; test_silu.py:18,21,51,68-69; test_matmul.py:17,
    69-70,87-88; test_matmul_kloop.py:60-69,100-103,153-158."""
    import torch
    out = {}
    # (the fp32 cases run on the widened fp16 inputs, so that each input is stored once)
    torch.manual_seed(11)
    x = torch.rand(128, 128, dtype=torch.float16)
    out["softmax_x"] = x.numpy()
    out["softmax_f16_expected"] = torch.nn.functional.softmax(x, dim=1, dtype=torch.float16).numpy()
    out["softmax_f32_expected"] = torch.nn.functional.softmax(x.float(), dim=1, dtype=torch.float32).numpy()
    torch.manual_seed(12)
    x = torch.rand(127, 513, dtype=torch.float16)
    w = torch.rand(513, dtype=torch.float16)
    out["rmsnorm_x"], out["rmsnorm_w"] = x.numpy(), w.numpy()
    out["rmsnorm_f16_expected"] = torch.nn.functional.rms_norm(x, (513,), weight=w, eps=1e-5).numpy()
    out["rmsnorm_f32_expected"] = torch.nn.functional.rms_norm(x.float(), (513,), weight=w.float(), eps=1e-5).numpy()
    torch.manual_seed(13)
    x = torch.rand(16384, dtype=torch.float16)
    out["silu_x"] = x.numpy()
    out["silu_f16_expected"] = torch.nn.functional.silu(x).numpy()
    out["silu_f32_expected"] = torch.nn.functional.silu(x.float()).numpy()
    torch.manual_seed(14)
    a = torch.rand((1024, 64), dtype=torch.float16)
    b = torch.rand((64, 512), dtype=torch.float16)
    out["matmul_a"], out["matmul_b"] = a.numpy(), b.numpy()
    out["matmul_expected_rows_0_4"] = torch.matmul(a, b).numpy()[0::4]  # every fourth row
    torch.manual_seed(0)  # the K-looped test seeds itself
    a = torch.rand((256, 512), dtype=torch.float16)
    b = torch.rand((512, 256), dtype=torch.float16)
    out["kloop_a"], out["kloop_b"] = a.numpy(), b.numpy()
    out["kloop_expected_f32"] = torch.matmul(a.float(), b.float()).numpy()
    out["tolerances"] = np.array(json.dumps({
        "softmax_f16_atol": 1e-3, "softmax_f32_atol": 1e-5, "rmsnorm_atol": 1e-2, "silu_atol": 1e-2,
        "matmul_atol": 2e-1, "kloop_rel": 2e-3, "kloop_block_k": 256}))
    np.savez_compressed(os.path.join(HERE, "device_tests_golden.npz"), **out)


def attention_fixture():
    """Outputs of the reference's own kernel sources, executed by Triton's interpreter (numpy on
    the CPU, every value fp32): attention_fwd_kernel (test_flash_attention.py:116-195) and
    online_softmax (test_online_softmax.py:27-77).  Inputs are torch.rand rounded to fp16 and
    stored as fp16, so that an implementation with fp16 operands starts from the same numbers."""
    os.environ["TRITON_INTERPRET"] = "1"
    assert "triton" not in sys.modules, "the interpreter switch is read when triton is imported"
    import torch

    def load(name):
        path = os.path.join(REF, "test", "python", "triton", name + ".py")
        src = open(path).read().replace("from .. import parameterize_func_name", "")
        mod = type(sys)("ref_" + name)
        mod.__file__ = path
        import linecache
        linecache.cache[path] = (len(src), None, src.splitlines(True), path)  # the jit reads sources
        exec(compile(src, path, "exec"), mod.__dict__)
        return mod

    fa = load("test_flash_attention")
    out = {}
    for tag, (n_ctx, block_n, seed) in {"a": (256, 64, 21), "b": (128, 32, 22)}.items():
        torch.manual_seed(seed)
        q, k, v = (torch.rand(1, 1, n_ctx, fa.D_HEAD).half() for _ in range(3))
        o = torch.zeros(1, 1, n_ctx, fa.D_HEAD)
        fa.attention_fwd_kernel[(1,)](
            pid1=0, Q=q.float(), K=k.float(), V=v.float(), sm_scale=fa.SCALE, Out=o, H=1, N_CTX=n_ctx,
            BLOCK_M=n_ctx, BLOCK_DMODEL=fa.D_HEAD, BLOCK_N=block_n, STAGE=fa.STAGE,
            stride_0=n_ctx * fa.D_HEAD, stride_1=n_ctx * fa.D_HEAD, stride_2=fa.D_HEAD, stride_3=1)
        out[f"attn_{tag}_q"], out[f"attn_{tag}_k"], out[f"attn_{tag}_v"] = q.numpy(), k.numpy(), v.numpy()
        out[f"attn_{tag}_out"] = o.numpy()
        out[f"attn_{tag}_block_n"] = np.array(block_n)
    out["attn_scale"] = np.array(fa.SCALE)
    out["attn_rel_tolerance"] = np.array(5e-3)  # test_flash_attention.py:248-249
    os_ = load("test_online_softmax")
    torch.manual_seed(23)
    rows, cols = os_.CONSTANTS["NUM_ROWS"], os_.CONSTANTS["NUM_COLS"]
    x = torch.rand(rows, cols)
    out["online_x"] = x.numpy()
    for threads in (1, 4):  # test_online_softmax.py:80-92: row and column blocks are rows/threads, cols/threads
        y = torch.empty_like(x)
        os_.online_softmax[(threads,)](x, y, NUM_ROWS=rows, NUM_COLS=cols, BLOCK_ROW_SIZE=rows // threads,
                                       BLOCK_COL_SIZE=cols // threads)
        out[f"online_y_threads{threads}"] = y.numpy()
    out["online_atol"] = np.array(os_.ATOL)
    np.savez_compressed(os.path.join(HERE, "attention_golden.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "attention":  # needs a process in which triton is not yet imported
        attention_fixture()
        sys.exit(0)
    layout_fixture()
    search_fixture()
    device_test_fixture()
    import subprocess
    subprocess.run([sys.executable, os.path.abspath(__file__), "attention"], check=True)
    print("wrote", sorted(os.listdir(HERE)))
