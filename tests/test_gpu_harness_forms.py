"""The callers either side of one GEMM call: the multi-span form, the manifest the dispatcher
publishes, the timed section with its perf.txt, and tensor files written from device memory."""
import re

import numpy as np
import pytest

from conftest import philox

pytestmark = pytest.mark.gpu


def test_multispan_matmul(hm):
    """2048^3 in 4x4 spans of 512x512, torch.rand-like inputs, rel < 2e-3 against fp32
    (test_matmul_multispan.py:56-73,110-190).  The defect that test guards against (every span
    written to the top-left block) signs rel 0.97; each span is also checked on its own."""
    rng = philox(0)
    a = rng.uniform(0, 1, (2048, 2048)).astype(np.float16)
    b = rng.uniform(0, 1, (2048, 2048)).astype(np.float16)
    c = np.zeros((2048, 2048), np.float16)
    hm.manifest_reset()
    hm.multispan_matmul[(1,)](a, b, c, 2048, 2048, 2048, 512, 512, enableMultiThreading=True,
                              enableVTCMTiling=True, enableConvertToHexagonmem=True,
                              enableHexagonmemCopyToDMA=True)
    ref = a.astype(np.float32) @ b.astype(np.float32)
    rel = np.linalg.norm(c.astype(np.float32) - ref) / np.linalg.norm(ref)
    assert rel < 2e-3
    for m0 in range(0, 2048, 512):
        for n0 in range(0, 2048, 512):
            blk, want = c[m0:m0 + 512, n0:n0 + 512].astype(np.float32), ref[m0:m0 + 512, n0:n0 + 512]
            assert np.linalg.norm(blk - want) / np.linalg.norm(want) < 2e-3, (m0, n0)
    plans = [(r["plan"], r["reason"]) for r in hm.manifest()["matmuls"]]
    assert plans == [("full-hmx", "selected-aligned")]  # the plan the reference test asserts


def test_manifest_vocabulary(hm):
    rng = philox(50)
    hm.manifest_reset()

    def run(m, n, k, times=1):
        a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
        b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
        c = np.zeros((m, n), np.float16)
        for _ in range(times):
            hm.matmul[(1,)](a, b, c)

    run(512, 512, 512, times=3)
    run(300, 520, 200)
    run(1, 64, 64)
    run(33, 45, 70)
    rows = {tuple(r["shape_mnk"]): r for r in hm.manifest()["matmuls"]}
    assert (rows[(512, 512, 512)]["plan"], rows[(512, 512, 512)]["reason"]) == ("full-hmx", "selected-aligned")
    assert rows[(512, 512, 512)]["launches"] == 3
    assert (rows[(300, 520, 200)]["plan"], rows[(300, 520, 200)]["reason"]) == ("hmx-tail", "selected-tail")
    assert (rows[(1, 64, 64)]["plan"], rows[(1, 64, 64)]["reason"]) == ("hvx", "min-rows")
    assert (rows[(33, 45, 70)]["plan"], rows[(33, 45, 70)]["reason"]) == ("hvx", "tile-alignment")
    canonical = {"selected-aligned", "selected-tail", "library-call", "vtcm-allocator-disabled", "non-rank-2",
                 "dynamic-shape", "unsupported-dtype", "min-rows", "tile-alignment", "unsupported-layout",
                 "vtcm-budget"}  # HmxManifest.h:88-111
    assert all(r["reason"] in canonical and r["plan"] in {"full-hmx", "hmx-tail", "hvx"} for r in rows.values())
    hm.set_option("gemmVariant", 99)
    try:
        hm.manifest_reset()
        run(512, 512, 512)
        (row,) = hm.manifest()["matmuls"]
        assert (row["plan"], row["reason"]) == ("hvx", "library-call")
    finally:
        hm.set_option("gemmVariant", -1)


def test_benchmark_report_writes_perf_txt(hm, cuda, tmp_path):
    x = cuda.randn((4096, 1024), device="cuda").half()
    y = cuda.empty_like(x)
    p = tmp_path / "perf.txt"
    us, cycles = hm.benchmark_report(lambda: hm.softmax_kernel[(1,)](x, y), 20, "softmax_kernel", p)
    text = p.read_text()
    m = re.fullmatch(r"Test_Info: \{\n\tName:softmax_kernel\n\tResult:Pass\n\tPerf:([0-9.]+)\n\tUnits:us\n\}\n"
                     r"PerfPcycles:([0-9]+)\n", text)
    assert m, text
    assert abs(float(m.group(1)) - us) < 1e-3 and int(m.group(2)) == cycles
    assert 1.0 < us < 1000.0
    # cycles / time must be a plausible SM clock (0.3 .. 2.2 GHz)
    assert 300.0 < cycles / us < 2200.0


def test_tensor_dump_from_device_memory(hm, cuda, tmp_path):
    t = cuda.arange(0, 4096, device="cuda").reshape(64, 64).half()
    p = tmp_path / "t.bin"
    hm.tensor_dump(p, t)
    back = hm.tensor_load(p)
    assert back.dtype == np.float16 and np.array_equal(back, t.cpu().numpy())
    dst = cuda.zeros((64, 64), dtype=cuda.float16, device="cuda")
    hm.tensor_load(p, out=dst)
    assert bool((dst == t).all())


@pytest.mark.parametrize("dist,p0,p1,dtype", [(0, -1.0, 1.0, np.float16), (1, 0.0, 3.0, np.float16),
                                              (1, 0.0, 0.02, np.float16), (2, -127, 127, np.int8),
                                              (0, 0.001, 0.02, np.float16), (1, 0.0, 1.0, np.float32)])
def test_device_generator_gives_the_oracles_bytes(hm, oracle, cuda, dist, p0, p1, dtype):
    """One counter-based generator, three implementations: the library's kernel must write the bytes
    the C++ loop beside the oracle writes (device tensor and host tensor alike)."""
    tdt = {np.float16: cuda.float16, np.float32: cuda.float32, np.int8: cuda.int8}[dtype]
    t = cuda.empty((1031, 517), dtype=tdt, device="cuda")
    hm.fill_random(t, 4, dist, p0, p1)
    want = oracle.fill_random((1031, 517), dtype, 4, dist, p0, p1)
    assert np.array_equal(t.cpu().numpy().view(np.uint8), want.view(np.uint8))
    h = np.empty((33, 7), dtype)
    hm.fill_random(h, 9, dist, p0, p1)
    assert np.array_equal(h.view(np.uint8), oracle.fill_random((33, 7), dtype, 9, dist, p0, p1).view(np.uint8))


def test_a_bounded_device_wait_runs_out_and_the_library_recovers(hm, oracle):
    """A one-CTA kernel waits about a millisecond on a barrier nothing arrives at: the wait gives up,
    the kernel returns, the host reads B200MLIR_ERR_DEVICE_WAIT with the site code, the status word
    is clean afterwards and a normal GEMM then passes.  (Refusal with a status word instead of a
    hang: bin/runtime/include/RuntimeDMA.h:19-37 of the reference.)"""
    assert hm.device_status() == 0
    hm.selftest_bounded_wait(1000)
    assert hm.device_status() == 90                    # the self-test's site code
    code, msg = hm._capi.last_error()
    assert code == 5 and "site 90" in msg and "detail 7" in msg
    assert hm.device_status() == 0                     # reading it cleared it
    rng = np.random.Generator(np.random.Philox(7))
    a = rng.uniform(-1, 1, (256, 512)).astype(np.float16)
    b = rng.uniform(-1, 1, (512, 256)).astype(np.float16)
    c = np.zeros((256, 256), np.float16)
    hm.matmul[(1,)](a, b, c)
    assert hm.device_status() == 0
    want = oracle.gemm_f16(a, b).astype(np.float32)
    assert np.abs(c.astype(np.float32) - want).max() / np.abs(want).max() <= 1e-2
    with pytest.raises(hm.B200Error):
        hm.selftest_bounded_wait(0)
