"""fp16 GEMM through the C ABI against the oracle.  North-star tolerance: max-abs-rel 1e-2;
the tensor-core path accumulates in fp32 like the oracle, so the observed error is an fp16 ulp."""
import numpy as np
import pytest

from conftest import max_abs_rel, philox

pytestmark = pytest.mark.gpu

TOL_GEMM = 1e-2
SIMT = 99


def run_matmul(hm, a, b, variant=-1, kernel=None, **opts):
    c = np.full((a.shape[0], b.shape[1]), np.float16(7), np.float16)
    hm.set_option("gemmVariant", variant)
    try:
        (kernel or hm.matmul)[(1,)](a, b, c, **opts)
    finally:
        hm.set_option("gemmVariant", -1)
    assert hm.device_status() == 0
    return c


def n_variants(hm):
    return len(hm.gemm_variants())


@pytest.mark.parametrize("variant", [SIMT, 0, 1, 2, 3, 4, 5, -1])
def test_c1_config(hm, oracle, variant):
    """M=N=K=1024, U[-1,1], seed 0."""
    rng = philox(0)
    a = rng.uniform(-1, 1, (1024, 1024)).astype(np.float16)
    b = rng.uniform(-1, 1, (1024, 1024)).astype(np.float16)
    want = oracle.gemm_f16(a, b)
    got = run_matmul(hm, a, b, variant)
    assert max_abs_rel(got, want) <= TOL_GEMM
    rel = np.linalg.norm(got.astype(np.float32) - want.astype(np.float32)) / np.linalg.norm(want.astype(np.float32))
    assert rel < 2e-3  # test_matmul_kloop.py:66-68
    assert (got.view(np.uint16) != want.view(np.uint16)).mean() < 0.05  # fp32 sum order only


def test_reference_test_shape(hm, oracle):
    """1024x512x64, torch.rand inputs, atol 2e-1 (test_matmul.py:17-22,86-88)."""
    rng = philox(40)
    a = rng.uniform(0, 1, (1024, 64)).astype(np.float16)
    b = rng.uniform(0, 1, (64, 512)).astype(np.float16)
    got = run_matmul(hm, a, b, N_ROWS=1024, N_COLUMNS=512, N_INNER=64, enableMultiThreading=True,
                     enableVTCMTiling=True, enableConvertToHexagonmem=True, enableHexagonmemCopyToDMA=True)
    ref = a.astype(np.float32) @ b.astype(np.float32)
    assert np.abs(got.astype(np.float32) - ref).max() <= 2e-1
    assert max_abs_rel(got, oracle.gemm_f16(a, b)) <= TOL_GEMM


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("mnk", [(128, 256, 64), (128, 64, 128), (5, 8, 8), (129, 264, 72),
                                 (300, 520, 200), (256, 256, 4096), (1000, 1000, 1000),
                                 (64, 2048, 512), (2048, 64, 320)])
def test_tensor_core_variants_edge_shapes(hm, oracle, variant, mnk):
    m, n, k = mnk
    rng = philox(41)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    assert hm.gemm_variant_verdict(variant, m, n, k) == "ok"
    assert max_abs_rel(run_matmul(hm, a, b, variant), oracle.gemm_f16(a, b)) <= TOL_GEMM


@pytest.mark.parametrize("mnk", [(1, 64, 64), (4, 32, 32), (33, 45, 70), (31, 33, 1), (64, 63, 64),
                                 (127, 129, 130), (2, 11008, 512)])
def test_shapes_the_engine_refuses_take_the_vector_path(hm, oracle, mnk):
    m, n, k = mnk
    rng = philox(42)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    assert hm.gemm_explain(m, n, k)["plan"] == "cuda-core"
    assert max_abs_rel(run_matmul(hm, a, b), oracle.gemm_f16(a, b)) <= TOL_GEMM


def test_strided_views_and_device_tensors(hm, oracle, cuda):
    rng = philox(43)
    big_a = cuda.from_numpy(rng.uniform(-1, 1, (256, 640)).astype(np.float16)).cuda()
    big_b = cuda.from_numpy(rng.uniform(-1, 1, (512, 1024)).astype(np.float16)).cuda()
    big_c = cuda.full((256, 2048), 3.0, dtype=cuda.float16, device="cuda")
    a, b, c = big_a[:, :512], big_b[:, 256:768], big_c[:, 512:1024]
    hm.matmul[(1,)](a, b, c)
    want = oracle.gemm_f16(np.ascontiguousarray(a.cpu().numpy()), np.ascontiguousarray(b.cpu().numpy()))
    assert max_abs_rel(c.cpu().numpy(), want) <= TOL_GEMM
    assert float((big_c[:, :512] - 3).abs().max()) == 0 and float((big_c[:, 1024:] - 3).abs().max()) == 0


@pytest.mark.parametrize("block_k", [32, 64, 128])
def test_klooped_matmul(hm, oracle, block_k):
    """256x256x512 K-looped (test_matmul_kloop.py:66-68): fp16 read-out per segment."""
    rng = philox(44)
    a = rng.uniform(-1, 1, (256, 512)).astype(np.float16)
    b = rng.uniform(-1, 1, (512, 256)).astype(np.float16)
    got = run_matmul(hm, a, b, kernel=hm.klooped_matmul, BLOCK_K=block_k)
    want = oracle.gemm_f16(a, b, block_k=block_k)
    assert max_abs_rel(got, want) <= TOL_GEMM
    assert (got.view(np.uint16) != want.view(np.uint16)).mean() < 0.05


@pytest.mark.parametrize("mnk,block_k", [((1024, 1024, 1024), 64), ((512, 384, 1000), 128), ((300, 520, 456), 64),
                                         ((2048, 1024, 2048), 256), ((128, 128, 192), 192)])
def test_klooped_matmul_on_tensor_cores(hm, oracle, mnk, block_k):
    """Segments of whole 64-deep k-blocks run on tcgen05: one accumulator per segment, rounded to
    fp16 by the read-out warps, which keep the fp32 running sum (HMXLayout.c:880-901).  Same
    arithmetic as the CUDA-core path, so the two must agree bit for bit almost everywhere and
    both with the oracle."""
    m, n, k = mnk
    rng = philox(48)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    hm.manifest_reset()
    got = run_matmul(hm, a, b, kernel=hm.klooped_matmul, BLOCK_K=block_k)
    (row,) = hm.manifest()["matmuls"]
    assert row["epilogue"] == "kloop-f16" and row["plan"] in ("full-hmx", "hmx-tail"), row
    want = oracle.gemm_f16(a, b, block_k=block_k)
    assert max_abs_rel(got, want) <= TOL_GEMM
    assert (got.view(np.uint16) != want.view(np.uint16)).mean() < 0.05
    simt = run_matmul(hm, a, b, variant=SIMT, kernel=hm.klooped_matmul, BLOCK_K=block_k)
    assert (got.view(np.uint16) != simt.view(np.uint16)).mean() < 0.05
    # the whole-K product differs: the segment roundings are really applied
    if k // block_k >= 4:
        whole = oracle.gemm_f16(a, b)
        assert (got.view(np.uint16) != whole.view(np.uint16)).mean() > 0.05


@pytest.mark.parametrize("variant", [SIMT, 0, 3])
def test_f32_readout_with_residual(hm, oracle, variant):
    rng = philox(45)
    a = rng.uniform(-1, 1, (256, 192)).astype(np.float16)
    b = rng.uniform(-1, 1, (192, 384)).astype(np.float16)
    r = rng.normal(0, 1, (256, 384)).astype(np.float32)
    hm.set_option("gemmVariant", variant)
    try:
        c = np.zeros((256, 384), np.float32)
        hm.matmul_f32out(a, b, c)
        assert max_abs_rel(c, oracle.gemm_f16_f32out(a, b)) <= TOL_GEMM
        # the read-out is an fp16 image widened: every value is exactly an fp16 number
        assert np.array_equal(c, c.astype(np.float16).astype(np.float32))
        hm.matmul_f32out(a, b, c, r)
        assert max_abs_rel(c, oracle.gemm_f16_f32out(a, b, r)) <= TOL_GEMM
    finally:
        hm.set_option("gemmVariant", -1)


@pytest.mark.parametrize("mnk", [(33, 45, 70), (256, 512, 1024), (1, 8, 4096)])
def test_int8_accumulation_bit_exact(hm, oracle, mnk):
    m, n, k = mnk
    rng = philox(46)
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    c = np.zeros((m, n), np.int32)
    hm.matmul_i8[(1,)](a, b, c)
    assert np.array_equal(c, oracle.gemm_i8_i32(a, b))


@pytest.mark.parametrize("m,n,k", [(256, 512, 384), (128, 128, 4096), (1000, 1028, 2064), (64, 64, 64),
                                   (300, 132, 208), (2048, 2048, 2048), (2100, 2052, 1040)])
def test_matmul_i8_on_tensor_cores_is_exact(hm, oracle, cuda, m, n, k):
    """int8 x int8 -> int32 through tcgen05 kind::i8 (B transposed on the way): the exact sums,
    equal to the CUDA-core loop and to the oracle, full range operands (-128 included)."""
    rng = philox(41)
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    a[0, :] = -128
    b[:, 0] = -128  # the largest magnitude a sum can reach: k * 16384
    at, bt = cuda.from_numpy(a).cuda(), cuda.from_numpy(b).cuda()
    ct = cuda.zeros((m, n), dtype=cuda.int32, device="cuda")
    before = hm.launch_count()
    hm.matmul_i8[(1,)](at, bt, ct)
    assert hm.launch_count() - before == 2  # transpose + tensor-core kernel
    assert hm.device_status() == 0
    got = ct.cpu().numpy()
    want = a.astype(np.int32) @ b.astype(np.int32) if m * n * k > 2 ** 30 else oracle.gemm_i8_i32(a, b)
    assert np.array_equal(got, want)
    hm.set_option("gemmVariant", -2)  # the CUDA-core loop
    try:
        c2 = cuda.zeros_like(ct)
        hm.matmul_i8[(1,)](at, bt, c2)
    finally:
        hm.set_option("gemmVariant", -1)
    assert cuda.equal(ct, c2)


def test_empty_and_bad_shapes(hm):
    a = np.zeros((0, 64), np.float16)
    hm.matmul[(1,)](a, np.zeros((64, 32), np.float16), np.zeros((0, 32), np.float16))
    with pytest.raises(hm.B200Error):
        hm.matmul[(1,)](np.zeros((8, 16), np.float16), np.zeros((8, 16), np.float16), np.zeros((8, 16), np.float16))


def test_linearity_at_scale(hm, cuda):
    """Size-independent property at a large shape: (2A)·B == 2(A·B) exactly in fp16."""
    g = cuda.Generator(device="cuda").manual_seed(4)
    a = (cuda.rand((2048, 4096), generator=g, device="cuda") * 2 - 1).half()
    b = (cuda.rand((4096, 4096), generator=g, device="cuda") * 2 - 1).half()
    c1 = cuda.empty((2048, 4096), dtype=cuda.float16, device="cuda")
    c2 = cuda.empty_like(c1)
    hm.matmul[(1,)](a, b, c1)
    hm.matmul[(1,)](a * 2, b, c2)
    assert hm.device_status() == 0
    # scaling by two commutes with every rounding except where fp16(A·B) is subnormal
    normal = c1.abs() >= 2.0 ** -14
    assert bool(((c1 * 2 == c2) | ~normal).all())
    assert float(((c1.float() * 2 - c2.float()).abs() * (~normal)).max()) <= 2.0 ** -23
    assert float(normal.float().mean()) > 0.99


def test_autotune_on_device(hm):
    hm.autotune_cache_clear()
    rep = hm.gemm_autotune(1024, 1024, 1024)
    assert rep["round_verdict"] == "valid", rep
    assert rep["measured_configs"] == len(hm.gemm_variants()), rep
    assert rep["champion_variant"] >= 0 and rep["unmeasured"] == []
    assert hm.gemm_explain(1024, 1024, 1024)["reason"] == "autotune cache"
    again = hm.gemm_autotune(1024, 1024, 1024)
    assert again.get("cache_hit") is True
    hm.autotune_cache_clear()


@pytest.mark.parametrize("mnk,pad", [((4096, 4096, 4096), 0), ((4360, 4104, 4096), 0), ((4096, 4224, 4096), 64),
                                     ((12288, 1024, 4096), 0), ((1280, 9000, 4096), 0), ((9000, 2048, 4096), 64)])
def test_host_buffers_take_the_pipelined_path(hm, oracle, mnk, pad):
    """All three tensors in host memory and >= 96 MB: panels go up, blocks are computed and come
    back down concurrently.  Checked on sampled rows against the oracle and, bit for bit, against
    the same product computed from device-resident tensors."""
    import torch
    m, n, k = mnk
    rng = philox(47)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (k, n + pad)).astype(np.float16)[:, :n]   # a strided view when pad > 0
    c_full = np.full((m, n + pad), np.float16(7), np.float16)
    c = c_full[:, :n]
    hm.manifest_reset()
    hm.matmul[(1,)](a, b, c)
    assert hm.device_status() == 0
    assert all(tuple(r["shape_mnk"]) != (m, n, k) for r in hm.manifest()["matmuls"])  # strips: the pipelined path ran
    rows = rng.choice(m, 48, replace=False)
    want = oracle.gemm_f16(np.ascontiguousarray(a[rows]), np.ascontiguousarray(b))
    assert max_abs_rel(c[rows], want) <= TOL_GEMM
    if pad:
        assert (c_full[:, n:] == np.float16(7)).all()  # bytes between rows are untouched
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(np.ascontiguousarray(b)).cuda()
    dc = torch.empty((m, n), dtype=torch.float16, device="cuda")
    hm.matmul[(1,)](da, db, dc)
    # the strips and the whole problem may take different variants; where a variant cuts a tile's K
    # between SM pairs the fp32 sum is associated differently, which can move the last fp16 bit
    got_dev = dc.cpu().numpy()
    same = got_dev.view(np.uint16) == np.ascontiguousarray(c).view(np.uint16)
    assert same.mean() > 0.9
    assert np.abs(got_dev.astype(np.float32) - c.astype(np.float32)).max() <= 2 * 2.0 ** -10 * np.abs(got_dev).max()
    hm.set_option("gemmVariant", 3)      # one whole-tile variant for every strip and for the whole problem:
    try:                                 # the same fp32 sums in the same order, so the same bytes
        c2 = np.zeros((m, n), np.float16)
        hm.matmul[(1,)](a, b, c2)
        hm.matmul[(1,)](da, db, dc)
    finally:
        hm.set_option("gemmVariant", -1)
    assert np.array_equal(dc.cpu().numpy().view(np.uint16), c2.view(np.uint16))


STREAMK = 5


@pytest.mark.parametrize("mnk", [(1024, 1024, 1024), (256, 11008, 4096), (2048, 4096, 1376), (2048, 1376, 4096),
                                 (300, 520, 200), (512, 512, 8192), (256, 256, 64 * 148), (4096, 4096, 512)])
def test_stream_k_cuts_tiles_between_pairs_and_stays_exact_in_order(hm, oracle, cuda, mnk):
    """The k-blocks of all tiles dealt out evenly over the SM pairs: tiles cut between pairs are
    combined from fp32 partials in a fixed order, so the result matches the oracle like any other
    variant AND is bit-identical run to run (the reduction order is the partition's, not arrival's).
    Shapes: the first config, the many-row w8a16 product, both GEMMs of a TP8 MLP shard (one with
    a K tail), an odd shape, one tile cut 74 ways, K of exactly one block per pair, uncut tiles."""
    m, n, k = mnk
    rng = philox(61)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    assert hm.gemm_variant_verdict(STREAMK, m, n, k) == "ok"
    want = oracle.gemm_f16(a, b)
    da, db = cuda.from_numpy(a).cuda(), cuda.from_numpy(b).cuda()
    outs = []
    hm.set_option("gemmVariant", STREAMK)
    try:
        for _ in range(3):
            c = cuda.full((m, n), 7.0, dtype=cuda.float16, device="cuda")
            hm.matmul[(1,)](da, db, c)
            outs.append(c)
    finally:
        hm.set_option("gemmVariant", -1)
    assert hm.device_status() == 0
    assert max_abs_rel(outs[0].cpu().numpy(), want) <= TOL_GEMM
    assert cuda.equal(outs[0], outs[1]) and cuda.equal(outs[0], outs[2])
    # and close to the whole-tile pair kernel: only the fp32 summation order differs
    hm.set_option("gemmVariant", 3)
    try:
        c3 = cuda.empty((m, n), dtype=cuda.float16, device="cuda")
        hm.matmul[(1,)](da, db, c3)
    finally:
        hm.set_option("gemmVariant", -1)
    assert float((outs[0].float() - c3.float()).abs().max()) <= 2 * 2.0 ** -10 * max(1.0, float(c3.abs().max()))


def test_stream_k_read_outs(hm, oracle):
    """The fused read-outs behind a combined tile: fp32 + residual, and the MLP block's SwiGLU and
    residual forms (both GEMMs of the block forced onto the variant)."""
    rng = philox(62)
    a = rng.uniform(-1, 1, (320, 4096)).astype(np.float16)
    b = rng.uniform(-1, 1, (4096, 520)).astype(np.float16)
    res = rng.normal(0, 1, (320, 520)).astype(np.float32)
    c32 = np.zeros((320, 520), np.float32)
    hm.set_option("gemmVariant", STREAMK)
    try:
        hm.matmul_f32out(a, b, c32, res)
        want = oracle.gemm_f16_f32out(a, b, res)
        assert max_abs_rel(c32, want) <= TOL_GEMM
        t, d, f = 512, 1024, 1376
        x = rng.normal(0, 1, (t, d)).astype(np.float16)
        gain = rng.uniform(0.5, 1.5, d).astype(np.float16)
        wg = rng.normal(0, 0.02, (d, f)).astype(np.float16)
        wu = rng.normal(0, 0.02, (d, f)).astype(np.float16)
        wd = rng.normal(0, 0.02, (f, d)).astype(np.float16)
        y = np.zeros_like(x)
        hm.manifest_reset()
        hm.mlp_block[(1,)](x, gain, wg, wu, wd, y, eps=1e-6, add_residual=True)
        names = [r["name"] for r in hm.manifest()["matmuls"]]
    finally:
        hm.set_option("gemmVariant", -1)
    assert hm.device_status() == 0
    assert names and all("streamk" in nm for nm in names), names
    assert max_abs_rel(y, oracle.mlp(x, gain, wg, wu, wd, 1e-6)) <= TOL_GEMM

