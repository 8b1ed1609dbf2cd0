"""w8a16 GEMM, the MLP block and the runtime seam on the device, against the oracle."""
import ctypes

import numpy as np
import pytest

from conftest import max_abs_rel, philox

pytestmark = pytest.mark.gpu

TOL_GEMM = 1e-2


def c3_inputs(m, k=4096, n=11008):
    rng = philox(2)
    a = rng.normal(0, 1, (m, k)).astype(np.float16)
    wq = rng.integers(-127, 128, (k, n), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, n).astype(np.float16)
    return a, wq, s


@pytest.mark.parametrize("m", [1, 16, 256])
def test_w8a16_c3_config(hm, oracle, cuda, m):
    a, wq, s = c3_inputs(m)
    want = oracle.w8a16(a, wq, s)
    at, wt, st = (cuda.from_numpy(x).cuda() for x in (a, wq, s))
    ct = cuda.zeros((m, 11008), dtype=cuda.float16, device="cuda")
    hm.w8a16_matmul[(1,)](at, wt, st, ct)
    assert max_abs_rel(ct.cpu().numpy(), want) <= TOL_GEMM
    # second call uses the resident image; the row-major weight may even be gone
    wt.zero_()
    ct2 = cuda.zeros_like(ct)
    hm.w8a16_matmul[(1,)](at, wt, st, ct2)
    assert max_abs_rel(ct2.cpu().numpy(), want) <= TOL_GEMM
    hm.unregister_w8a16_weight(wt)


@pytest.mark.parametrize("mkn", [(1, 64, 40), (3, 16, 8), (17, 200, 264), (64, 1024, 96), (65, 96, 520)])
def test_w8a16_edge_shapes_host_buffers(hm, oracle, mkn):
    m, k, n = mkn
    rng = philox(50)
    a = rng.normal(0, 1, (m, k)).astype(np.float16)
    wq = rng.integers(-128, 128, (k, n), dtype=np.int8)  # includes -128
    s = rng.uniform(0.001, 0.02, n).astype(np.float16)
    c = np.zeros((m, n), np.float16)
    hm.w8a16_matmul[(1,)](a, wq, s, c, enableWeightResident=0)
    hm.set_option("enableWeightResident", 1)
    assert max_abs_rel(c, oracle.w8a16(a, wq, s)) <= TOL_GEMM


@pytest.mark.parametrize("mkn", [(16, 512, 32000), (40, 512, 20000), (70, 256, 20000), (200, 384, 1408), (128, 128, 2048),
                                 (3, 128, 2048), (16, 64, 4096)])
def test_w8a16_wide_ranges_row_passes_and_reproducibility(hm, oracle, cuda, mkn):
    """More than 128 channels per CTA (two channel passes), more than 128 rows (two row passes),
    K of one step, and every activation-tile width (16/64/128 rows): each CTA owns its channels
    for all of K and the ring slots have fixed owners, so repeated launches agree bit for bit —
    also right after a different kernel has run (a converter getting a ring turn ahead would
    show here as a run-to-run difference)."""
    m, k, n = mkn
    rng = philox(52)
    a = rng.normal(0, 1, (m, k)).astype(np.float16)
    wq = rng.integers(-127, 128, (k, n), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, n).astype(np.float16)
    want = oracle.w8a16(a, wq, s)
    at, wt, st = (cuda.from_numpy(x).cuda() for x in (a, wq, s))
    x = cuda.randn((1024, 1024), device="cuda").half()
    y = cuda.empty_like(x)
    outs = []
    for rep in range(4):
        if rep % 2:
            hm.softmax_kernel[(1,)](x, y)  # another kernel in between
        ct = cuda.full((m, n), 7.0, dtype=cuda.float16, device="cuda")
        hm.w8a16_matmul[(1,)](at, wt, st, ct)
        outs.append(ct.cpu().numpy())
    assert hm.device_status() == 0
    assert max_abs_rel(outs[0], want) <= TOL_GEMM
    for o in outs[1:]:
        assert np.array_equal(o.view(np.uint16), outs[0].view(np.uint16))
    hm.unregister_w8a16_weight(wt)


def test_w8a16_integer_core_is_exact(hm, oracle):
    """Unit scales and integer activations: fp32 accumulation of int8 products is exact."""
    rng = philox(51)
    a = rng.integers(-8, 9, (16, 512)).astype(np.float16)
    wq = rng.integers(-127, 128, (512, 256), dtype=np.int8)
    s = np.ones(256, np.float16)
    c = np.zeros((16, 256), np.float16)
    hm.w8a16_matmul[(1,)](a, wq, s, c, enableWeightResident=0)
    hm.set_option("enableWeightResident", 1)
    exact = a.astype(np.int32) @ wq.astype(np.int32)
    assert np.array_equal(c, exact.astype(np.float32).astype(np.float16))


@pytest.mark.parametrize("tdf", [(256, 512, 1408), (37, 256, 520), (8, 64, 128)])
def test_mlp_block_small(hm, oracle, tdf):
    t, d, f = tdf
    rng = philox(3)
    x = rng.normal(0, 1, (t, d)).astype(np.float16)
    gain = rng.uniform(0.5, 1.5, d).astype(np.float16)
    wg = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wu = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wd = rng.normal(0, 0.02, (f, d)).astype(np.float16)
    y = np.zeros_like(x)
    hm.mlp_block[(1,)](x, gain, wg, wu, wd, y, eps=1e-6, add_residual=True)
    assert hm.device_status() == 0
    assert max_abs_rel(y, oracle.mlp(x, gain, wg, wu, wd, 1e-6)) <= TOL_GEMM
    # tensor-parallel form: column-split gate/up, row-split down, sum of partials + residual
    parts = []
    for r in range(2):
        sl = slice(r * f // 2, (r + 1) * f // 2)
        p = np.zeros_like(x)
        hm.mlp_block[(1,)](x, gain, np.ascontiguousarray(wg[:, sl]), np.ascontiguousarray(wu[:, sl]),
                           np.ascontiguousarray(wd[sl]), p, eps=1e-6, add_residual=False)
        parts.append(p.astype(np.float32))
    tp = (parts[0] + parts[1]).astype(np.float16)
    tp = (tp.astype(np.float32) + x.astype(np.float32)).astype(np.float16)
    assert max_abs_rel(tp, oracle.mlp(x, gain, wg, wu, wd, 1e-6)) <= TOL_GEMM


def test_mlp_block_c4_config(hm, oracle, cuda):
    """2048 tokens x 4096, ffn 11008, N(0,1) inputs, N(0,0.02) weights, gain 1, eps 1e-6, seed 3."""
    rng = philox(3)
    t, d, f = 2048, 4096, 11008
    x = rng.normal(0, 1, (t, d)).astype(np.float16)
    gain = np.ones(d, np.float16)
    wg = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wu = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wd = rng.normal(0, 0.02, (f, d)).astype(np.float16)
    dev = [cuda.from_numpy(v).cuda() for v in (x, gain, wg, wu, wd)]
    y = cuda.zeros((t, d), dtype=cuda.float16, device="cuda")
    hm.mlp_block[(1,)](*dev, y, eps=1e-6, add_residual=True)
    assert hm.device_status() == 0
    got = y.cpu().numpy()
    rows = np.sort(philox(99).choice(t, 96, replace=False))  # bounded oracle sample of tokens
    want = oracle.mlp(x[rows], gain, wg, wu, wd, 1e-6)
    assert max_abs_rel(got[rows], want) <= TOL_GEMM


def test_layout_images_match_reference_golden(hm, oracle):
    import os
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "layout_golden.npz"))
    for name, shape in [("w64x96", (64, 96)), ("w70x45", (70, 45)), ("w32x32", (32, 32)), ("w1x33", (1, 33))]:
        src = gold[f"{name}_src"].view(np.float16)
        assert np.array_equal(hm.pack_weight_f16(src), gold[f"{name}_weight_image"])
        assert np.array_equal(hm.pack_act_f16(src), gold[f"{name}_act_image"])
        assert np.array_equal(hm.unpack_acc_f16(gold[f"{name}_act_image"], *shape), gold[f"{name}_unpacked"])
    packer = hm.WeightPrepack()
    f = gold["f32_src"]
    with np.errstate(over="ignore"):
        img = np.frombuffer(packer.pack(f), np.uint16)
    assert np.array_equal(img, gold["f32_weight_image"])
    assert packer.pack(f) is packer.pack(f.copy())  # content-hash cache
    big = philox(60).uniform(-1, 1, (1024, 2048)).astype(np.float16)
    assert np.array_equal(hm.pack_weight_f16(big), oracle.pack_weight_f16(big))


def test_runtime_seam_on_device(hm, cuda):
    lib = hm._capi.lib()
    hm.init(0)
    assert lib.hexagon_runtime_resident_scope_enter_v2(0x1234, 0x5678) == 0
    p = lib.hexagon_runtime_alloc_1d(4096, 128, True)
    assert p and p % 128 == 0
    src = np.arange(1024, dtype=np.float32)
    dst = np.zeros_like(src)
    lib.hexagon_runtime_copy(p, src.ctypes.data, 4096, True, False)
    lib.hexagon_runtime_copy(dst.ctypes.data, p, 4096, False, True)
    assert np.array_equal(src, dst)
    # tile-pointer alias: entry i points at byte i*2048 of the source, and maps back to it
    tab = lib.hexagon_runtime_build_crouton(p, 4096)
    assert tab and lib.hexagon_runtime_get_contiguous_memref(tab) == p
    ptrs = np.zeros(2, np.uint64)
    lib.hexagon_runtime_copy(ptrs.ctypes.data, tab, 16, False, True)
    assert ptrs.tolist() == [p, p + 2048]
    assert lib.hexagon_runtime_build_crouton(p, 4000) is None and hm._capi.last_error()[0] == 2
    assert lib.hexagon_runtime_get_contiguous_memref(p) is None
    lib.hexagon_runtime_free_1d(tab)
    assert lib.hexagon_runtime_get_contiguous_memref(tab) is None
    lib.hexagon_runtime_free_1d(p)
    assert lib.hexagon_runtime_alloc_1d(0, 128, False) is None and hm._capi.last_error()[0] == 2
    # workspace residency: same (key, instance) -> same address; instances are separate
    w0 = lib.hexagon_runtime_workspace_resident_v2(77, 8192, 2048, 0)
    w1 = lib.hexagon_runtime_workspace_resident_v2(77, 8192, 2048, 1)
    assert w0 and w1 and w0 != w1 and w0 % 2048 == 0
    assert lib.hexagon_runtime_workspace_resident_v2(77, 8192, 2048, 0) == w0
    assert lib.hexagon_runtime_workspace_resident_v2(77, 4096, 2048, 0) is None  # descriptor mismatch
    assert lib.hexagon_runtime_workspace_resident_v2(78, 64, 3, 0) is None  # alignment not a power of two
    # weight residency: copied once, same address forever, source not re-read
    img = np.arange(2048, dtype=np.uint8)
    r0 = lib.hexagon_runtime_weight_resident_v2(img.ctypes.data, 2048, 2048)
    img[:] = 0
    r1 = lib.hexagon_runtime_weight_resident_v2(img.ctypes.data, 2048, 2048)
    assert r0 and r0 == r1
    back = np.zeros(2048, np.uint8)
    lib.hexagon_runtime_copy(back.ctypes.data, r0, 2048, False, True)
    assert np.array_equal(back, np.arange(2048, dtype=np.uint8))
    assert lib.hexagon_runtime_resident_free_v2(r0, 2048) == 0
    assert lib.hexagon_runtime_resident_free_v2(r0, 1024) == -1
    # 2-D asynchronous copy with tokens
    a = np.arange(64 * 48, dtype=np.uint8).reshape(64, 48)
    b = np.zeros((64, 32), np.uint8)
    st = ctypes.c_int(5)
    tok = lib.hexagon_runtime_dma2d_start(a.ctypes.data, 0, b.ctypes.data, 0, 32, 64, 48, 32, False, False,
                                          True, 0, ctypes.byref(st))
    assert tok != 0xFFFFFFFF and st.value == 0
    lib.hexagon_runtime_dma_wait(tok)
    assert np.array_equal(b, a[:, :32])
    tok = lib.hexagon_runtime_dma2d_start(a.ctypes.data, 0, b.ctypes.data, 0, 32, 64, 16, 32, False, False,
                                          True, 0, ctypes.byref(st))
    assert tok == 0xFFFFFFFF and st.value == -1
