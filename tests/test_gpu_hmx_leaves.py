"""The 29 engine / layout leaves of seam 2 (HMXAPI.h:53-293) on device addresses, driven the way the
reference's generated code drives them — one tile, one row pair or one bulk run per call — and
checked against the oracle's layout functions (which the CPU suite pins byte for byte to the
reference's own compiled HMXLayout.c) and against `oracle.gemm_f16` for the engine."""
import numpy as np
import pytest

from conftest import philox

pytestmark = pytest.mark.gpu


@pytest.fixture()
def L(hm, cuda):
    hm.init(0)
    lib = hm._capi.lib()

    class Leaves:
        def __getattr__(self, name):
            fn = getattr(lib, name)

            def call(*args):
                fn(*[a.data_ptr() if hasattr(a, "data_ptr") else int(a) for a in args])
                hm._capi.check()
            return call
    return Leaves()


def rounded(oracle, x):
    """The fp16 matrix the f32 packs see: "+0.0", then round to nearest even (the oracle's pinned rule)."""
    x = np.ascontiguousarray(x)
    return oracle.f32_pack_rounding(x).view(np.float16).reshape(x.shape)


def dev(cuda, a):
    return cuda.from_numpy(np.ascontiguousarray(a)).cuda()


def leaf_names():
    import re, os
    text = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "b200mlir_capi.h")).read()
    return sorted(set(re.findall(r"B200_API void (hmx_\w+)\(", text)))


def test_all_29_leaf_names_are_exported(hm):
    names = leaf_names()
    assert len(names) == 29
    lib = hm._capi.lib()
    assert all(hasattr(lib, n) for n in names)


@pytest.mark.parametrize("rows,cols,pad", [(64, 96, 0), (70, 45, 3), (33, 32, 0)])
def test_pack_leaves_tile_by_tile(hm, oracle, cuda, L, rows, cols, pad):
    """act / weight, f16 / f32, single / bulk / transposed / tail forms: every tile the calls write
    equals the oracle's image of the same matrix (zero fill at the ragged edges included)."""
    rng = philox(70)
    stride = cols + pad
    src = rng.uniform(-4, 4, (rows, stride)).astype(np.float32)
    src[0, 0] = -0.0
    s16 = src.astype(np.float16)
    s32 = s16.astype(np.float32) + rng.uniform(-1e-4, 1e-4, src.shape).astype(np.float32)  # not fp16-representable
    want16 = oracle.pack_act_f16(np.ascontiguousarray(s16[:, :cols]))
    want32 = oracle.pack_act_f16(rounded(oracle, s32[:, :cols]))
    mt, kt = (rows + 31) // 32, (cols + 31) // 32
    d16, d32 = dev(cuda, s16), dev(cuda, s32)
    # activation order [Mt, Kt]: single tiles, then one bulk call per row tile
    out = cuda.zeros(mt * kt * 1024, dtype=cuda.float16, device="cuda")
    for tr in range(mt):
        for tc in range(kt):
            L.hmx_pack_act_f16(out[(tr * kt + tc) * 1024:], d16, rows, cols, stride, tr, tc)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want16.view(np.uint16).ravel())
    out.zero_()
    for tr in range(mt):
        L.hmx_pack_act_f16_bulk(out[tr * kt * 1024:], d16, rows, cols, stride, tr, 0, kt)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want16.view(np.uint16).ravel())
    out.zero_()
    for tr in range(mt):
        L.hmx_pack_act_f32_bulk(out[tr * kt * 1024:], d32, rows, cols, stride, tr, 0, kt)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want32.view(np.uint16).ravel())
    out.zero_()
    for tr in range(mt):
        for tc in range(kt):
            L.hmx_pack_act_f32(out[(tr * kt + tc) * 1024:], d32, rows, cols, stride, tr, tc)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want32.view(np.uint16).ravel())
    # weight order [Nt, Kt] of a [K, N] = [rows, cols] matrix: bulk over k tiles per n tile
    wwant = oracle.pack_weight_f16(np.ascontiguousarray(s16[:, :cols]))
    nt, kkt = kt, mt
    for leaf, srcdev in (("hmx_pack_weight_f16", d16), ("hmx_pack_weight_f16_bulk", d16)):
        out.zero_()
        for n_t in range(nt):
            if leaf.endswith("bulk"):
                L.hmx_pack_weight_f16_bulk(out[n_t * kkt * 1024:], srcdev, rows, cols, stride, 0, n_t, kkt)
            else:
                for k_t in range(kkt):
                    L.hmx_pack_weight_f16(out[(n_t * kkt + k_t) * 1024:], srcdev, rows, cols, stride, k_t, n_t)
        assert np.array_equal(out.cpu().numpy().view(np.uint16), wwant.view(np.uint16).ravel()), leaf
    # transposed source: the [n][k] transpose input gives the same image
    t16 = dev(cuda, np.ascontiguousarray(s16[:, :cols].T))           # [cols(n), rows(k)]
    t32 = dev(cuda, np.ascontiguousarray(s32[:, :cols].T))
    want32w = oracle.pack_weight_f16(rounded(oracle, s32[:, :cols]))
    for leaf, srcdev, want in (("f16_T", t16, wwant), ("f32_T", t32, want32w)):
        out.zero_()
        for n_t in range(nt):
            getattr(L, f"hmx_pack_weight_{leaf}_bulk")(out[n_t * kkt * 1024:], srcdev, rows, cols, rows, 0, n_t, kkt)
        assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16).ravel()), leaf
        out.zero_()
        for n_t in range(nt):
            for k_t in range(kkt):
                getattr(L, f"hmx_pack_weight_{leaf}")(out[(n_t * kkt + k_t) * 1024:], srcdev, rows, cols, rows, k_t, n_t)
        assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16).ravel()), leaf
    # bounds-safe tails: only valid_rows x valid_cols of tile (0, 0) survive
    vr, vc = 5, 7
    clipped = np.zeros((32, 32), np.float16)
    clipped[:vr, :vc] = s16[:vr, :vc]
    twant = oracle.pack_act_f16(clipped)
    one = cuda.zeros(1024, dtype=cuda.float16, device="cuda")
    for name, args in (("hmx_pack_act_tail_f16", (d16, rows, cols, stride)), ("hmx_pack_weight_tail_f16", (d16, rows, cols, stride)),
                       ("hmx_pack_weight_tail_f16_T", (t16, rows, cols, rows))):
        one.fill_(9.0)
        if name.endswith("_T"):
            getattr(L, name)(one, *args, 0, 0, vr, vc)
        else:
            getattr(L, name)(one, *args, 0, 0, vr, vc)
        assert np.array_equal(one.cpu().numpy().view(np.uint16), twant.view(np.uint16).ravel()), name
    c32 = np.zeros((32, 32), np.float32)
    c32[:vr, :vc] = s32[:vr, :vc]
    t32want = oracle.pack_act_f16(rounded(oracle, c32))
    for name, args in (("hmx_pack_act_tail_f32", (d32, rows, cols, stride)), ("hmx_pack_weight_tail_f32", (d32, rows, cols, stride)),
                       ("hmx_pack_weight_tail_f32_T", (t32, rows, cols, rows))):
        one.fill_(9.0)
        getattr(L, name)(one, *args, 0, 0, vr, vc)
        assert np.array_equal(one.cpu().numpy().view(np.uint16), t32want.view(np.uint16).ravel()), name


def test_unpack_leaves(hm, oracle, cuda, L):
    """A [70, 100] read-out in an N-split destination (row stride 128): pair by pair, in bulk, with
    the fp32 widening and residual, and the bounds-safe single-tile forms."""
    rng = philox(71)
    rows, cols, stride = 70, 100, 128
    c = rng.uniform(-8, 8, (rows, cols)).astype(np.float16)
    tiles = oracle.pack_act_f16(c)                   # a read-out tile has the pack's image
    mt, nt = 3, 4
    dt = dev(cuda, tiles.view(np.float16))
    want = np.full((rows, stride), np.float16(7))
    want[:, :cols] = c
    out = cuda.full((rows, stride), 7.0, dtype=cuda.float16, device="cuda")
    for tr in range(mt):
        for j in range(16):
            L.hmx_unpack_acc_f16(out, dt[tr * nt * 1024:], rows, cols, stride, tr, j)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    out.fill_(7.0)
    for tr in range(mt):
        L.hmx_unpack_acc_f16_bulk(out, dt[tr * nt * 1024:], rows, cols, stride, tr, 16)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    # fp32 read-out: exact widening, optional residual with its own stride
    res = rng.normal(0, 1, (rows, 104)).astype(np.float32)
    dres = dev(cuda, res)
    o32 = cuda.full((rows, stride), 7.0, dtype=cuda.float32, device="cuda")
    for tr in range(mt):
        L.hmx_unpack_acc_f32_bulk(o32, dres, 1, dt[tr * nt * 1024:], rows, cols, stride, 104, tr, 16)
    w32 = np.full((rows, stride), np.float32(7))
    w32[:, :cols] = c.astype(np.float32) + res[:, :cols]
    assert np.array_equal(o32.cpu().numpy(), w32)
    o32.fill_(7.0)
    for tr in range(mt):
        for j in range(16):
            L.hmx_unpack_acc_f32(o32, 0, 0, dt[tr * nt * 1024:], rows, cols, stride, 0, tr, j)
    w32[:, :cols] = c.astype(np.float32)
    assert np.array_equal(o32.cpu().numpy(), w32)
    # tails: pair 2 of tile row 1, valid 5 x 9 -> only row 36 (= 32 + 4), columns 0..8
    out.fill_(7.0)
    L.hmx_unpack_acc_tail_f16(out, dt[1 * nt * 1024:], rows, cols, stride, 1, 2, 5, 9)
    w = np.full((rows, stride), np.float16(7))
    w[36, :9] = c[36, :9]
    assert np.array_equal(out.cpu().numpy().view(np.uint16), w.view(np.uint16))
    o32.fill_(7.0)
    L.hmx_unpack_acc_tail_f32(o32, dres, 1, dt[1 * nt * 1024:], rows, cols, stride, 104, 1, 2, 6, 9)
    w32 = np.full((rows, stride), np.float32(7))
    w32[36:38, :9] = c[36:38, :9].astype(np.float32) + res[36:38, :9]
    assert np.array_equal(o32.cpu().numpy(), w32)


def test_engine_leaves_compute_a_matmul(hm, oracle, cuda, L):
    """The generated loop nest of one matmul (docs of the partition pass: per (m, n) tile clear,
    mma over the K tiles, store, unpack): C[64, 96] = A[64, 128] . W[128, 96] through the leaves."""
    rng = philox(72)
    m, n, k = 64, 96, 128
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    w = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    da, dw = dev(cuda, a), dev(cuda, w)
    mt, nt, kt = m // 32, n // 32, k // 32
    act = cuda.zeros(mt * kt * 1024, dtype=cuda.float16, device="cuda")
    wt = cuda.zeros(nt * kt * 1024, dtype=cuda.float16, device="cuda")
    ar = cuda.zeros(mt * nt * 1024, dtype=cuda.float16, device="cuda")
    bias = cuda.zeros(64, dtype=cuda.int32, device="cuda")
    for tr in range(mt):
        L.hmx_pack_act_f16_bulk(act[tr * kt * 1024:], da, m, k, k, tr, 0, kt)
    for tn in range(nt):
        L.hmx_pack_weight_f16_bulk(wt[tn * kt * 1024:], dw, k, n, n, 0, tn, kt)
    L.hmx_bias_init_unit_f16(bias)
    assert bias.cpu().tolist() == [0x3C00] * 32 + [0] * 32
    L.hmx_bias_load_f16(bias, 0)
    for tr in range(mt):
        for tn in range(nt):
            L.hmx_acc_clear_f16()
            # two calls of two tiles each: the accumulator carries over between calls
            L.hmx_mma_f16(act[(tr * kt) * 1024:], wt[(tn * kt) * 1024:], 2)
            L.hmx_mma_f16(act[(tr * kt + 2) * 1024:], wt[(tn * kt + 2) * 1024:], 2)
            L.hmx_acc_store_f16(ar[(tr * nt + tn) * 1024:], 0)
    c = cuda.zeros((m, n), dtype=cuda.float16, device="cuda")
    for tr in range(mt):
        L.hmx_unpack_acc_f16_bulk(c, ar[tr * nt * 1024:], m, n, n, tr, 16)
    want = oracle.gemm_f16(a, w)
    got = c.cpu().numpy()
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 2.0 ** -10 * np.abs(want).max()
    assert (got.view(np.uint16) == want.view(np.uint16)).mean() > 0.99
    # the store cleared the accumulator: storing again gives zeros
    z = cuda.full((1024,), 3.0, dtype=cuda.float16, device="cuda")
    L.hmx_acc_store_f16(z, 0)
    assert float(z.abs().max()) == 0.0


def test_a_host_address_is_refused_not_dereferenced(hm, cuda):
    lib = hm._capi.lib()
    host = np.zeros(1024, np.float16)
    d = cuda.zeros(1024, dtype=cuda.float16, device="cuda")
    lib.hmx_pack_act_f16(d.data_ptr(), host.ctypes.data, 32, 32, 32, 0, 0)
    code, msg = hm._capi.last_error()
    assert code == 2 and "device address" in msg
    lib.hmx_mma_f16(0, d.data_ptr(), 1)
    assert hm._capi.last_error()[0] == 2
    assert hm.device_status() == 0
