"""The oracle against the reference's own outputs (committed golden fixtures) and
against the closed-form rules its contract tests state.  CPU only."""
import os

import numpy as np
import pytest

from conftest import philox

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def layout_gold():
    return np.load(os.path.join(GOLD, "layout_golden.npz"))


def closed_form_tile(block):
    """lane_byte(r,c) = 128*(r>>1) + 4*c + 2*(r&1)
    (bin/runtime/test/test_hmx_layout_permutation_contract.py:137-148 of the reference)."""
    out = np.zeros(1024, np.uint16)
    for r in range(32):
        for c in range(32):
            out[(128 * (r >> 1) + 4 * c + 2 * (r & 1)) // 2] = block[r, c]
    return out


@pytest.mark.parametrize("name,shape", [("w64x96", (64, 96)), ("w70x45", (70, 45)),
                                        ("w32x32", (32, 32)), ("w1x33", (1, 33))])
def test_pack_unpack_match_reference_leaves(oracle, layout_gold, name, shape):
    src = layout_gold[f"{name}_src"].view(np.float16)
    assert src.shape == shape
    assert np.array_equal(oracle.pack_weight_f16(src), layout_gold[f"{name}_weight_image"])
    assert np.array_equal(oracle.pack_act_f16(src), layout_gold[f"{name}_act_image"])
    tiles = layout_gold[f"{name}_act_image"]
    assert np.array_equal(oracle.unpack_acc_f16(tiles, *shape), layout_gold[f"{name}_unpacked"])
    # fp32 read-out with residual: widen exactly, add in fp32
    want = layout_gold[f"{name}_unpacked_f32_res"]
    got = src.astype(np.float32) + layout_gold[f"{name}_res"]
    assert np.array_equal(got, want)


def test_f32_pack_rounding_matches_reference(oracle, layout_gold):
    f = layout_gold["f32_src"]
    with np.errstate(over="ignore"):
        h = oracle.f32_pack_rounding(f).view(np.float16).reshape(f.shape)
    assert np.array_equal(oracle.pack_weight_f16(h), layout_gold["f32_weight_image"])
    assert h[0, 0].view(np.uint16) == 0  # -0.0 -> +0.0


def test_closed_form_rule_and_numpy_permute(oracle):
    rng = philox(7)
    w = rng.integers(0, 65535, (64, 96), dtype=np.uint16)
    img = oracle.pack_weight_f16(w.view(np.float16)).reshape(3, 2, 1024)  # [Nt, Kt, tile]
    for nt in range(3):
        for kt in range(2):
            blk = w[kt * 32:(kt + 1) * 32, nt * 32:(nt + 1) * 32]
            assert np.array_equal(img[nt, kt], closed_form_tile(blk))
    # the host packer's vectorised form (backend/hmx_weight_prepack.py:170-183)
    permuted = w.reshape(2, 16, 2, 3, 32).transpose(3, 0, 1, 4, 2).ravel()
    assert np.array_equal(permuted, img.ravel())


def test_gemm_whole_k_is_one_rounding(oracle):
    rng = philox(0)
    a = rng.uniform(-1, 1, (96, 160)).astype(np.float16)
    b = rng.uniform(-1, 1, (160, 72)).astype(np.float16)
    c = oracle.gemm_f16(a, b)
    ref64 = a.astype(np.float64) @ b.astype(np.float64)
    # fp32 accumulation error is far below half an fp16 ulp of these magnitudes almost everywhere
    diff = np.abs(c.astype(np.float64) - ref64)
    assert diff.max() <= 2.0 ** -11 * np.abs(ref64).max() * 1.01 + 1e-6
    # threads do not change the result
    assert np.array_equal(c, oracle.gemm_f16(a, b, threads=1))


def test_gemm_kloop_rounds_each_segment(oracle):
    rng = philox(3)
    a = rng.uniform(-1, 1, (64, 256)).astype(np.float16)
    b = rng.uniform(-1, 1, (256, 64)).astype(np.float16)
    got = oracle.gemm_f16(a, b, block_k=64)
    acc = np.zeros((64, 64), np.float32)
    for k0 in range(0, 256, 64):
        seg = oracle.gemm_f16(a[:, k0:k0 + 64], b[k0:k0 + 64])  # fp16 read-out of the segment
        acc += seg.astype(np.float32)
    assert np.array_equal(got, acc.astype(np.float16))
    # rel error signature of the clean K-looped form (test_matmul_kloop.py:66-68: rel < 2e-3)
    ref = a.astype(np.float32) @ b.astype(np.float32)
    rel = np.linalg.norm(got.astype(np.float32) - ref) / np.linalg.norm(ref)
    assert rel < 2e-3


def test_f32_readout_is_widened_fp16_plus_residual(oracle):
    rng = philox(4)
    a = rng.uniform(-1, 1, (40, 64)).astype(np.float16)
    b = rng.uniform(-1, 1, (64, 48)).astype(np.float16)
    r = rng.normal(0, 1, (40, 48)).astype(np.float32)
    c16 = oracle.gemm_f16(a, b)
    assert np.array_equal(oracle.gemm_f16_f32out(a, b), c16.astype(np.float32))
    assert np.array_equal(oracle.gemm_f16_f32out(a, b, r), c16.astype(np.float32) + r)


def test_gemm_i8_exact(oracle):
    rng = philox(5)
    a = rng.integers(-128, 128, (33, 70), dtype=np.int8)
    b = rng.integers(-128, 128, (70, 45), dtype=np.int8)
    assert np.array_equal(oracle.gemm_i8_i32(a, b), a.astype(np.int32) @ b.astype(np.int32))


def test_w8a16_definition(oracle):
    rng = philox(2)
    a = rng.normal(0, 1, (16, 128)).astype(np.float16)
    wq = rng.integers(-127, 128, (128, 96), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, 96).astype(np.float16)
    w16 = (wq.astype(np.float32) * s.astype(np.float32)[None, :]).astype(np.float16)
    assert np.array_equal(oracle.w8a16(a, wq, s), oracle.gemm_f16(a, w16))


def test_softmax_steps(oracle):
    """The four lowered steps (docs/tutorials/triton/softmax.md:167-219)."""
    rng = philox(1)
    x = rng.normal(0, 3, (64, 1024)).astype(np.float16)
    y = oracle.softmax(x)
    m = x.max(axis=1, keepdims=True)
    z = (x - m).astype(np.float16)
    e = np.exp(z.astype(np.float32)).astype(np.float16)
    s = e.astype(np.float32).sum(axis=1, keepdims=True, dtype=np.float32)
    want = (e.astype(np.float32) / s).astype(np.float16)
    # libm expf vs numpy exp and the summation order differ by at most an fp16 ulp
    assert np.abs(y.astype(np.float32) - want.astype(np.float32)).max() <= 2.0 ** -11
    ref = np.exp(x.astype(np.float64) - x.astype(np.float64).max(1, keepdims=True))
    ref /= ref.sum(1, keepdims=True)
    assert np.abs(y.astype(np.float64) - ref).max() < 1e-3  # test_softmax.py:27-28 ATOL_FP16
    x32 = x.astype(np.float32)
    assert np.abs(oracle.softmax(x32).astype(np.float64) - ref).max() < 1e-5  # ATOL_FP32


def test_rmsnorm_and_silu_against_definitions(oracle):
    rng = philox(6)
    x = rng.uniform(0, 1, (127, 513)).astype(np.float16)  # test_rms_norm.py:18-19
    g = rng.uniform(0, 1, 513).astype(np.float16)
    y = oracle.rmsnorm(x, g, 1e-5)
    x64 = x.astype(np.float64)
    ref = x64 / np.sqrt((x64 ** 2).mean(1, keepdims=True) + 1e-5) * g.astype(np.float64)
    assert np.abs(y.astype(np.float64) - ref).max() < 1e-2  # test_rms_norm.py:24
    v = rng.uniform(0, 1, 16384).astype(np.float16)
    s = oracle.silu(v)
    v64 = v.astype(np.float64)
    assert np.abs(s.astype(np.float64) - v64 / (1 + np.exp(-v64))).max() < 1e-2  # test_silu.py:18
    u = rng.normal(0, 1, 16384).astype(np.float16)
    assert np.array_equal(oracle.swiglu(v, u),
                          (s.astype(np.float32) * u.astype(np.float32)).astype(np.float16))


def test_mlp_is_the_composition(oracle):
    rng = philox(3)
    t, d, f = 24, 64, 160
    x = rng.normal(0, 1, (t, d)).astype(np.float16)
    gain = np.ones(d, np.float16)
    wg = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wu = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wd = rng.normal(0, 0.02, (f, d)).astype(np.float16)
    y = oracle.mlp(x, gain, wg, wu, wd, 1e-6)
    h = oracle.rmsnorm(x, gain, 1e-6)
    a = oracle.swiglu(oracle.gemm_f16(h, wg), oracle.gemm_f16(h, wu))
    want = oracle.add_f16(oracle.gemm_f16(a, wd), x)
    assert np.array_equal(y, want)
