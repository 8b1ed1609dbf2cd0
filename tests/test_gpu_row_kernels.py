"""Row kernels through the C ABI against the oracle.  Tolerances: 1e-3 (softmax, RMSNorm,
stated by the north star) and the reference tests' own 1e-2 for SiLU."""
import numpy as np
import pytest

from conftest import max_abs_rel, philox

pytestmark = pytest.mark.gpu

TOL_ROW = 1e-3


def test_softmax_c2_config(hm, oracle, cuda):
    """[4096,1024] fp16, N(0,3), seed 1."""
    x = philox(1).normal(0, 3, (4096, 1024)).astype(np.float16)
    want = oracle.softmax(x)
    xt = cuda.from_numpy(x).cuda()
    yt = cuda.empty_like(xt)
    hm.softmax_kernel[(4,)](xt, yt, NUM_ROWS=4096, NUM_COLS=1024, BLOCK_SIZE=1024)
    got = yt.cpu().numpy()
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= TOL_ROW
    # same rounding points as the lowering: almost every element is bit-identical
    assert (got.view(np.uint16) != want.view(np.uint16)).mean() < 0.02
    assert np.abs(got.astype(np.float32).sum(1) - 1).max() < 4e-3


@pytest.mark.parametrize("shape", [(128, 128), (127, 513), (3, 8), (1, 1), (33, 2048), (5, 4096),
                                   (4, 8192), (2, 20000), (9, 1000)])
def test_softmax_shapes_host_buffers(hm, oracle, shape):
    x = philox(11).uniform(0, 1, shape).astype(np.float16) * 8
    y = np.zeros_like(x)
    hm.softmax_kernel[(1,)](x, y)
    assert np.abs(y.astype(np.float32) - oracle.softmax(x).astype(np.float32)).max() <= TOL_ROW


def test_softmax_f32_and_strided_rows(hm, oracle, cuda):
    x = philox(12).normal(0, 3, (128, 128)).astype(np.float32)
    y = np.zeros_like(x)
    hm.softmax_kernel[(1,)](x, y)
    assert np.abs(y - oracle.softmax(x)).max() <= 1e-5  # test_softmax.py:27 ATOL_FP32
    wide = cuda.from_numpy(philox(13).normal(0, 2, (64, 512)).astype(np.float16)).cuda()
    view = wide[:, :256]  # row stride 512, 256 columns
    out = cuda.zeros_like(wide)
    hm.softmax_kernel[(1,)](view, out[:, :256])
    want = oracle.softmax(np.ascontiguousarray(view.cpu().numpy()))
    assert np.abs(out[:, :256].cpu().numpy().astype(np.float32) - want.astype(np.float32)).max() <= TOL_ROW
    assert float(out[:, 256:].abs().max()) == 0.0  # bytes between rows untouched


@pytest.mark.parametrize("shape,dtype", [((127, 513), np.float16), ((127, 513), np.float32),
                                         ((2048, 4096), np.float16), ((16, 256), np.float16),
                                         ((7, 11008), np.float16)])
def test_rms_norm(hm, oracle, shape, dtype):
    rng = philox(21)
    x = rng.uniform(0, 1, shape).astype(dtype)
    w = rng.uniform(0, 1, shape[1]).astype(dtype)
    y = np.zeros_like(x)
    hm.rms_norm_fwd_kernel[(4,)](x, y, w, EPSILON=1e-5, NUM_ROWS=shape[0], NUM_COLS=shape[1])
    want = oracle.rmsnorm(x, w, 1e-5)
    assert max_abs_rel(y, want) <= TOL_ROW
    assert np.abs(y.astype(np.float32) - want.astype(np.float32)).max() <= 1e-2  # test_rms_norm.py:24


def test_rms_norm_c4_inputs(hm, oracle):
    x = philox(3).normal(0, 1, (2048, 4096)).astype(np.float16)
    g = np.ones(4096, np.float16)
    y = np.zeros_like(x)
    hm.rms_norm_fwd_kernel[(1,)](x, y, g, EPSILON=1e-6)
    assert max_abs_rel(y, oracle.rmsnorm(x, g, 1e-6)) <= TOL_ROW
    hm.set_option("rmsNormEpsilon", 1e-5)


@pytest.mark.parametrize("n", [16384, 1, 7, 8, 100003])
def test_silu_swiglu_add(hm, oracle, n):
    rng = philox(31)
    x = rng.normal(0, 2, n).astype(np.float16)
    u = rng.normal(0, 1, n).astype(np.float16)
    y = np.zeros_like(x)
    hm.silu_kernel[(4,)](x, y, BLOCK_SIZE=4096)
    assert np.abs(y.astype(np.float32) - oracle.silu(x).astype(np.float32)).max() <= 1e-2  # test_silu.py:18
    assert max_abs_rel(y, oracle.silu(x)) <= 2e-3
    hm.swiglu_kernel[(1,)](x, u, y)
    assert max_abs_rel(y, oracle.swiglu(x, u)) <= 2e-3
    hm.add_kernel[(1,)](x, u, y)
    assert np.array_equal(y, oracle.add_f16(x, u))
    x32 = x.astype(np.float32)
    y32 = np.zeros_like(x32)
    hm.silu_kernel[(1,)](x32, y32)
    assert np.abs(y32 - oracle.silu(x32)).max() <= 1e-5


def test_empty_and_mismatched(hm):
    e = np.zeros((0, 64), np.float16)
    hm.softmax_kernel[(1,)](e, e.copy())
    with pytest.raises(hm.B200Error):
        hm.softmax_kernel[(1,)](np.zeros((4, 8), np.float16), np.zeros((4, 16), np.float16))
    with pytest.raises(hm.B200Error):
        hm.softmax_kernel[(2,)](np.zeros((4, 8), np.float16).T, np.zeros((8, 4), np.float16))


def test_launch_counter_counts_kernels(hm):
    hm.reset_launch_count()
    x = np.ones((8, 64), np.float16)
    hm.softmax_kernel[(3,)](x, x.copy())  # three program instances, one kernel
    assert hm.launch_count() == 1
