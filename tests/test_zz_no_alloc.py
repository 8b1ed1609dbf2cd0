"""The w8a16 entry point that allocates nothing, against the allocating one.

Collected last on purpose (file name): if it fails, a run that stops at the first
failure has already run everything else.  It calls the C ABI directly with device
pointers; the weight image is built here on the host from the layout the header
documents, so the test also pins that description.
"""
import ctypes

import numpy as np
import pytest

from conftest import max_abs_rel, philox

pytestmark = pytest.mark.gpu

TOL_GEMM = 1e-2  # the tolerance of the other GEMM tests


def build_image(wq: np.ndarray) -> np.ndarray:
    """[strip][kstep][lane][16 B]: byte 4j+e = q[16*kstep + kk[t][e], 32*strip + 8j + g] + 128."""
    k, n = wq.shape
    ksteps, strips = -(-k // 16), -(-n // 32)
    pad = np.zeros((ksteps * 16, strips * 32), np.int16)
    pad[:k, :n] = wq
    w = pad.reshape(ksteps, 16, strips, 4, 8)                      # [ks, kin, strip, j, g]
    kk = np.array([[2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9] for t in range(4)])  # [t, e]
    w = w[:, kk]                                                   # [ks, t, e, strip, j, g]
    w = w.transpose(3, 0, 5, 1, 4, 2)                              # [strip, ks, g, t, j, e]
    return np.ascontiguousarray((w + 128).astype(np.uint8)).ravel()


@pytest.mark.parametrize("m,k,n", [(1, 4096, 11008), (16, 4096, 11008), (64, 512, 1000), (33, 72, 40)])
def test_static_scratch_matches_allocating_entry(hm, oracle, cuda, m, k, n):
    rng = philox(2)
    a = rng.normal(0, 1, (m, k)).astype(np.float16)
    wq = rng.integers(-128, 128, (k, n), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, n).astype(np.float16)
    at, wt, st = (cuda.from_numpy(x).cuda() for x in (a, wq, s))
    want_t = cuda.zeros((m, n), dtype=cuda.float16, device="cuda")
    hm.w8a16_matmul[(1,)](at, wt, st, want_t)           # the existing entry point
    hm.unregister_w8a16_weight(wt)
    want = want_t.cpu().numpy()
    img = cuda.from_numpy(build_image(wq)).cuda()
    lib = hm._capi.lib()
    stream = cuda.cuda.current_stream().cuda_stream
    for call in range(2):                                # two calls in a row share the scratch
        out = cuda.full((m, n), 9.0, dtype=cuda.float16, device="cuda")
        rc = lib.b200mlir_w8a16_matmul_static_scratch(at.data_ptr(), k, img.data_ptr(), st.data_ptr(),
                                                      out.data_ptr(), n, m, n, k, stream)
        assert rc == 0, hm._capi.last_error()
        cuda.cuda.synchronize()
        got = out.cpu().numpy()
        assert max_abs_rel(got, want) <= TOL_GEMM, call
        # same kernels, same image: only the order of the fp32 partial sums can differ
        assert (got.view(np.uint16) != want.view(np.uint16)).mean() < 0.02, call
    assert max_abs_rel(got, oracle.w8a16(a, wq, s)) <= TOL_GEMM


def test_static_scratch_rejects_oversize_and_bad_arguments(hm, cuda):
    lib = hm._capi.lib()
    buf = cuda.zeros(1 << 20, dtype=cuda.uint8, device="cuda")
    p = buf.data_ptr()
    assert lib.b200mlir_w8a16_matmul_static_scratch(p, 64, p, p, p, 16385, 1, 16385, 64, None) == 6
    assert "exceed" in hm._capi.last_error()[1]
    assert lib.b200mlir_w8a16_matmul_static_scratch(p, 64, p, p, p, 64, 65, 64, 64, None) == 6
    assert lib.b200mlir_w8a16_matmul_static_scratch(None, 64, p, p, p, 64, 1, 64, 64, None) == 2
    assert lib.b200mlir_w8a16_matmul_static_scratch(p, 60, p, p, p, 64, 1, 64, 60, None) == 2
    assert lib.b200mlir_w8a16_matmul_static_scratch(p + 2, 64, p, p, p, 64, 1, 64, 64, None) == 2
