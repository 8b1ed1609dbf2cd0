"""The reference's own device tests, replayed: same shapes and input distributions, the expected
values those tests compute with torch (committed fixture, tests/golden/make_golden.py), the
tolerance each test applies.  The oracle must pass them on the CPU; the kernels on the GPU."""
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "device_tests_golden.npz")


@pytest.fixture(scope="module")
def gold():
    z = np.load(GOLD)
    return z, json.loads(str(z["tolerances"]))


def check_all(gold, softmax16, softmax32, rms16, rms32, silu16, silu32, matmul, kloop):
    z, tol = gold
    x = z["softmax_x"]
    assert np.abs(softmax16(x).astype(np.float32) - z["softmax_f16_expected"].astype(np.float32)).max() <= tol["softmax_f16_atol"]
    assert np.abs(softmax32(x.astype(np.float32)) - z["softmax_f32_expected"]).max() <= tol["softmax_f32_atol"]
    x, w = z["rmsnorm_x"], z["rmsnorm_w"]
    assert np.abs(rms16(x, w).astype(np.float32) - z["rmsnorm_f16_expected"].astype(np.float32)).max() <= tol["rmsnorm_atol"]
    assert np.abs(rms32(x.astype(np.float32), w.astype(np.float32)) - z["rmsnorm_f32_expected"]).max() <= tol["rmsnorm_atol"]
    x = z["silu_x"]
    assert np.abs(silu16(x).astype(np.float32) - z["silu_f16_expected"].astype(np.float32)).max() <= tol["silu_atol"]
    assert np.abs(silu32(x.astype(np.float32)) - z["silu_f32_expected"]).max() <= tol["silu_atol"]
    got = matmul(z["matmul_a"], z["matmul_b"])[0::4]
    assert np.abs(got.astype(np.float32) - z["matmul_expected_rows_0_4"].astype(np.float32)).max() <= tol["matmul_atol"]
    got = kloop(z["kloop_a"], z["kloop_b"], tol["kloop_block_k"]).astype(np.float32)
    ref = z["kloop_expected_f32"]
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < tol["kloop_rel"]


def test_oracle_passes_the_reference_device_tests(oracle, gold):
    check_all(gold, oracle.softmax, oracle.softmax, lambda x, w: oracle.rmsnorm(x, w, 1e-5),
              lambda x, w: oracle.rmsnorm(x, w, 1e-5), oracle.silu, oracle.silu, oracle.gemm_f16,
              lambda a, b, bk: oracle.gemm_f16(a, b, block_k=bk))


@pytest.mark.gpu
def test_kernels_pass_the_reference_device_tests(hm, gold):
    def run2(kernel, x, **opts):
        y = np.empty_like(x)
        kernel[(1,)](x, y, **opts)
        return y

    def rms(x, w):
        y = np.empty_like(x)
        hm.rms_norm_fwd_kernel[(1,)](x, y, w, EPSILON=1e-5, NUM_ROWS=127, NUM_COLS=513, BLOCK_SIZE=1024)
        return y

    def mm(kernel, a, b, **opts):
        c = np.zeros((a.shape[0], b.shape[1]), np.float16)
        kernel[(1,)](a, b, c, **opts)
        return c

    check_all(gold, lambda x: run2(hm.softmax_kernel, x, NUM_ROWS=128, NUM_COLS=128, BLOCK_SIZE=128),
              lambda x: run2(hm.softmax_kernel, x), rms, rms,
              lambda x: run2(hm.silu_kernel, x, BLOCK_SIZE=16384), lambda x: run2(hm.silu_kernel, x),
              lambda a, b: mm(hm.matmul, a, b), lambda a, b, bk: mm(hm.klooped_matmul, a, b, BLOCK_K=bk))
    assert hm.device_status() == 0
