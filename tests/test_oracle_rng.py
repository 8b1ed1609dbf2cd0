"""The synthetic-input generator: Philox4x32-10 pinned to the published known-answer vectors of
the algorithm (Salmon et al., SC'11; the Random123 distribution's kat_vectors), and the C++ loop
beside the oracle equal, byte for byte, to the numpy twin for every distribution and dtype the
configs use.  (The GPU kernel of the library is held to the same bytes in the -m gpu suite.)"""
import numpy as np
import pytest

KAT = [  # counter, key, output
    ((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
    ((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2, (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
    ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
     (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
]


@pytest.mark.parametrize("counter,key,want", KAT)
def test_philox_known_answers(oracle, counter, key, want):
    c = [np.array([x], np.uint64) for x in counter]
    got = tuple(int(x[0]) for x in oracle._philox_np(*c, key[0], key[1]))
    assert got == want


CASES = [  # the configs' distributions: (dist, p0, p1, dtype)
    (0, -1.0, 1.0, np.float16),      # GEMM operands, U[-1, 1]
    (1, 0.0, 3.0, np.float16),       # softmax input, N(0, 3)
    (1, 0.0, 1.0, np.float16),       # activations, N(0, 1)
    (1, 0.0, 0.02, np.float16),      # MLP weights, N(0, 0.02)
    (2, -127, 127, np.int8),         # quantised weight
    (0, 0.001, 0.02, np.float16),    # per-channel scales
    (0, 0.0, 1.0, np.float32),
    (1, 0.0, 1.0, np.float32),
]


@pytest.mark.parametrize("dist,p0,p1,dtype", CASES)
def test_cpp_loop_equals_numpy_twin(oracle, dist, p0, p1, dtype):
    for seed in (0, 4, 0x1234_5678_9ABC_DEF0):
        a = oracle.fill_random((257, 129), dtype, seed, dist, p0, p1)
        b = oracle.fill_random_numpy((257, 129), dtype, seed, dist, p0, p1)
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
    # statistics of what the configs ask for
    x = a.astype(np.float64)
    if dist == 0:
        hi = float(np.asarray(p1, dtype))   # the bound itself rounds to the tensor's type
        assert p0 <= x.min() and x.max() <= hi and abs(x.mean() - (p0 + p1) / 2) < 0.02 * (p1 - p0)
    elif dist == 1:
        assert abs(x.mean() - p0) < 0.03 * p1 and abs(x.std() / p1 - 1) < 0.03
    else:
        assert x.min() == p0 and x.max() == p1


def test_any_slice_can_be_drawn_alone(oracle):
    """Counter-based: element i depends on (seed, i) only, so a tile of a 16384 x 8192 operand is
    drawn without the rest, and a different thread count changes nothing."""
    full = oracle.fill_random((4096,), np.float16, 4, 0, -1, 1, threads=1)
    assert np.array_equal(full, oracle.fill_random((4096,), np.float16, 4, 0, -1, 1, threads=7))
    part = oracle.fill_random_numpy((100,), np.float16, 4, 0, -1, 1, start=3001)
    assert np.array_equal(full[3001:3101], part)
    far = oracle.fill_random_numpy((8,), np.float16, 4, 0, -1, 1, start=(1 << 34) + 5)   # past 2^32 blocks
    assert np.isfinite(far.astype(np.float32)).all() and len(set(far.tolist())) > 1
    assert not np.array_equal(oracle.fill_random((64,), np.float16, 5, 0, -1, 1), full[:64])
