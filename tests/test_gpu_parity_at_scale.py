"""Parity at the shapes the benchmark quotes: the large GEMM 16384 x 16384 x 8192 (seed 4,
U[-1, 1]) and its per-rank column shards, and the MLP block at the tensor-parallel shard shapes
of 2, 4 and 8 ranks — all on ONE GPU, so the shapes a multi-GPU run times are checked wherever
the single-GPU suite runs.

A CPU GEMM of 4.4 TFLOP is out of reach, so the oracle checks >= 64 random 128 x 128 output tiles
with full K (operand rows and columns are drawn on the CPU from the same counter-based generator
that filled the device tensors: nothing is copied down but the results), and the whole output is
tied to those samples by row-sum / column-sum checksums against the CUDA-core path and by the
algebraic column checksum sum_i C[i, j] = (sum_i A[i, :]) . B[:, j].  Tolerance: max-abs-rel 1e-2
(the north star's), relative Frobenius 2e-3 (test/python/triton/test_matmul_kloop.py:157-163)."""
import numpy as np
import pytest

from conftest import max_abs_rel, philox

pytestmark = pytest.mark.gpu

M, N, K = 16384, 16384, 8192
SEED_A, SEED_B = 4, 5
TILE = 128


@pytest.fixture(scope="module")
def operands(hm, cuda):
    a = cuda.empty((M, K), dtype=cuda.float16, device="cuda")
    b = cuda.empty((K, N), dtype=cuda.float16, device="cuda")
    hm.fill_random(a, SEED_A, hm.UNIFORM, -1.0, 1.0)
    hm.fill_random(b, SEED_B, hm.UNIFORM, -1.0, 1.0)
    yield a, b
    del a, b
    cuda.cuda.empty_cache()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_large_gemm_and_its_shards_against_the_oracle(hm, oracle, cuda, operands, world):
    a, b_full = operands
    rank = world - 1                                  # the last rank: a non-zero column offset
    lo, hi = rank * N // world, (rank + 1) * N // world
    n_loc = hi - lo
    b = b_full[:, lo:hi].contiguous() if world > 1 else b_full
    c = cuda.empty((M, n_loc), dtype=cuda.float16, device="cuda")
    hm.matmul[(1,)](a, b, c)
    assert hm.device_status() == 0
    assert hm.gemm_explain(M, n_loc, K)["plan"] == "tcgen05"

    # ---- 64 random tiles, full K, against the oracle --------------------------------------------
    rng = philox(1000 + world)
    tiles = {(int(rng.integers(M // TILE)), int(rng.integers(n_loc // TILE))) for _ in range(80)}
    tiles = sorted(tiles)[:64]
    assert len(tiles) == 64
    worst, num, den = 0.0, 0.0, 0.0
    rows_cache = {}
    for tm, tn in tiles:
        if tm not in rows_cache:
            rows_cache[tm] = oracle.random_rows(tm * TILE, TILE, K, np.float16, SEED_A, oracle.UNIFORM, -1.0, 1.0)
        cols = oracle.random_cols(lo + tn * TILE, TILE, K, N, np.float16, SEED_B, oracle.UNIFORM, -1.0, 1.0)
        want = oracle.gemm_f16(rows_cache[tm], cols).astype(np.float32)
        got = c[tm * TILE:(tm + 1) * TILE, tn * TILE:(tn + 1) * TILE].cpu().numpy().astype(np.float32)
        worst = max(worst, max_abs_rel(got, want))
        num += float(((got - want) ** 2).sum())
        den += float((want ** 2).sum())
    assert worst <= 1e-2, worst
    assert (num / den) ** 0.5 < 2e-3
    # the device tensors really hold the generator's bytes (one tile of each operand)
    assert np.array_equal(a[:TILE].cpu().numpy(), oracle.random_rows(0, TILE, K, np.float16, SEED_A, 0, -1.0, 1.0))
    assert np.array_equal(b_full[:, lo:lo + 8].cpu().numpy(),
                          oracle.random_cols(lo, 8, K, N, np.float16, SEED_B, 0, -1.0, 1.0))

    # ---- checksums over the whole output ----------------------------------------------------------
    c_simt = cuda.empty_like(c)
    hm.set_option("gemmVariant", 99)                  # the CUDA-core path
    try:
        hm.matmul[(1,)](a, b, c_simt)
    finally:
        hm.set_option("gemmVariant", -1)
    assert hm.device_status() == 0
    cd, sd = c.double(), c_simt.double()
    scale = float(sd.abs().sum(dim=1).max())
    assert float((cd.sum(dim=1) - sd.sum(dim=1)).abs().max()) <= 1e-4 * scale      # row sums
    scale = float(sd.abs().sum(dim=0).max())
    assert float((cd.sum(dim=0) - sd.sum(dim=0)).abs().max()) <= 1e-4 * scale      # column sums
    assert float((cd - sd).abs().max()) <= 1e-2 * float(sd.abs().max())            # and element-wise
    # algebraic: column sums of C from the operands alone (fp64); the only error left is the fp16
    # rounding of each of the 16384 summed elements (|c| up to ~200: half an ulp is 0.0625)
    want_cols = (a.double().sum(dim=0, keepdim=True) @ b.double()).squeeze(0)
    assert float((cd.sum(dim=0) - want_cols).abs().max()) <= 0.0625 * M ** 0.5 * 6
    del c, c_simt, cd, sd


@pytest.mark.parametrize("world", [2, 4, 8])
def test_mlp_block_at_tensor_parallel_shard_shapes(hm, oracle, cuda, world):
    """2048 x 4096, ffn 11008 (seed 3) cut the way `tp.shard_bounds` cuts it for `world` ranks; every
    rank's partial is computed here in turn and the partials are summed in fp16, the way an fp16
    all-reduce sums them.  Twice: with rank 0's partial carrying the residual, and with the ranks
    taking turns by 256-row block (options mlpResidualMod / mlpResidualRem, what the tensor-parallel
    entries do), where exactly one partial of every block differs from its residual-free self."""
    from hexagon_mlir_b200 import tp
    t, d, f = 2048, 4096, 11008
    x = cuda.empty((t, d), dtype=cuda.float16, device="cuda")
    wg = cuda.empty((d, f), dtype=cuda.float16, device="cuda")
    wu = cuda.empty((d, f), dtype=cuda.float16, device="cuda")
    wd = cuda.empty((f, d), dtype=cuda.float16, device="cuda")
    hm.fill_random(x, 3, hm.NORMAL, 0.0, 1.0)
    hm.fill_random(wg, 31, hm.NORMAL, 0.0, 0.02)
    hm.fill_random(wu, 32, hm.NORMAL, 0.0, 0.02)
    hm.fill_random(wd, 33, hm.NORMAL, 0.0, 0.02)
    gain = cuda.ones(d, dtype=cuda.float16, device="cuda")
    total, shared = None, None
    widths = []
    for r in range(world):
        lo, hi = tp.shard_bounds(f, r, world)
        widths.append(hi - lo)
        shard = (wg[:, lo:hi].contiguous(), wu[:, lo:hi].contiguous(), wd[lo:hi].contiguous())
        part = cuda.zeros((t, d), dtype=cuda.float16, device="cuda")
        hm.mlp_block[(1,)](x, gain, *shard, part, eps=1e-6, add_residual=(r == 0))
        total = part if total is None else total + part          # fp16 add, rounded per step
        bare = part if r != 0 else None
        if bare is None:
            bare = cuda.zeros((t, d), dtype=cuda.float16, device="cuda")
            hm.mlp_block[(1,)](x, gain, *shard, bare, eps=1e-6, add_residual=False)
        turn = cuda.zeros((t, d), dtype=cuda.float16, device="cuda")
        hm.set_option("mlpResidualMod", world)
        hm.set_option("mlpResidualRem", r)
        try:
            hm.mlp_block[(1,)](x, gain, *shard, turn, eps=1e-6, add_residual=True)
        finally:
            hm.set_option("mlpResidualMod", 1)
            hm.set_option("mlpResidualRem", 0)
        blocks_changed = (turn != bare).view(t // 256, 256 * d).any(dim=1).cpu().numpy()
        assert np.array_equal(np.nonzero(blocks_changed)[0], np.arange(r, t // 256, world))   # this rank's blocks only
        shared = turn if shared is None else shared + turn
    assert hm.device_status() == 0
    assert sum(widths) == f and max(widths) - min(widths) <= 8
    rows = np.sort(philox(99).choice(t, 96, replace=False))
    xh = oracle.fill_random((t, d), np.float16, 3, oracle.NORMAL, 0.0, 1.0)
    assert np.array_equal(xh[rows], x.cpu().numpy()[rows])          # same bytes on both sides
    W = [oracle.fill_random(s, np.float16, seed, oracle.NORMAL, 0.0, 0.02)
         for s, seed in (((d, f), 31), ((d, f), 32), ((f, d), 33))]
    want = oracle.mlp(xh[rows], np.ones(d, np.float16), *W, 1e-6)
    assert max_abs_rel(total.cpu().numpy()[rows], want) <= 1e-2
    assert max_abs_rel(shared.cpu().numpy()[rows], want) <= 1e-2
