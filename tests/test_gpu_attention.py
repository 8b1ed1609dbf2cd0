"""Attention block through the C ABI against the oracle and the fixtures made from the
reference's own kernel source.  Tolerance: the reference test's relative Frobenius error
below 5e-3 (test/python/triton/test_flash_attention.py:248-249); this kernel keeps S and P·V in
fp32, so it is also held to 3e-4 against the oracle's fp16-operand form."""
import os

import numpy as np
import pytest

from conftest import philox

pytestmark = pytest.mark.gpu

REF_TOL = 5e-3
TIGHT = 3e-4
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz"))


def _rel(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / np.linalg.norm(want))


def test_reference_case_float32(hm, oracle, cuda):
    """Z=H=1, N_CTX=1024, D_HEAD=64, fp32 tensors of torch.rand, sm_scale 0.5, launched as the reference does."""
    cuda.manual_seed(0)
    q, k, v = (cuda.rand(1, 1, 1024, 64, device="cuda") for _ in range(3))
    out = cuda.zeros_like(q)
    hm.attention_fwd_kernel[(1,)](pid1=0, Q=q, K=k, V=v, sm_scale=0.5, Out=out, H=1, N_CTX=1024, BLOCK_M=1024,
                                  BLOCK_DMODEL=64, BLOCK_N=64, STAGE=1, stride_0=65536, stride_1=65536,
                                  stride_2=64, stride_3=1, enableVectorization=True, enableMultiThreading=True,
                                  enableConvertToHexagonmem=True, enableHexagonmemCopyToDMA=False)
    want = cuda.nn.functional.scaled_dot_product_attention(q, k, v, scale=0.5)
    rel = float((out - want).norm() / want.norm())
    assert rel < REF_TOL
    o = oracle.attention(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), 0.5, block_n=64)
    assert _rel(out.cpu().numpy(), o) < TIGHT
    assert hm.device_status() == 0


def test_golden_from_reference_kernel(hm):
    for tag in "ab":
        q, k, v = (GOLD[f"attn_{tag}_{n}"] for n in "qkv")  # fp16, host
        out = np.zeros(q.shape, np.float16)
        hm.attention(q, k, v, out, float(GOLD["attn_scale"]))
        assert _rel(out, GOLD[f"attn_{tag}_out"]) < 6e-4  # fp16 output rounding included
        out32 = np.zeros(q.shape, np.float32)
        hm.attention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), out32, float(GOLD["attn_scale"]))
        assert _rel(out32, GOLD[f"attn_{tag}_out"]) < TIGHT


@pytest.mark.parametrize("shape,tiles", [((2, 3, 200, 64), 0), ((2, 3, 200, 64), 2), ((1, 2, 384, 128), 1),
                                         ((1, 2, 384, 128), 2), ((1, 1, 1, 64), 0), ((1, 5, 129, 64), 2),
                                         ((3, 1, 72, 128), 0), ((1, 2, 1000, 64), 1)])
def test_shapes_ragged_and_both_tilings(hm, oracle, cuda, shape, tiles):
    rng = philox(31)
    q, k, v = (rng.normal(0, 1, shape).astype(np.float16) for _ in range(3))
    scale = 1.0 / np.sqrt(shape[-1])
    want = oracle.attention(q, k, v, scale, block_n=64)
    hm.set_option("attentionTiles", tiles)
    try:
        qt, kt, vt = (cuda.from_numpy(t).cuda() for t in (q, k, v))
        out = cuda.zeros_like(qt)
        hm.attention(qt, kt, vt, out, scale)
        got = out.cpu().numpy()
    finally:
        hm.set_option("attentionTiles", 0)
    assert _rel(got, want) < 8e-4  # fp16 output
    assert hm.device_status() == 0


def test_strided_heads_and_pid1(hm, oracle, cuda):
    """[Z, N, H, D] storage viewed as [Z, H, N, D]; and one (batch, head) per call through pid1."""
    rng = philox(32)
    z, h, n, d = 2, 4, 320, 64
    base = [rng.normal(0, 1, (z, n, h, d)).astype(np.float16) for _ in range(3)]
    q, k, v = (cuda.from_numpy(t).cuda().permute(0, 2, 1, 3) for t in base)
    want = oracle.attention(*(np.ascontiguousarray(t.transpose(0, 2, 1, 3)) for t in base), 0.25, block_n=64)
    out = cuda.zeros(z, h, n, d, dtype=cuda.float16, device="cuda")
    hm.attention(q, k, v, out, 0.25)
    assert _rel(out.cpu().numpy(), want) < 8e-4
    out2 = cuda.zeros(z, n, h, d, dtype=cuda.float16, device="cuda").permute(0, 2, 1, 3)
    for pid1 in range(z * h):
        hm.attention_fwd_kernel[(1,)](pid1, q, k, v, 0.25, out2, h)
    assert cuda.equal(out2, out)


def test_large_against_torch_and_repeatable(hm, cuda):
    cuda.manual_seed(3)
    q, k, v = (cuda.randn(2, 8, 2048, 64, device="cuda", dtype=cuda.float16) for _ in range(3))
    out = cuda.zeros_like(q)
    hm.attention(q, k, v, out, 0.125)
    want = cuda.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), scale=0.125)
    assert float((out.float() - want).norm() / want.norm()) < 8e-4
    again = cuda.zeros_like(q)
    hm.attention(q, k, v, again, 0.125)
    assert cuda.equal(out, again)
    # rows of softmax(QK)·1 are 1: V of ones gives ones, whatever the scores
    ones = cuda.ones_like(v)
    hm.attention(q, k, ones, out, 0.125)
    assert float((out.float() - 1).abs().max()) < 2e-3


@pytest.mark.parametrize("d,tiles", [(64, 0), (64, 2), (128, 0), (128, 2)])
def test_scores_that_grow_block_by_block(hm, oracle, cuda, d, tiles):
    """The kernel keeps O in TMEM scaled by a lazily updated maximum and rescales it only when a
    row's maximum grows by more than 2^8: keys whose scores rise by ~11.5 (in log2) per 64-key
    block force that on every block, for the rows of the second half of each tile only."""
    rng = philox(33)
    n = 576  # nine blocks
    q = rng.uniform(-0.02, 0.02, (2, 2, n, d)).astype(np.float16)
    q[:, :, np.arange(n) % 128 >= 64] += np.float16(16.0 / d)   # these rows see the growing scores
    k = (np.arange(n) // 64 * 0.5)[None, None, :, None] + rng.uniform(-0.05, 0.05, (2, 2, n, d))
    k = k.astype(np.float16)
    v = rng.normal(0, 1, (2, 2, n, d)).astype(np.float16)
    want = oracle.attention(q, k, v, 1.0, block_n=64)
    hm.set_option("attentionTiles", tiles)
    try:
        out = np.zeros_like(q)
        hm.attention(q, k, v, out, 1.0)
    finally:
        hm.set_option("attentionTiles", 0)
    assert np.isfinite(out.astype(np.float32)).all()
    assert _rel(out, want) < 8e-4
    assert hm.device_status() == 0
    # and the other way round: the largest scores first, nothing to rescale afterwards
    k2 = np.ascontiguousarray(k[:, :, ::-1])
    want2 = oracle.attention(q, k2, v, 1.0, block_n=64)
    out2 = np.zeros_like(q)
    hm.attention(q, k2, v, out2, 1.0)
    assert _rel(out2, want2) < 8e-4


@pytest.mark.parametrize("shape,splits", [((1, 1, 1024, 64), 0), ((1, 1, 1024, 64), 8), ((1, 2, 1000, 128), 3),
                                          ((2, 1, 520, 64), 9), ((1, 1, 2048, 128), 0)])
def test_keys_split_over_ctas(hm, oracle, cuda, shape, splits):
    """Few query tiles: the key blocks are shared out over several CTAs per tile and merged by a
    second kernel (automatically, or with option attentionSplits)."""
    rng = philox(34)
    q, k, v = (rng.normal(0, 1, shape).astype(np.float16) for _ in range(3))
    k[..., shape[2] // 2:, :] *= np.float16(3.0)  # the later splits see larger maxima
    scale = 1.0 / np.sqrt(shape[-1])
    want = oracle.attention(q, k, v, scale, block_n=64)
    hm.set_option("attentionSplits", splits)
    try:
        out = cuda.zeros(shape, dtype=cuda.float16, device="cuda")
        qt, kt, vt = (cuda.from_numpy(t).cuda() for t in (q, k, v))
        before = hm.launch_count()
        hm.attention(qt, kt, vt, out, scale)
        launches = hm.launch_count() - before
        out32 = np.zeros(shape, np.float32)
        hm.attention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), out32, scale)
    finally:
        hm.set_option("attentionSplits", 0)
    assert launches == 2  # the split kernel and the merge
    assert _rel(out.cpu().numpy(), want) < 8e-4
    assert _rel(out32, want) < TIGHT
    assert hm.device_status() == 0


@pytest.mark.parametrize("shape", [(2, 3, 200, 64), (1, 2, 1000, 128), (1, 1, 64, 64), (1, 4, 2048, 64)])
def test_causal(hm, oracle, cuda, shape):
    """STAGE = 3 of the reference kernel's signature: query i sees keys 0..i.  The reference's loop does
    not implement it, so the oracle's causal form is itself checked against torch here."""
    rng = philox(35)
    q, k, v = (rng.normal(0, 1, shape).astype(np.float16) for _ in range(3))
    scale = 1.0 / np.sqrt(shape[-1])
    want = oracle.attention(q, k, v, scale, block_n=64, causal=True)
    qt, kt, vt = (cuda.from_numpy(t).cuda() for t in (q, k, v))
    ref = cuda.nn.functional.scaled_dot_product_attention(qt.float(), kt.float(), vt.float(), scale=scale, is_causal=True)
    assert _rel(want, ref.cpu().numpy()) < 3e-4
    out = cuda.zeros_like(qt)
    hm.attention(qt, kt, vt, out, scale, causal=True)
    assert _rel(out.cpu().numpy(), want) < 8e-4
    out32 = np.zeros(shape, np.float32)
    hm.attention_fwd_kernel[(1,)](Q=q.astype(np.float32), K=k.astype(np.float32), V=v.astype(np.float32), Out=out32,
                                  sm_scale=scale, STAGE=3)
    assert _rel(out32, want) < TIGHT
    # the stage is per launch: the next plain call sees every key again
    hm.attention(qt, kt, vt, out, scale)
    assert _rel(out.cpu().numpy(), oracle.attention(q, k, v, scale, block_n=64)) < 8e-4
    assert hm.device_status() == 0


def test_online_softmax_as_the_reference_launches_it(hm, oracle, cuda):
    """test_online_softmax.py:80-110: 128 x 128 fp32, 1 and 4 programs, atol 1e-5 against torch."""
    x = GOLD["online_x"]
    for threads in (1, 4):
        xt = cuda.from_numpy(x).cuda()
        out = cuda.empty_like(xt)
        hm.online_softmax[(threads,)](xt, out, NUM_ROWS=128, NUM_COLS=128, BLOCK_ROW_SIZE=128 // threads,
                                      BLOCK_COL_SIZE=128 // threads, enableMultiThreading=threads == 1,
                                      enableVTCMTiling=threads == 1, enableConvertToHexagonmem=threads == 1,
                                      enableHexagonmemCopyToDMA=threads == 1)
        got = out.cpu().numpy()
        atol = float(GOLD["online_atol"])
        assert np.abs(got - GOLD[f"online_y_threads{threads}"]).max() < atol  # the reference kernel's own output
        assert np.abs(got - oracle.online_softmax(x, 128 // threads)).max() < atol
        assert cuda.allclose(out, cuda.nn.functional.softmax(xt, dim=1), atol=atol)


def test_refusals(hm, cuda):
    q = cuda.zeros(1, 1, 64, 32, device="cuda", dtype=cuda.float16)
    with pytest.raises(hm.B200Error) as e:
        hm.attention(q, q, q, cuda.zeros_like(q), 0.5)
    assert e.value.code == 6  # head size
    q = cuda.zeros(1, 1, 64, 64, device="cuda", dtype=cuda.float16)
    with pytest.raises(hm.B200Error) as e:
        hm.attention(q, q, q, cuda.zeros_like(q), -1.0)
    assert e.value.code == 2
    with pytest.raises(hm.B200Error) as e:
        hm.attention(q, q[:, :, :32], q, cuda.zeros_like(q), 0.5)
    assert e.value.code == 2
