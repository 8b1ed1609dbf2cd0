"""The attention / online-softmax restatements of the oracle against outputs of the reference's
own kernel sources (tests/golden/attention_golden.npz, written by tests/golden/make_golden.py)."""
import os

import numpy as np

import oracle

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz"))


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / np.linalg.norm(b.astype(np.float64)))


def test_attention_oracle_matches_reference_kernel():
    scale = float(GOLD["attn_scale"])
    for tag in "ab":
        q, k, v = (GOLD[f"attn_{tag}_{n}"] for n in "qkv")
        want = GOLD[f"attn_{tag}_out"]
        bn = int(GOLD[f"attn_{tag}_block_n"])
        # same arithmetic as the kernel source (p kept in fp32): agreement to fp32 round-off
        got = oracle.attention(q, k, v, scale, block_n=bn, p_f32=True)
        assert got.shape == want.shape and np.abs(got - want).max() < 2e-6
        # fp16 p, and the engine's fp16 read-out: inside the reference test's own budget
        tol = float(GOLD["attn_rel_tolerance"])
        assert _rel(oracle.attention(q, k, v, scale, block_n=bn), want) < 1e-4 < tol
        assert _rel(oracle.attention(q, k, v, scale, block_n=bn, engine_rounding=True), want) < 1e-3 < tol


def test_attention_oracle_block_size_and_ragged_tail():
    rng = np.random.default_rng(5)
    q, k, v = (rng.random((2, 3, 200, 64), dtype=np.float32).astype(np.float16) for _ in range(3))
    base = oracle.attention(q, k, v, 0.5, block_n=64)     # 200 = 3 blocks + a tail of 8
    other = oracle.attention(q, k, v, 0.5, block_n=200)   # one block: plain softmax
    assert _rel(base, other) < 1e-4
    s = np.einsum("bhnd,bhmd->bhnm", q.astype(np.float64), k.astype(np.float64)) * 0.5
    p = np.exp(s - s.max(-1, keepdims=True))
    want = np.einsum("bhnm,bhmd->bhnd", p / p.sum(-1, keepdims=True), v.astype(np.float64))
    assert _rel(base, want) < 2e-4


def test_online_softmax_oracle_matches_reference_kernel():
    x = GOLD["online_x"]
    for threads in (1, 4):
        got = oracle.online_softmax(x, x.shape[1] // threads)
        assert np.abs(got - GOLD[f"online_y_threads{threads}"]).max() < 1e-7
    assert np.abs(oracle.online_softmax(x, 32) - oracle.softmax(x)).max() < float(GOLD["online_atol"])


def test_attention_oracle_causal_form():
    """STAGE = 3 of the kernel's signature has no reference output (its loop implements STAGE = 1 only):
    the oracle's causal form is checked against a float64 masked softmax."""
    rng = np.random.default_rng(6)
    q, k, v = (rng.normal(0, 1, (2, 2, 150, 64)).astype(np.float16) for _ in range(3))
    got = oracle.attention(q, k, v, 0.125, block_n=64, causal=True)
    s = np.einsum("bhnd,bhmd->bhnm", q.astype(np.float64), k.astype(np.float64)) * 0.125
    s = np.where(np.tril(np.ones((150, 150), bool)), s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    want = np.einsum("bhnm,bhmd->bhnd", p / p.sum(-1, keepdims=True), v.astype(np.float64))
    assert _rel(got, want) < 2e-4
    # the first query sees only the first key: its output is v[0]
    assert np.allclose(got[..., 0, :], v[..., 0, :].astype(np.float32), atol=1e-6)
    # block size does not matter beyond rounding
    assert _rel(oracle.attention(q, k, v, 0.125, block_n=32, causal=True), got) < 1e-4
