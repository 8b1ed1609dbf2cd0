"""TEST INFRASTRUCTURE — NOT PRODUCT CODE.

ctypes front end of the CPU oracle (``hexmlir_oracle.cpp``) and, when it has
been built, of the reference project's own layout leaves (``_ref/``).  Only the
test-suite, the smoke check and the benchmark's CPU-baseline leg may import
this package; the shipped library never does.

Parity status: layout functions are pinned against the reference's compiled
``HMXLayout.c`` and its closed-form byte rule; engine arithmetic and the
vector-math library cannot run off-device, so for matmul / softmax / RMSNorm /
SiLU bit-level parity is UNPINNED and the oracle is anchored on the
reference's own end-to-end tolerances.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_f32 = ctypes.c_float
_u32 = ctypes.c_uint


def build(with_ref: bool = True, ref_root: str | None = None) -> None:
    """Compile ``liboracle.so`` and, when a reference checkout is named (argument, else the
    environment variable HEXMLIR_REFERENCE_ROOT) and exists, ``_ref/`` from its sources in place."""
    subprocess.run(["make", "-s", "-C", _HERE, "all"], check=True)
    ref_root = ref_root or os.environ.get("HEXMLIR_REFERENCE_ROOT", "")
    if with_ref and ref_root and os.path.isdir(ref_root):
        subprocess.run(["make", "-s", "-C", _HERE, "ref", f"REF={ref_root}"],
                       check=True, stderr=subprocess.DEVNULL)


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build(with_ref=False)
        _LIB = ctypes.CDLL(path)
        _LIB.oracle_hw_threads.restype = _int
    return _LIB


def ref_lib():
    """The reference's compiled layout leaves, or None when not built."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libhmxlayout_ref.so")
        if not os.path.exists(path):
            return None
        _REF = ctypes.CDLL(path)
        if _REF.ref_layout_init() != 0:
            _REF = None
    return _REF


def hw_threads() -> int:
    return int(lib().oracle_hw_threads())


def _ptr(a: np.ndarray):
    return ctypes.c_void_p(a.ctypes.data)


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.dtype(dtype), (a.dtype, dtype)
    return a


def _nt(threads):
    return int(threads) if threads else hw_threads()


def gemm_f16(a, b, block_k: int = 0, threads: int = 0):
    a, b = _c(a, np.float16), _c(b, np.float16)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.float16)
    lib().oracle_gemm_f16(_ptr(a), _ptr(b), _ptr(c), _i64(m), _i64(n), _i64(k),
                          _i64(k), _i64(n), _i64(n), _i64(block_k), _int(_nt(threads)))
    return c


def gemm_f16_f32out(a, b, res=None, threads: int = 0):
    a, b = _c(a, np.float16), _c(b, np.float16)
    m, k = a.shape
    _, n = b.shape
    c = np.empty((m, n), np.float32)
    r = _c(res, np.float32) if res is not None else None
    lib().oracle_gemm_f16_f32out(_ptr(a), _ptr(b), _ptr(c),
                                 _ptr(r) if r is not None else None,
                                 _i64(m), _i64(n), _i64(k), _i64(k), _i64(n),
                                 _i64(n), _i64(n), _int(_nt(threads)))
    return c


def gemm_i8_i32(a, b, threads: int = 0):
    a, b = _c(a, np.int8), _c(b, np.int8)
    m, k = a.shape
    _, n = b.shape
    c = np.empty((m, n), np.int32)
    lib().oracle_gemm_i8_i32(_ptr(a), _ptr(b), _ptr(c), _i64(m), _i64(n), _i64(k),
                             _int(_nt(threads)))
    return c


def w8a16(a, wq, scales, threads: int = 0):
    a, wq, scales = _c(a, np.float16), _c(wq, np.int8), _c(scales, np.float16)
    m, k = a.shape
    _, n = wq.shape
    c = np.empty((m, n), np.float16)
    lib().oracle_w8a16(_ptr(a), _ptr(wq), _ptr(scales), _ptr(c), _i64(m), _i64(n),
                       _i64(k), _int(_nt(threads)))
    return c


def softmax(x, threads: int = 0):
    x = np.ascontiguousarray(x)
    y = np.empty_like(x)
    fn = {np.dtype(np.float16): lib().oracle_softmax_f16,
          np.dtype(np.float32): lib().oracle_softmax_f32}[x.dtype]
    fn(_ptr(x), _ptr(y), _i64(x.shape[0]), _i64(x.shape[1]), _int(_nt(threads)))
    return y


def rmsnorm(x, g, eps: float, threads: int = 0):
    x, g = np.ascontiguousarray(x), np.ascontiguousarray(g)
    assert x.dtype == g.dtype
    y = np.empty_like(x)
    fn = {np.dtype(np.float16): lib().oracle_rmsnorm_f16,
          np.dtype(np.float32): lib().oracle_rmsnorm_f32}[x.dtype]
    fn(_ptr(x), _ptr(g), _ptr(y), _i64(x.shape[0]), _i64(x.shape[1]), _f32(eps),
       _int(_nt(threads)))
    return y


def silu(x, threads: int = 0):
    x = np.ascontiguousarray(x)
    y = np.empty_like(x)
    fn = {np.dtype(np.float16): lib().oracle_silu_f16,
          np.dtype(np.float32): lib().oracle_silu_f32}[x.dtype]
    fn(_ptr(x), _ptr(y), _i64(x.size), _int(_nt(threads)))
    return y


def swiglu(gate, up, threads: int = 0):
    gate, up = _c(gate, np.float16), _c(up, np.float16)
    y = np.empty_like(gate)
    lib().oracle_swiglu_f16(_ptr(gate), _ptr(up), _ptr(y), _i64(gate.size),
                            _int(_nt(threads)))
    return y


def add_f16(a, b, threads: int = 0):
    a, b = _c(a, np.float16), _c(b, np.float16)
    y = np.empty_like(a)
    lib().oracle_add_f16(_ptr(a), _ptr(b), _ptr(y), _i64(a.size), _int(_nt(threads)))
    return y


def mlp(x, gain, wg, wu, wd, eps: float, threads: int = 0):
    x, gain = _c(x, np.float16), _c(gain, np.float16)
    wg, wu, wd = _c(wg, np.float16), _c(wu, np.float16), _c(wd, np.float16)
    t, d = x.shape
    f = wg.shape[1]
    assert wg.shape == (d, f) and wu.shape == (d, f) and wd.shape == (f, d)
    y = np.empty_like(x)
    lib().oracle_mlp_f16(_ptr(x), _ptr(gain), _ptr(wg), _ptr(wu), _ptr(wd), _ptr(y),
                         _i64(t), _i64(d), _i64(f), _f32(eps), _int(_nt(threads)))
    return y


def attention(q, k, v, sm_scale: float, block_n: int = 64, engine_rounding: bool = False,
              p_f32: bool = False, causal: bool = False, threads: int = 0):
    """Attention block in the reference kernel's order; q, k, v are [..., N, D] (fp32 inputs
    are rounded to fp16 first, as the engine's pack leaf does); returns fp32 of q's shape."""
    q, k, v = (_c(np.asarray(t).astype(np.float16), np.float16) for t in (q, k, v))
    assert q.shape == k.shape == v.shape and q.ndim >= 2
    n, d = q.shape[-2:]
    bh = q.size // (n * d)
    o = np.empty(q.shape, np.float32)
    _f64 = ctypes.c_double
    lib().oracle_attention_f16(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _i64(bh), _i64(n), _i64(d),
                               _f64(sm_scale), _int(block_n),
                               _int((1 if engine_rounding else 0) | (2 if p_f32 else 0) | (4 if causal else 0)),
                               _int(_nt(threads)))
    return o


def online_softmax(x, block_cols: int, threads: int = 0):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    lib().oracle_online_softmax_f32(_ptr(x), _ptr(y), _i64(x.shape[0]), _i64(x.shape[1]),
                                    _i64(block_cols), _int(_nt(threads)))
    return y


# ---- tile layout -----------------------------------------------------------

def _tiles(n):
    return (n + 31) // 32


def pack_weight_f16(w):
    w = np.ascontiguousarray(w)
    bits = w.view(np.uint16)
    k, n = bits.shape
    out = np.empty(_tiles(n) * _tiles(k) * 1024, np.uint16)
    lib().oracle_pack_weight_f16(_ptr(bits), _ptr(out), _i64(k), _i64(n), _i64(n))
    return out


def pack_act_f16(a):
    bits = np.ascontiguousarray(a).view(np.uint16)
    r, c = bits.shape
    out = np.empty(_tiles(r) * _tiles(c) * 1024, np.uint16)
    lib().oracle_pack_act_f16(_ptr(bits), _ptr(out), _i64(r), _i64(c), _i64(c))
    return out


def unpack_acc_f16(tiles, rows, cols):
    tiles = _c(tiles, np.uint16)
    out = np.zeros((rows, cols), np.uint16)
    lib().oracle_unpack_acc_f16(_ptr(tiles), _ptr(out), _i64(rows), _i64(cols), _i64(cols))
    return out


def f32_pack_rounding(x):
    x = _c(x, np.float32).ravel()
    out = np.empty(x.size, np.uint16)
    lib().oracle_f32_to_f16_pack_rounding(_ptr(x), _ptr(out), _i64(x.size))
    return out


# ---- the reference's own compiled leaves (when built) -----------------------

def ref_pack_weight_f16(w):
    r = ref_lib()
    bits = np.ascontiguousarray(w).view(np.uint16)
    k, n = bits.shape
    out = np.empty(_tiles(n) * _tiles(k) * 1024, np.uint16)
    rc = r.ref_pack_weight_f16(_ptr(bits), _ptr(out), _u32(k), _u32(n), _u32(n))
    assert rc == 0
    return out


def ref_pack_weight_f32(w):
    r = ref_lib()
    w = _c(w, np.float32)
    k, n = w.shape
    out = np.empty(_tiles(n) * _tiles(k) * 1024, np.uint16)
    rc = r.ref_pack_weight_f32(_ptr(w), _ptr(out), _u32(k), _u32(n), _u32(n))
    assert rc == 0
    return out


def ref_pack_act_f16(a):
    r = ref_lib()
    bits = np.ascontiguousarray(a).view(np.uint16)
    rows, cols = bits.shape
    out = np.empty(_tiles(rows) * _tiles(cols) * 1024, np.uint16)
    rc = r.ref_pack_act_f16(_ptr(bits), _ptr(out), _u32(rows), _u32(cols), _u32(cols))
    assert rc == 0
    return out


def ref_unpack_acc_f16(tiles, rows, cols):
    r = ref_lib()
    tiles = _c(tiles, np.uint16)
    out = np.zeros((rows, cols), np.uint16)
    rc = r.ref_unpack_acc_f16(_ptr(tiles), _ptr(out), _u32(rows), _u32(cols), _u32(cols))
    assert rc == 0
    return out


def ref_unpack_acc_f32(tiles, rows, cols, res=None):
    r = ref_lib()
    tiles = _c(tiles, np.uint16)
    out = np.zeros((rows, cols), np.float32)
    rr = _c(res, np.float32) if res is not None else None
    rc = r.ref_unpack_acc_f32(_ptr(tiles), _ptr(out),
                              _ptr(rr) if rr is not None else None,
                              _u32(rows), _u32(cols), _u32(cols))
    assert rc == 0
    return out


# ---- synthetic inputs: the counter-based generator (three implementations, one byte stream) ----

_DTYPE_IDS = {np.dtype(np.float16): 1, np.dtype(np.float32): 2, np.dtype(np.int8): 4}
UNIFORM, NORMAL, INTEGERS = 0, 1, 2


def fill_random(shape, dtype, seed: int, dist: int, p0: float, p1: float, threads: int = 0):
    """The C++ loop of the generator (see hexmlir_oracle.cpp: Philox4x32-10, element i = word i&3
    of block i>>2)."""
    out = np.empty(shape, dtype)
    lib().oracle_fill_random(_ptr(out), _int(_DTYPE_IDS[out.dtype]), _i64(out.size), ctypes.c_uint64(seed),
                             _int(dist), _f32(p0), _f32(p1), _int(_nt(threads)))
    return out


def _philox_np(c0, c1, c2, c3, k0, k1):
    m0, m1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    mask, sh = np.uint64(0xFFFFFFFF), np.uint64(32)
    k0, k1 = np.uint64(k0), np.uint64(k1)
    for _ in range(10):
        p0, p1 = m0 * c0, m1 * c2          # 32 x 32 -> 64 bits, held in uint64
        c0, c1, c2, c3 = (p1 >> sh) ^ c1 ^ k0, p1 & mask, (p0 >> sh) ^ c3 ^ k1, p0 & mask
        k0, k1 = (k0 + np.uint64(0x9E3779B9)) & mask, (k1 + np.uint64(0xBB67AE85)) & mask
    return c0, c1, c2, c3


def fill_random_numpy(shape, dtype, seed: int, dist: int, p0: float, p1: float, start: int = 0, index=None):
    """numpy twin of the generator; `start` offsets the element index (or `index` names every
    element's index outright), so any slice of a large tensor can be drawn without the rest —
    what a counter-based generator is for."""
    n = int(np.prod(shape))
    i = np.arange(start, start + n, dtype=np.uint64) if index is None else np.asarray(index, np.uint64).reshape(-1)
    assert i.size == n
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    zero = np.zeros(n, np.uint64)
    f32 = np.float32
    if dist == NORMAL:
        total = np.zeros(n, np.uint64)
        for j in range(3):
            w = _philox_np(i & np.uint64(0xFFFFFFFF), i >> np.uint64(32), zero + np.uint64(j), zero + np.uint64(1),
                           k0, k1)
            for x in w:
                total += x >> np.uint64(12)
        z = total.astype(f32) * f32(2.0 ** -20) - f32(6.0)
        v = f32(p0) + f32(p1) * z
    else:
        blk = i >> np.uint64(2)
        w = _philox_np(blk & np.uint64(0xFFFFFFFF), blk >> np.uint64(32), zero, zero, k0, k1)
        x = np.choose((i & np.uint64(3)).astype(np.int64), w)
        if dist == INTEGERS:
            lo, hi = int(p0), int(p1)
            v = (x % np.uint64(hi - lo + 1)).astype(np.int64) + lo
        else:
            u = (x >> np.uint64(8)).astype(f32) * f32(2.0 ** -24)
            v = f32(p0) + u * (f32(p1) - f32(p0))
    return np.asarray(v).astype(dtype).reshape(shape)


def random_rows(r0: int, rows: int, ld: int, dtype, seed, dist, p0, p1):
    """Rows [r0, r0 + rows) of a row-major [*, ld] tensor filled by the generator."""
    return fill_random_numpy((rows, ld), dtype, seed, dist, p0, p1, start=r0 * ld)


def random_cols(c0: int, cols: int, rows: int, ld: int, dtype, seed, dist, p0, p1):
    """Columns [c0, c0 + cols) of a row-major [rows, ld] tensor filled by the generator."""
    idx = (np.arange(rows, dtype=np.uint64)[:, None] * np.uint64(ld) + np.uint64(c0)
           + np.arange(cols, dtype=np.uint64)[None, :])
    return fill_random_numpy((rows, cols), dtype, seed, dist, p0, p1, index=idx)
