// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// CPU restatement of the arithmetic the hexagon-mlir backend lowers its
// operators into.  It exists to check the CUDA path and to serve as the timed
// CPU baseline; nothing in the shipped library links, loads or calls it.
//
// Parity pinning: the layout functions are pinned against the reference's own
// HMXLayout.c compiled on the host (see ref_layout_shim.c in this directory)
// and against the closed-form byte rule of its contract test.  The engine
// arithmetic (HMXAPI.c) and the compiler-generated vector loops cannot run
// without Hexagon silicon / LLVM, and the SDK math library (qhmath_hvx, Hexagon
// SDK 6.4.0.2) is not in the reference tree: for those pieces parity is
// UNPINNED at the bit level and is anchored on the reference's end-to-end test
// tolerances instead (matmul rel<2e-3, softmax atol 1e-3, rms_norm/silu 1e-2).
//
// Every function cites the reference file:line it follows (paths relative to
// the reference project root).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

typedef _Float16 f16;

namespace {

template <class F>
void parallel_for(int64_t n, int nthreads, F f) {
  if (nthreads < 1) nthreads = 1;
  if ((int64_t)nthreads > n) nthreads = (int)std::max<int64_t>(n, 1);
  if (nthreads == 1) { f((int64_t)0, n); return; }
  std::vector<std::thread> pool;
  int64_t chunk = (n + nthreads - 1) / nthreads;
  for (int t = 0; t < nthreads; ++t) {
    int64_t lo = t * chunk, hi = std::min<int64_t>(n, lo + chunk);
    if (lo >= hi) break;
    pool.emplace_back([=] { f(lo, hi); });
  }
  for (auto &th : pool) th.join();
}

// One output row of C = A·B, fp32 accumulation in ascending k.  A product of
// two fp16 values is exact in fp32 (11+11 significant bits), so the only
// roundings are the fp32 adds and the final conversions.
//
// block_k == 0: whole-K form — one accumulator chain, one fp16 rounding
//   (test/python/triton/test_matmul.py:64-67; engine semantics
//   qcom_hexagon_backend/bin/runtime/hmx/src/HMXAPI.c:36-55).
// block_k  > 0: K-segmented form — each BLOCK_K segment is accumulated wide,
//   read out as fp16, widened, and added to a running fp32
//   (test/python/triton/test_matmul_kloop.py:87-98;
//   qcom_hexagon_backend/bin/runtime/hmx/src/HMXLayout.c:880-901).
void gemm_row(const f16 *a_row, const float *Bf, float *acc, float *seg,
              int64_t N, int64_t K, int64_t block_k) {
  if (block_k <= 0) {
    std::fill(acc, acc + N, 0.0f);
    for (int64_t k = 0; k < K; ++k) {
      float a = (float)a_row[k];
      const float *b = Bf + k * N;
      for (int64_t j = 0; j < N; ++j) acc[j] += a * b[j];
    }
    return;
  }
  std::fill(acc, acc + N, 0.0f);
  for (int64_t k0 = 0; k0 < K; k0 += block_k) {
    std::fill(seg, seg + N, 0.0f);
    int64_t k1 = std::min(K, k0 + block_k);
    for (int64_t k = k0; k < k1; ++k) {
      float a = (float)a_row[k];
      const float *b = Bf + k * N;
      for (int64_t j = 0; j < N; ++j) seg[j] += a * b[j];
    }
    for (int64_t j = 0; j < N; ++j) acc[j] += (float)(f16)seg[j];
  }
}

std::vector<float> widen(const f16 *B, int64_t K, int64_t N, int64_t ldb,
                         int nthreads) {
  std::vector<float> Bf((size_t)K * N);
  parallel_for(K, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t k = lo; k < hi; ++k)
      for (int64_t j = 0; j < N; ++j) Bf[k * N + j] = (float)B[k * ldb + j];
  });
  return Bf;
}

}  // namespace

extern "C" {

int oracle_hw_threads() {
  unsigned n = std::thread::hardware_concurrency();
  return n ? (int)n : 1;
}

// fp16 GEMM, fp32 accumulate, fp16 output (overwrites C, never accumulates:
// qcom_hexagon_backend/include/hexagon/Dialect/Hmx/IR/HmxOps.td:81-84).
void oracle_gemm_f16(const f16 *A, const f16 *B, f16 *C, int64_t M, int64_t N,
                     int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                     int64_t block_k, int nthreads) {
  std::vector<float> Bf = widen(B, K, N, ldb, nthreads);
  parallel_for(M, nthreads, [&](int64_t lo, int64_t hi) {
    std::vector<float> acc(N), seg(N);
    for (int64_t i = lo; i < hi; ++i) {
      gemm_row(A + i * lda, Bf.data(), acc.data(), seg.data(), N, K, block_k);
      for (int64_t j = 0; j < N; ++j) C[i * ldc + j] = (f16)acc[j];
    }
  });
}

// fp32 read-out with optional fp32 residual: the engine's result is always an
// fp16 tile; the f32 image is that tile widened (x1.0, exact) and the residual
// is added in fp32 afterwards
// (qcom_hexagon_backend/bin/runtime/hmx/src/HMXLayout.c:876-901).
void oracle_gemm_f16_f32out(const f16 *A, const f16 *B, float *C,
                            const float *R, int64_t M, int64_t N, int64_t K,
                            int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr,
                            int nthreads) {
  std::vector<float> Bf = widen(B, K, N, ldb, nthreads);
  parallel_for(M, nthreads, [&](int64_t lo, int64_t hi) {
    std::vector<float> acc(N), seg(N);
    for (int64_t i = lo; i < hi; ++i) {
      gemm_row(A + i * lda, Bf.data(), acc.data(), seg.data(), N, K, 0);
      for (int64_t j = 0; j < N; ++j) {
        float v = (float)(f16)acc[j];
        if (R) v += R[i * ldr + j];
        C[i * ldc + j] = v;
      }
    }
  });
}

// int8 x int8 -> int32, exact.  The reference sends integer matmuls to exact
// integer vector loops (refusal reason "unsupported-dtype",
// qcom_hexagon_backend/include/hexagon/Dialect/Hmx/Transforms/HmxTarget.h:198-200).
void oracle_gemm_i8_i32(const int8_t *A, const int8_t *B, int32_t *C,
                        int64_t M, int64_t N, int64_t K, int nthreads) {
  parallel_for(M, nthreads, [&](int64_t lo, int64_t hi) {
    std::vector<int32_t> acc(N);
    for (int64_t i = lo; i < hi; ++i) {
      std::fill(acc.begin(), acc.end(), 0);
      for (int64_t k = 0; k < K; ++k) {
        int32_t a = A[i * K + k];
        const int8_t *b = B + k * N;
        for (int64_t j = 0; j < N; ++j) acc[j] += a * (int32_t)b[j];
      }
      std::memcpy(C + i * N, acc.data(), sizeof(int32_t) * N);
    }
  });
}

// w8a16: the reference has no such op; its own lowering of one would be a
// dequantising elementwise generic (sitofp + mulf, then truncf to f16 —
// qcom_hexagon_backend/lib/Conversion/LinalgToLLVM/LinalgToLLVMPass.cpp:322-328)
// followed by the fp16 matmul above.  W16[k,n] = f16(f32(q[k,n]) * f32(s[n])).
void oracle_w8a16(const f16 *A, const int8_t *Wq, const f16 *scales, f16 *C,
                  int64_t M, int64_t N, int64_t K, int nthreads) {
  std::vector<float> Wf((size_t)K * N);
  parallel_for(K, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t k = lo; k < hi; ++k)
      for (int64_t j = 0; j < N; ++j)
        Wf[k * N + j] = (float)(f16)((float)Wq[k * N + j] * (float)scales[j]);
  });
  parallel_for(M, nthreads, [&](int64_t lo, int64_t hi) {
    std::vector<float> acc(N), seg(N);
    for (int64_t i = lo; i < hi; ++i) {
      gemm_row(A + i * K, Wf.data(), acc.data(), seg.data(), N, K, 0);
      for (int64_t j = 0; j < N; ++j) C[i * N + j] = (f16)acc[j];
    }
  });
}

// Row softmax as the backend lowers it
// (docs/tutorials/triton/softmax.md:167-219; source kernel
// test/python/triton/test_softmax.py:39-70):
//   1. m = max_j x[j]                       running max in f16
//   2. e[j] = f16(exp(f32(x[j] - m)))       subtract in f16, exp in f32, store f16
//   3. s = sum_j f32(e[j])                  f32 sum of the f16-rounded values
//   4. y[j] = f16(f32(e[j]) / s)
void oracle_softmax_f16(const f16 *X, f16 *Y, int64_t rows, int64_t cols,
                        int nthreads) {
  parallel_for(rows, nthreads, [&](int64_t lo, int64_t hi) {
    std::vector<f16> e(cols);
    for (int64_t r = lo; r < hi; ++r) {
      const f16 *x = X + r * cols;
      f16 m = x[0];
      for (int64_t j = 1; j < cols; ++j) m = x[j] > m ? x[j] : m;
      float s = 0.0f;
      for (int64_t j = 0; j < cols; ++j) {
        f16 z = (f16)((float)x[j] - (float)m);  // f16 subtract (exact in f32, then RNE)
        e[j] = (f16)std::exp((float)z);
        s += (float)e[j];
      }
      for (int64_t j = 0; j < cols; ++j) Y[r * cols + j] = (f16)((float)e[j] / s);
    }
  });
}

void oracle_softmax_f32(const float *X, float *Y, int64_t rows, int64_t cols,
                        int nthreads) {
  parallel_for(rows, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t r = lo; r < hi; ++r) {
      const float *x = X + r * cols;
      float m = x[0];
      for (int64_t j = 1; j < cols; ++j) m = std::max(m, x[j]);
      float s = 0.0f;
      for (int64_t j = 0; j < cols; ++j) {
        float e = std::exp(x[j] - m);
        Y[r * cols + j] = e;
        s += e;
      }
      for (int64_t j = 0; j < cols; ++j) Y[r * cols + j] /= s;
    }
  });
}

// RMSNorm (test/python/triton/test_rms_norm.py:45-60): ms = sum(x*x)/N,
// rms = sqrt(ms + eps), y = (x / rms) * g.  The row reduce upcasts to f32
// (qcom_hexagon_backend/lib/Conversion/LinalgToLLVM/VectorRowReducePass.cpp:18-22)
// and x/sqrt(.) becomes x*rsqrt(.)
// (qcom_hexagon_backend/lib/Transforms/FastInversePass.cpp:99-137).
void oracle_rmsnorm_f16(const f16 *X, const f16 *G, f16 *Y, int64_t rows,
                        int64_t cols, float eps, int nthreads) {
  parallel_for(rows, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t r = lo; r < hi; ++r) {
      const f16 *x = X + r * cols;
      float ss = 0.0f;
      for (int64_t j = 0; j < cols; ++j) ss += (float)x[j] * (float)x[j];
      float inv = 1.0f / std::sqrt(ss / (float)cols + eps);
      for (int64_t j = 0; j < cols; ++j)
        Y[r * cols + j] = (f16)((float)x[j] * inv * (float)G[j]);
    }
  });
}

void oracle_rmsnorm_f32(const float *X, const float *G, float *Y, int64_t rows,
                        int64_t cols, float eps, int nthreads) {
  parallel_for(rows, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t r = lo; r < hi; ++r) {
      const float *x = X + r * cols;
      float ss = 0.0f;
      for (int64_t j = 0; j < cols; ++j) ss += x[j] * x[j];
      float inv = 1.0f / std::sqrt(ss / (float)cols + eps);
      for (int64_t j = 0; j < cols; ++j) Y[r * cols + j] = x[j] * inv * G[j];
    }
  });
}

// SiLU (test/python/triton/test_silu.py:45-49):
//   x / (1 + f16(exp(f32(-x))))  with the add and the divide in the tensor dtype.
static inline f16 silu_one(f16 x) {
  f16 e = (f16)std::exp(-(float)x);
  f16 d = (f16)(1.0f + (float)e);
  return (f16)((float)x / (float)d);
}

void oracle_silu_f16(const f16 *X, f16 *Y, int64_t n, int nthreads) {
  parallel_for(n, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) Y[i] = silu_one(X[i]);
  });
}

void oracle_silu_f32(const float *X, float *Y, int64_t n, int nthreads) {
  parallel_for(n, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) Y[i] = X[i] / (1.0f + std::exp(-X[i]));
  });
}

// SwiGLU = silu(gate) * up.  Not a reference kernel: it is the two-input fused
// elementwise generic the fusion pass forms from the ops above
// (qcom_hexagon_backend/lib/Conversion/LinalgToLLVM/FusionPass.cpp).
void oracle_swiglu_f16(const f16 *Gt, const f16 *Up, f16 *Y, int64_t n,
                       int nthreads) {
  parallel_for(n, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i)
      Y[i] = (f16)((float)silu_one(Gt[i]) * (float)Up[i]);
  });
}

// Residual add through the f32 read-out path:
//   out = f16(f32(tile_f16) + f32(res))
// (qcom_hexagon_backend/bin/runtime/hmx/src/HMXLayout.c:880-901).
void oracle_add_f16(const f16 *A, const f16 *B, f16 *Y, int64_t n, int nthreads) {
  parallel_for(n, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) Y[i] = (f16)((float)A[i] + (float)B[i]);
  });
}

// Llama-style MLP block as a composition, fp16 wherever a tensor is
// materialised between stages:
//   h = rmsnorm(x, gain); g = h·Wg; u = h·Wu; a = swiglu(g, u);
//   y = f16(f32(f16(a·Wd)) + f32(x))
// Rows [row_lo, row_hi) only, so a bounded sample of tokens can be timed.
void oracle_mlp_f16(const f16 *X, const f16 *Gain, const f16 *Wg, const f16 *Wu,
                    const f16 *Wd, f16 *Y, int64_t T, int64_t D, int64_t F,
                    float eps, int nthreads) {
  std::vector<f16> h((size_t)T * D), g((size_t)T * F), u((size_t)T * F),
      a((size_t)T * F), d((size_t)T * D);
  oracle_rmsnorm_f16(X, Gain, h.data(), T, D, eps, nthreads);
  oracle_gemm_f16(h.data(), Wg, g.data(), T, F, D, D, F, F, 0, nthreads);
  oracle_gemm_f16(h.data(), Wu, u.data(), T, F, D, D, F, F, 0, nthreads);
  oracle_swiglu_f16(g.data(), u.data(), a.data(), T * F, nthreads);
  oracle_gemm_f16(a.data(), Wd, d.data(), T, D, F, F, D, D, 0, nthreads);
  oracle_add_f16(d.data(), X, Y, T * D, nthreads);
}

// Attention block (QK·softmax·PV), one row of queries at a time, in the order of the
// reference's flash-attention kernel (test/python/triton/test_flash_attention.py:43-113 is
// the loop over key blocks, :172-195 the prologue and the final division):
//   qk_scale = sm_scale * 1.44269504;  m = -99999999999999, l = 1, acc = 0
//   per BLOCK_N keys:  qk = q·kᵀ;  m' = max(m, max_j(qk)·qk_scale);  p = exp2(qk·qk_scale − m');
//                      alpha = exp2(m − m');  l = l·alpha + Σp;  acc = acc·alpha + p·v;  m = m'
//   out = acc / l
// Both products take fp16 operands with a wide accumulate: Q, K, V arrive as fp16 (an fp32
// tensor is rounded by the pack leaf, same file :239-246) and p is rounded to fp16 before p·v.
// flags bit 0: each product's read-out is rounded to fp16 before it is used in fp32, as the
//              engine's read-out tile is (include/hexagon/Dialect/Hmx/IR/HmxOps.td:308-316);
// flags bit 1: p stays fp32 (what the kernel source computes when no operand is quantised;
//              used to pin this function against the kernel run by Triton's interpreter).
// flags bit 2: causal — query i sees keys 0..i only (STAGE = 3 of the kernel's signature,
//              test_flash_attention.py:183-185; the reference's inner loop implements STAGE = 1 only,
//              so this form has no reference output to pin against and is checked against torch).
// Q, K, V: [BH, N, D] contiguous; O: [BH, N, D] fp32.
void oracle_attention_f16(const f16 *Q, const f16 *K, const f16 *V, float *O, int64_t BH,
                          int64_t N, int64_t D, double sm_scale, int block_n, int flags,
                          int nthreads) {
  const float qk_scale = (float)(sm_scale * 1.44269504);
  const bool round_out = flags & 1, p_f32 = flags & 2, causal = flags & 4;
  parallel_for(BH * N, nthreads, [&](int64_t lo, int64_t hi) {
    std::vector<float> qk(block_n), p(block_n), acc(D), pv(D), qf(D);
    for (int64_t row = lo; row < hi; ++row) {
      const int64_t bh = row / N;
      const f16 *q = Q + row * D;
      const f16 *Kb = K + bh * N * D, *Vb = V + bh * N * D;
      for (int64_t d = 0; d < D; ++d) qf[d] = (float)q[d];
      float m = -99999999999999.0f, l = 1.0f;
      std::fill(acc.begin(), acc.end(), 0.0f);
      const int64_t last_key = causal ? row - bh * N : N - 1;
      for (int64_t n0 = 0; n0 <= last_key; n0 += block_n) {
        const int64_t nb = std::min<int64_t>(block_n, last_key + 1 - n0);
        float mx = -INFINITY;
        for (int64_t j = 0; j < nb; ++j) {
          const f16 *kr = Kb + (n0 + j) * D;
          float a = 0.0f;
          for (int64_t d = 0; d < D; ++d) a += qf[d] * (float)kr[d];
          if (round_out) a = (float)(f16)a;
          qk[j] = a;
          mx = std::max(mx, a);
        }
        const float m_new = std::max(m, mx * qk_scale);
        float lsum = 0.0f;
        for (int64_t j = 0; j < nb; ++j) {
          const float e = exp2f(qk[j] * qk_scale - m_new);
          lsum += e;
          p[j] = p_f32 ? e : (float)(f16)e;
        }
        const float alpha = exp2f(m - m_new);
        l = l * alpha + lsum;
        std::fill(pv.begin(), pv.end(), 0.0f);
        for (int64_t j = 0; j < nb; ++j) {
          const f16 *vr = Vb + (n0 + j) * D;
          const float pj = p[j];
          for (int64_t d = 0; d < D; ++d) pv[d] += pj * (float)vr[d];
        }
        for (int64_t d = 0; d < D; ++d)
          acc[d] = acc[d] * alpha + (round_out ? (float)(f16)pv[d] : pv[d]);
        m = m_new;
      }
      float *o = O + row * D;
      for (int64_t d = 0; d < D; ++d) o[d] = acc[d] / l;
    }
  });
}

// Two-phase ("online") softmax over column blocks, fp32
// (test/python/triton/test_online_softmax.py:27-77): phase 1 keeps a running maximum m and a
// running sum l = l·exp(m − m') + Σ exp(x − m') per block; phase 2 writes exp(x − m)/l.
void oracle_online_softmax_f32(const float *X, float *Y, int64_t rows, int64_t cols,
                               int64_t block_cols, int nthreads) {
  parallel_for(rows, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t r = lo; r < hi; ++r) {
      const float *x = X + r * cols;
      float m = -INFINITY, l = 0.0f;
      for (int64_t c0 = 0; c0 < cols; c0 += block_cols) {
        const int64_t c1 = std::min(cols, c0 + block_cols);
        float mx = m;
        for (int64_t c = c0; c < c1; ++c) mx = std::max(mx, x[c]);
        float s = 0.0f;
        for (int64_t c = c0; c < c1; ++c) s += expf(x[c] - mx);
        l = l * expf(m - mx) + s;
        m = mx;
      }
      for (int64_t c = 0; c < cols; ++c) Y[r * cols + c] = expf(x[c] - m) / l;
    }
  });
}

// ---- tile ("crouton") layout -------------------------------------------
// One 32x32 fp16 tile is 2048 bytes; element (r, c) lives at byte
//   128*(r>>1) + 4*c + 2*(r&1)
// (qcom_hexagon_backend/bin/runtime/hmx/src/HMXLayout.c:9-14; closed form
// qcom_hexagon_backend/bin/runtime/test/test_hmx_layout_permutation_contract.py:137-148).
static inline int64_t tile_elem(int r, int c) {
  return (128 * (r >> 1) + 4 * c + 2 * (r & 1)) / 2;
}

// Activation pack: row-major [rows, cols] (row stride `stride` elements) ->
// tile grid [Mt, Kt]; out-of-range elements read as zero
// (HMXLayout.c:70-151; declaration hmx/include/HMXAPI.h:81-106).
void oracle_pack_act_f16(const uint16_t *src, uint16_t *dst, int64_t rows,
                         int64_t cols, int64_t stride) {
  int64_t Mt = (rows + 31) / 32, Kt = (cols + 31) / 32;
  for (int64_t tr = 0; tr < Mt; ++tr)
    for (int64_t tc = 0; tc < Kt; ++tc) {
      uint16_t *t = dst + (tr * Kt + tc) * 1024;
      for (int r = 0; r < 32; ++r)
        for (int c = 0; c < 32; ++c) {
          int64_t gr = tr * 32 + r, gc = tc * 32 + c;
          t[tile_elem(r, c)] = (gr < rows && gc < cols) ? src[gr * stride + gc] : 0;
        }
    }
}

// Weight pack: row-major [K, N] -> image [Nt, Kt, 16, 32, 2]; physical
// (n_tile, k_tile, j, c, h) holds logical (k = 32*k_tile + 2*j + h,
// n = 32*n_tile + c)
// (qcom_hexagon_backend/backend/hmx_weight_prepack.py:170-183;
// qcom_hexagon_backend/test/test_hmx_weight_prepack_f32.py:46-52).
void oracle_pack_weight_f16(const uint16_t *src, uint16_t *dst, int64_t K,
                            int64_t N, int64_t stride) {
  int64_t Kt = (K + 31) / 32, Nt = (N + 31) / 32;
  for (int64_t nt = 0; nt < Nt; ++nt)
    for (int64_t kt = 0; kt < Kt; ++kt) {
      uint16_t *t = dst + (nt * Kt + kt) * 1024;
      for (int j = 0; j < 16; ++j)
        for (int c = 0; c < 32; ++c)
          for (int h = 0; h < 2; ++h) {
            int64_t k = kt * 32 + 2 * j + h, n = nt * 32 + c;
            t[(j * 32 + c) * 2 + h] = (k < K && n < N) ? src[k * stride + n] : 0;
          }
    }
}

// f32 source: "+0.0f" (maps -0 to +0) then round-to-nearest-even to fp16
// (HMXLayout.c:257-264; host twin hmx_weight_prepack.py:197-212).  NaN
// payloads are not reproduced, as the reference's host twin documents.
void oracle_f32_to_f16_pack_rounding(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    f16 h = (f16)(src[i] + 0.0f);
    std::memcpy(dst + i, &h, 2);
  }
}

// Read-out: tile row [Nt tiles] -> row-major fp16, first dst_cols columns of
// rows tile_row*32 .. (HMXLayout.c:776-863).
void oracle_unpack_acc_f16(const uint16_t *tiles, uint16_t *dst, int64_t rows,
                           int64_t cols, int64_t stride) {
  int64_t Mt = (rows + 31) / 32, Nt = (cols + 31) / 32;
  for (int64_t tr = 0; tr < Mt; ++tr)
    for (int64_t tc = 0; tc < Nt; ++tc) {
      const uint16_t *t = tiles + (tr * Nt + tc) * 1024;
      for (int r = 0; r < 32; ++r)
        for (int c = 0; c < 32; ++c) {
          int64_t gr = tr * 32 + r, gc = tc * 32 + c;
          if (gr < rows && gc < cols) dst[gr * stride + gc] = t[tile_elem(r, c)];
        }
    }
}

}  // extern "C"

// ---- synthetic inputs: one counter-based generator, the same bytes everywhere -------------
// Philox4x32-10 (Salmon et al., SC'11).  Element i of a tensor takes word (i & 3) of the block
// with counter (i >> 2, stream, lane) and key = seed; no state, so the GPU kernel of the library
// (b200mlir_fill_random), this loop and the numpy twin in oracle/__init__.py produce identical
// bytes for the same (seed, distribution, parameters).  No counterpart in the reference, whose
// tests draw inputs with torch.rand/randn; BASELINE's shapes and distributions are kept.
//   dist 0: uniform [p0, p1):  p0 + (w >> 8) * 2^-24 * (p1 - p0), unfused multiply then add
//   dist 1: normal(p0, p1) as an Irwin-Hall sum of twelve 20-bit uniforms (exact integer sum S,
//           z = S * 2^-20 - 6, tails end at 6 sigma), x = p0 + p1 * z
//   dist 2: integers uniform in [p0, p1] (w mod range)
static inline void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                 uint32_t out[4]) {
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

static inline float fill_value(int64_t i, uint64_t seed, int dist, float p0, float p1) {
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  const uint32_t blk_lo = (uint32_t)((uint64_t)i >> 2), blk_hi = (uint32_t)((uint64_t)i >> 34);
  uint32_t w[4];
  if (dist == 1) {
    uint32_t sum = 0;
    for (uint32_t j = 0; j < 3; ++j) {
      philox4x32_10((uint32_t)((uint64_t)i), (uint32_t)((uint64_t)i >> 32), j, 1u, k0, k1, w);
      sum += (w[0] >> 12) + (w[1] >> 12) + (w[2] >> 12) + (w[3] >> 12);
    }
    const float z = (float)sum * 9.5367431640625e-07f - 6.0f;  // 2^-20
    const float t = p1 * z;
    return p0 + t;
  }
  philox4x32_10(blk_lo, blk_hi, 0u, 0u, k0, k1, w);
  const uint32_t x = w[i & 3];
  if (dist == 2) {
    const int lo = (int)p0, hi = (int)p1;
    return (float)(lo + (int)(x % (uint32_t)(hi - lo + 1)));
  }
  const float u = (float)(x >> 8) * 5.9604644775390625e-08f;  // 2^-24
  const float t = u * (p1 - p0);
  return p0 + t;
}

extern "C" void oracle_fill_random(void *dst, int dtype_id, int64_t n, uint64_t seed, int dist, float p0, float p1,
                                   int nthreads) {
  parallel_for(n, nthreads, [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
      const float v = fill_value(i, seed, dist, p0, p1);
      if (dtype_id == 1) ((f16 *)dst)[i] = (f16)v;          // dtype ids of the raw tensor files: 1 f16
      else if (dtype_id == 2) ((float *)dst)[i] = v;         // 2 f32
      else ((int8_t *)dst)[i] = (int8_t)(int)v;              // 4 int8
    }
  });
}
