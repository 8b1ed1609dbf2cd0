// Any-shape GEMM on the CUDA cores.
//
// The reference refuses its matrix engine for shapes that are not multiples of
// the 32-element tile edge or have M <= 4 and sends them to its vector path
// (plans "hmx-tail" / "hvx";
// qcom_hexagon_backend/include/hexagon/Dialect/Hmx/Transforms/HmxTarget.h:195-222).
// This file is that path here: shared-memory tiled, fp32 accumulation in
// ascending k (the oracle's order), every epilogue of the tensor-core kernels,
// no alignment or stride preconditions.  It is also the exact int8 -> int32
// contraction.  Not a performance path.
#include "common.h"

namespace b200 {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__device__ __forceinline__ __half silu_h(__half x) {
  __half e = __float2half_rn(__expf(-__half2float(x)));
  __half d = __float2half_rn(1.0f + __half2float(e));
  return __float2half_rn(__fdividef(__half2float(x), __half2float(d)));
}

template <int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const __half *__restrict__ A, const __half *__restrict__ B,
                 const __half *__restrict__ B2, void *__restrict__ Cv,
                 const void *__restrict__ Rv, int64_t M, int64_t N, int64_t K, int64_t lda,
                 int64_t ldb, int64_t ldc, int64_t ldr, int block_k, int res_mod, int res_rem) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN];
  __shared__ float B2s[EPI == EPI_SWIGLU ? TK : 1][TN];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  float acc[4][4] = {}, acc2[4][4] = {}, run[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      int r = i / TK, kk = i % TK;
      int64_t gm = m0 + r, gk = k0 + kk;
      As[kk][r] = (gm < M && gk < K) ? __half2float(A[gm * lda + gk]) : 0.0f;
    }
    for (int i = threadIdx.x; i < TK * TN; i += 256) {
      int kk = i / TN, c = i % TN;
      int64_t gk = k0 + kk, gn = n0 + c;
      bool ok = gk < K && gn < N;
      Bs[kk][c] = ok ? __half2float(B[gk * ldb + gn]) : 0.0f;
      if (EPI == EPI_SWIGLU) B2s[kk][c] = ok ? __half2float(B2[gk * ldb + gn]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4], b2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        b[j] = Bs[kk][tx * 4 + j];
        if (EPI == EPI_SWIGLU) b2[j] = B2s[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (EPI == EPI_SWIGLU) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
    if (EPI == EPI_KLOOP_F16 && ((k0 + TK) % block_k == 0 || k0 + TK >= K)) {
      // segment boundary: read the segment out as fp16, widen, add in fp32
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          run[i][j] += __half2float(__float2half_rn(acc[i][j]));
          acc[i][j] = 0.0f;
        }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm >= M || gn >= N) continue;
      if (EPI == EPI_F16) {
        ((__half *)Cv)[gm * ldc + gn] = __float2half_rn(acc[i][j]);
      } else if (EPI == EPI_KLOOP_F16) {
        ((__half *)Cv)[gm * ldc + gn] = __float2half_rn(run[i][j]);
      } else if (EPI == EPI_F32_RES) {
        float v = __half2float(__float2half_rn(acc[i][j]));
        if (Rv) v += ((const float *)Rv)[gm * ldr + gn];
        ((float *)Cv)[gm * ldc + gn] = v;
      } else if (EPI == EPI_F16_RES16) {
        const bool mine = res_mod <= 1 || (int)((gm >> 8) % res_mod) == res_rem;
        float v = __half2float(__float2half_rn(acc[i][j])) +
                  (mine ? __half2float(((const __half *)Rv)[gm * ldr + gn]) : 0.0f);
        ((__half *)Cv)[gm * ldc + gn] = __float2half_rn(v);
      } else {  // EPI_SWIGLU
        __half g = __float2half_rn(acc[i][j]), u = __float2half_rn(acc2[i][j]);
        ((__half *)Cv)[gm * ldc + gn] =
            __float2half_rn(__half2float(silu_h(g)) * __half2float(u));
      }
    }
}

__global__ void __launch_bounds__(256)
gemm_i8_simt_kernel(const int8_t *__restrict__ A, const int8_t *__restrict__ B,
                    int32_t *__restrict__ C, int64_t M, int64_t N, int64_t K, int64_t lda,
                    int64_t ldb, int64_t ldc) {
  __shared__ int As[TK][TM + 1];
  __shared__ int Bs[TK][TN];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  int acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      int r = i / TK, kk = i % TK;
      int64_t gm = m0 + r, gk = k0 + kk;
      As[kk][r] = (gm < M && gk < K) ? (int)A[gm * lda + gk] : 0;
    }
    for (int i = threadIdx.x; i < TK * TN; i += 256) {
      int kk = i / TN, c = i % TN;
      int64_t gk = k0 + kk, gn = n0 + c;
      Bs[kk][c] = (gk < K && gn < N) ? (int)B[gk * ldb + gn] : 0;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += As[kk][ty * 4 + i] * Bs[kk][tx * 4 + j];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < M && gn < N) C[gm * ldc + gn] = acc[i][j];
    }
}

}  // namespace

int launch_gemm_simt(const GemmArgs &g) {
  B200_TRY(ensure_ready());
  if (g.m <= 0 || g.n <= 0) return 0;
  if (g.epilogue == EPI_KLOOP_F16 && (g.block_k < TK || g.block_k % TK != 0))
    return set_error(B200MLIR_ERR_BAD_ARG, "klooped matmul: BLOCK_K=%d must be a multiple of %d",
                     g.block_k, TK);
  dim3 grid((unsigned)((g.n + TN - 1) / TN), (unsigned)((g.m + TM - 1) / TM));
  if (grid.y > 65535) return set_error(B200MLIR_ERR_UNSUPPORTED, "simt gemm: M too large");
  cudaStream_t s = ctx().stream;
  const __half *A = (const __half *)g.a, *B = (const __half *)g.b, *B2 = (const __half *)g.b2;
#define SIMT_LAUNCH(E)                                                                      \
  gemm_simt_kernel<E><<<grid, 256, 0, s>>>(A, B, B2, g.c, g.res, g.m, g.n, g.k, g.lda, g.ldb, \
                                           g.ldc, g.ldres, g.block_k, g.res_mod, g.res_rem)
  switch (g.epilogue) {
    case EPI_F16: SIMT_LAUNCH(EPI_F16); break;
    case EPI_F32_RES: SIMT_LAUNCH(EPI_F32_RES); break;
    case EPI_KLOOP_F16: SIMT_LAUNCH(EPI_KLOOP_F16); break;
    case EPI_F16_RES16: SIMT_LAUNCH(EPI_F16_RES16); break;
    case EPI_SWIGLU: SIMT_LAUNCH(EPI_SWIGLU); break;
    default: return set_error(B200MLIR_ERR_BAD_ARG, "simt gemm: unknown epilogue %d", g.epilogue);
  }
#undef SIMT_LAUNCH
  return check_launch("gemm_simt");
}

int launch_gemm_i8_simt(const int8_t *a, const int8_t *b, int32_t *c, int64_t m, int64_t n,
                        int64_t k, int64_t lda, int64_t ldb, int64_t ldc) {
  B200_TRY(ensure_ready());
  if (m <= 0 || n <= 0) return 0;
  dim3 grid((unsigned)((n + TN - 1) / TN), (unsigned)((m + TM - 1) / TM));
  if (grid.y > 65535) return set_error(B200MLIR_ERR_UNSUPPORTED, "simt gemm: M too large");
  gemm_i8_simt_kernel<<<grid, 256, 0, ctx().stream>>>(a, b, c, m, n, k, lda, ldb, ldc);
  return check_launch("gemm_i8_simt");
}

}  // namespace b200
