// w8a16 GEMM: fp16 activations x int8 weights with per-output-channel fp16
// scales, fp32 accumulate, fp16 output.
//
// The reference has no such operator (its matrix engine admits f16/f32 only,
// include/hexagon/Dialect/Hmx/IR/HmxDType.h:59,69); what it does have, and
// what this file keeps, is the weight-residency contract: a weight is packed
// once into the layout the engine consumes and the same resident image is used
// by every later launch (lib/Dialect/Hmx/Transforms/WeightResidentPass.cpp:9-93,
// backend/hmx_weight_prepack.py:124-212).
//
// The product path (`w8a16_matmul`, the registry's resident image) is the tcgen05 kernel of
// w8a16_tmem.cu; this file holds the row-pass loop around it and the one entry point that
// may not allocate, which keeps its own kernels:
//
// Caller-built image of that entry: [strip = n/32][kstep = k/16][lane 0..31][16 bytes].  The
// 16 bytes of a lane are exactly the B fragments of four m16n8k16 MMAs (four n8 tiles of the
// strip) for one k16 step, stored as q+128 so that two bytes become two fp16 values with one
// byte-permute and one subtract.  A warp streams one strip: 512 contiguous bytes per k-step;
// the work list (n-block, k-step) is cut into equal contiguous ranges over 2 CTAs per SM,
// partial sums go to the fixed fp32 scratch with red.add and a small second kernel scales,
// rounds and re-zeroes it.
#include <mma.h>

#include <mutex>
#include <unordered_map>

#include "common.h"

namespace b200 {
namespace {

constexpr int WARPS = 8;              // strips per CTA (n-block = 256 columns)
constexpr int KC_STEPS = 64;          // k16 steps of A held in shared memory at once (1024 k)
constexpr int A_PITCH = KC_STEPS * 16 + 8;  // halves; +8 keeps ldmatrix conflict-free

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Two biased bytes -> two fp16 values: 0x64xx is 1024 + xx, minus 1152 gives xx - 128.
__device__ __forceinline__ uint32_t dq2(uint32_t word, uint32_t selector) {
  uint32_t h;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(h) : "r"(word), "r"(0x64646464u), "r"(selector));
  const uint32_t bias = 0x64806480u;  // half2(1152, 1152)
  uint32_t out;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(out) : "r"(h), "r"(bias));
  return out;
}

// MT = number of 16-row tiles of A (M <= 16*MT).  The image is strip-major [strip][kstep][lane].
template <int MT>
__global__ void __launch_bounds__(WARPS * 32, MT >= 4 ? 1 : 2)
w8a16_stream_kernel(const __half *__restrict__ A, int64_t lda, const uint4 *__restrict__ image,
                    float *__restrict__ ws, int M, int N, int K, int ksteps, int n_blocks,
                    int n_strips) {
  extern __shared__ __half a_smem[];  // [MT*16][A_PITCH]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t total = (int64_t)n_blocks * ksteps;
  const int64_t u_begin = total * blockIdx.x / gridDim.x;
  const int64_t u_end = total * (blockIdx.x + 1) / gridDim.x;

  int64_t u = u_begin;
  while (u < u_end) {
    const int nb = (int)(u / ksteps);
    const int ks0 = (int)(u - (int64_t)nb * ksteps);
    const int64_t want_end = (int64_t)ks0 + (u_end - u);
    int ks1 = want_end < (int64_t)ksteps ? (int)want_end : ksteps;
    if (ks1 - ks0 > KC_STEPS) ks1 = ks0 + KC_STEPS;
    const int nsteps = ks1 - ks0;
    const int strip = nb * WARPS + warp;

    // stage A[:, ks0*16 : ks1*16] (zero rows beyond M, zero columns beyond K)
    __syncthreads();
    const int vec_per_row = nsteps * 2;  // 16-byte vectors
    for (int i = threadIdx.x; i < MT * 16 * vec_per_row; i += WARPS * 32) {
      const int r = i / vec_per_row, v = i - r * vec_per_row;
      const int k = ks0 * 16 + v * 8;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < M && k < K) val = *reinterpret_cast<const uint4 *>(A + (int64_t)r * lda + k);
      *reinterpret_cast<uint4 *>(a_smem + r * A_PITCH + v * 8) = val;
    }
    __syncthreads();

    if (strip < n_strips) {
      float acc[MT][4][4];
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[m][j][e] = 0.0f;

      // address of this lane's 16 bytes for local step s (global k-step ks0 + s)
      auto wptr = [&](int s) -> const uint4 * {
        const int ks = ks0 + s;
        return image + ((int64_t)strip * ksteps + ks) * 32 + lane;
      };
      // ldmatrix source row/col of this lane inside a 16x16 A tile
      const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int lcol = (lane >> 4) * 8;
      const uint32_t a_base =
          (uint32_t)__cvta_generic_to_shared(a_smem) + (uint32_t)(lrow * A_PITCH + lcol) * 2u;

      constexpr int PF = 8;  // weight vectors in flight per lane
      uint4 wbuf[PF];
#pragma unroll
      for (int i = 0; i < PF; ++i)
        if (i < nsteps) wbuf[i] = __ldg(wptr(i));

      for (int s0 = 0; s0 < nsteps; s0 += PF) {
#pragma unroll
        for (int i = 0; i < PF; ++i) {
          const int s = s0 + i;
          if (s >= nsteps) break;
          const uint4 w = wbuf[i];
          if (s + PF < nsteps) wbuf[i] = __ldg(wptr(s + PF));
          const uint32_t words[4] = {w.x, w.y, w.z, w.w};
          uint32_t b[4][2];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            b[j][0] = dq2(words[j], 0x5140u);  // k = 2t, 2t+1
            b[j][1] = dq2(words[j], 0x5342u);  // k = 2t+8, 2t+9
          }
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            uint32_t a[4];
            ldmatrix_x4(a, a_base + (uint32_t)((m * 16 * A_PITCH + s * 16) * 2));
#pragma unroll
            for (int j = 0; j < 4; ++j) mma_16816(acc[m][j], a, b[j][0], b[j][1]);
          }
        }
      }

      // flush partial sums: c0,c1 -> (row g, cols 2t,2t+1); c2,c3 -> (row g+8, ...)
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = strip * 32 + j * 8 + 2 * t;
          const int r0 = m * 16 + g, r1 = r0 + 8;
          if (col < N) {
            if (r0 < M) {
              atomicAdd(ws + (int64_t)r0 * N + col, acc[m][j][0]);
              if (col + 1 < N) atomicAdd(ws + (int64_t)r0 * N + col + 1, acc[m][j][1]);
            }
            if (r1 < M) {
              atomicAdd(ws + (int64_t)r1 * N + col, acc[m][j][2]);
              if (col + 1 < N) atomicAdd(ws + (int64_t)r1 * N + col + 1, acc[m][j][3]);
            }
          }
        }
    }
    u += nsteps;
  }
}

// C = f16(ws * scale[n]).  (The scratch is cleared at the start of every call, not here.)
__global__ void __launch_bounds__(256)
w8a16_finalize_kernel(float *__restrict__ ws, const __half *__restrict__ scales,
                      __half *__restrict__ C, int M, int N, int64_t ldc) {
  const int64_t total = (int64_t)M * N;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * 256) {
    const int r = (int)(i / N), c = (int)(i - (int64_t)r * N);
    const float v = ws[i];
    C[(int64_t)r * ldc + c] = __float2half_rn(v * __half2float(scales[c]));
  }
}

}  // namespace

int launch_w8a16(const __half *a, const W8A16Weight &w, __half *c, int64_t m, int64_t lda,
                 int64_t ldc) {
  B200_TRY(ensure_ready());
  if (m <= 0 || w.n <= 0) return 0;
  if (((uintptr_t)a & 15u) || lda % 8)
    return set_error(B200MLIR_ERR_BAD_ARG,
                     "w8a16: activations must be 16-byte aligned with a row stride multiple of 8");
  if (w.k % 8) return set_error(B200MLIR_ERR_BAD_ARG, "w8a16: K must be a multiple of 8");
  if (m > (int64_t)ctx().opt.w8a16_expand_rows && w.w16) {
    // many rows: compute-bound; the expanded fp16 weight goes through the fp16 GEMM
    GemmArgs g;
    g.a = a; g.b = w.w16; g.c = c;
    g.m = m; g.n = w.n; g.k = w.k;
    g.lda = lda; g.ldb = w.n; g.ldc = ldc;
    g.epilogue = EPI_F16;
    g.b_kblocked = true;  // the registry's expanded weight is the K-blocked image
    return gemm_dispatch(g);
  }
  // rows in passes of at most 128 (the widest activation tile the kernel holds)
  for (int64_t m0 = 0; m0 < m; m0 += 128) {
    const int64_t mp = (m - m0) < 128 ? (m - m0) : 128;
    B200_TRY(launch_w8a16_tmem(a + m0 * lda, w.image, (const __half *)w.scales_dev, w.k, w.n, c + m0 * ldc, mp,
                               lda, ldc));
  }
  return 0;
}

}  // namespace b200

// ---- w8a16 for callers that cannot allocate ----------------------------------------------
// Some hosts hand this library a fixed set of device buffers and forbid any
// further allocation on their thread: a serving loop that has already carved
// up the whole device, a plugin running inside another runtime's memory
// budget, code between stream-capture begin and end.  For them the fp32
// partial-sum scratch of the decode GEMM lives in the library image itself.
namespace b200 {
namespace {

constexpr int kStaticMaxRows = 64;
constexpr int kStaticMaxCols = 16384;
// 4 MiB per GPU that loads the library, held until the process exits.
static __device__ __align__(256) float g_static_scratch[kStaticMaxRows * kStaticMaxCols];

struct StaticDevice {
  bool ready = false;
  float *scratch = nullptr;  // device address of g_static_scratch on this device
  int sm_count = 0;
};
constexpr int kMaxDevices = 64;
StaticDevice g_static_dev[kMaxDevices];
std::mutex g_static_mu;

// Once per device, with that device current.  In host code the array's name is
// only a handle; the address a kernel can use comes from cudaGetSymbolAddress.
int static_device_setup(int dev, StaticDevice **out) {
  std::lock_guard<std::mutex> lk(g_static_mu);
  StaticDevice &d = g_static_dev[dev];
  if (!d.ready) {
    float *p = nullptr;
    B200_CUDA(cudaGetSymbolAddress((void **)&p, g_static_scratch));
    int sms = 0;
    B200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    B200_CUDA(cudaFuncSetAttribute(w8a16_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)(1 * 16 * A_PITCH * sizeof(__half))));
    B200_CUDA(cudaFuncSetAttribute(w8a16_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)(2 * 16 * A_PITCH * sizeof(__half))));
    B200_CUDA(cudaFuncSetAttribute(w8a16_stream_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)(4 * 16 * A_PITCH * sizeof(__half))));
    d.scratch = p;
    d.sm_count = sms;
    d.ready = true;
  }
  *out = &d;
  return 0;
}

template <int MT>
void launch_stream_static(cudaStream_t s, int sm_count, const __half *a, int64_t lda, const uint4 *image,
                          float *ws, int m, int n, int k) {
  const int ksteps = (k + 15) / 16;
  const int n_strips = (n + 31) / 32;
  const int n_blocks = (n_strips + WARPS - 1) / WARPS;
  const size_t smem = (size_t)MT * 16 * A_PITCH * sizeof(__half);
  int64_t total = (int64_t)n_blocks * ksteps;
  int grid = sm_count * 2;
  if (grid > total) grid = (int)total;
  w8a16_stream_kernel<MT><<<grid, WARPS * 32, smem, s>>>(a, lda, image, ws, m, n, k, ksteps, n_blocks, n_strips);
}

}  // namespace
}  // namespace b200

extern "C" int b200mlir_w8a16_matmul_static_scratch(const void *a, int64_t lda, const void *image,
                                                    const void *scales, void *c, int64_t ldc, int64_t m,
                                                    int64_t n, int64_t k, void *cuda_stream) {
  using namespace b200;
  clear_error();
  if (!a || !image || !scales || !c)
    return set_error(B200MLIR_ERR_BAD_ARG, "w8a16 static-scratch: null pointer");
  if (m < 1 || n < 1 || k < 1)
    return set_error(B200MLIR_ERR_BAD_ARG, "w8a16 static-scratch: empty shape");
  if (m > kStaticMaxRows || n > kStaticMaxCols)
    return set_error(B200MLIR_ERR_UNSUPPORTED,
                     "w8a16 static-scratch: M=%lld, N=%lld exceed the built-in scratch (M <= %d, N <= %d); "
                     "use w8a16_matmul, which takes any shape (and may allocate)",
                     (long long)m, (long long)n, kStaticMaxRows, kStaticMaxCols);
  if (((uintptr_t)a & 15u) || ((uintptr_t)image & 15u) || lda % 8 || k % 8)
    return set_error(B200MLIR_ERR_BAD_ARG,
                     "w8a16 static-scratch: A and the image must be 16-byte aligned, K and lda multiples of 8");
  if (lda < k || ldc < n)
    return set_error(B200MLIR_ERR_BAD_ARG, "w8a16 static-scratch: row strides below the row lengths (lda %lld < K %lld or ldc %lld < N %lld)",
                     (long long)lda, (long long)k, (long long)ldc, (long long)n);
  if (((k + 15) / 16) * (((n + 31) / 32 + WARPS - 1) / WARPS) > 0x7fffffffLL)
    return set_error(B200MLIR_ERR_UNSUPPORTED, "w8a16 static-scratch: K x N exceeds the kernel's 32-bit work index");
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return set_error(B200MLIR_ERR_BAD_ARG, "device index %d out of range", dev);
  StaticDevice *d = nullptr;
  B200_TRY(static_device_setup(dev, &d));
  cudaStream_t s = (cudaStream_t)cuda_stream;
  float *ws = d->scratch;
  // the array keeps whatever the previous call left: the partial sums must start at zero
  B200_CUDA(cudaMemsetAsync(ws, 0, (size_t)m * (size_t)n * sizeof(float), s));
  const __half *ap = (const __half *)a;
  const uint4 *img = (const uint4 *)image;
  if (m <= 16) launch_stream_static<1>(s, d->sm_count, ap, lda, img, ws, (int)m, (int)n, (int)k);
  else if (m <= 32) launch_stream_static<2>(s, d->sm_count, ap, lda, img, ws, (int)m, (int)n, (int)k);
  else launch_stream_static<4>(s, d->sm_count, ap, lda, img, ws, (int)m, (int)n, (int)k);
  B200_TRY(check_launch("w8a16_stream(static scratch)"));
  int64_t total = m * n;
  int64_t blocks = (total + 255) / 256;
  int64_t cap = (int64_t)d->sm_count * 8;
  if (blocks > cap) blocks = cap;
  w8a16_finalize_kernel<<<(unsigned)blocks, 256, 0, s>>>(ws, (const __half *)scales, (__half *)c, (int)m, (int)n, ldc);
  return check_launch("w8a16_finalize(static scratch)");
}
