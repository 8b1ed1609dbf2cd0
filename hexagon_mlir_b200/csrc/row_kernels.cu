// Vector row kernels: softmax, RMSNorm, SiLU, SwiGLU, add.
//
// The reference lowers these to loops over one 128-byte HVX vector with a
// rotate-butterfly reduction
// (qcom_hexagon_backend/lib/Conversion/LinalgToLLVM/VectorRowReducePass.cpp:9-34,
//  include/hexagon/Dialect/Hvx/IR/HvxOps.td:28-64).  Here a row is held in
// registers by a group of threads: one pass over HBM, 128-bit loads and
// stores, shuffle-butterfly reductions, fp32 internals.  The fp16 kernels keep
// the reference's rounding points (f16 subtract, f16-rounded exponentials,
// f32 sum) so results differ from it only through exp/rsqrt approximations.
#include "common.h"

namespace b200 {
namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Reduce over the TPR threads that share a row.  TPR == 32: one warp, shuffles
// only.  TPR > 32: the whole block shares one row; partials cross warps
// through shared memory.
template <int TPR, bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float *scratch) {
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  if (TPR > 32) {
    constexpr int NW = TPR / 32;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();  // scratch may still be read from the previous reduction
    if (l == 0) scratch[w] = v;
    __syncthreads();
    float t = l < NW ? scratch[l] : (IS_MAX ? -INFINITY : 0.0f);
    v = IS_MAX ? warp_max(t) : warp_sum(t);
  }
  return v;
}

union H8 {
  uint4 u;
  __half2 h2[4];
  __half h[8];
};

// ---- softmax, fp16, row in registers ------------------------------------------------
// One row per group of TPR threads (a warp, or the whole block).  The grid may be smaller than
// the row count: a group then walks rows `first, first + stride, ...` and issues the loads of its
// NEXT row before it reduces the current one, so that a launch which is one wave deep still has
// reads arriving while earlier rows are being written (stores of row i, arithmetic of row i+1 and
// loads of row i+2 are in flight together).
template <int TPR, int VPL>
__global__ void __launch_bounds__(TPR > 32 ? TPR : 256)
softmax_f16_kernel(const __half *__restrict__ x, __half *__restrict__ y, int64_t rows, int cols,
                   int64_t ldx, int64_t ldy) {
  __shared__ float scratch[32];
  constexpr int ROWS_PER_BLOCK = TPR > 32 ? 1 : 256 / 32;
  const int lane = TPR > 32 ? threadIdx.x : (threadIdx.x & 31);
  int64_t row = (int64_t)blockIdx.x * ROWS_PER_BLOCK + (TPR > 32 ? 0 : (threadIdx.x >> 5));
  const int64_t stride = (int64_t)gridDim.x * ROWS_PER_BLOCK;
  pdl_trigger();
  if (TPR == 32 && row >= rows) return;  // (block-wide groups: every block owns at least one row)
  const int nvec = cols >> 3;
  pdl_wait();

  H8 v[VPL], nv[VPL];
  {
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + row * ldx);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      int idx = i * TPR + lane;
      if (idx < nvec) v[i].u = __ldg(xr + idx);
    }
  }
  for (; row < rows; row += stride) {
    const int64_t next = row + stride;
    if (next < rows) {
      const uint4 *xn = reinterpret_cast<const uint4 *>(x + next * ldx);
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        int idx = i * TPR + lane;
        if (idx < nvec) nv[i].u = __ldg(xn + idx);
      }
    }
    uint4 *yr = reinterpret_cast<uint4 *>(y + row * ldy);
    // 1. running max in f16 (softmax.md:167-177), two lanes per instruction
    __half2 m2 = __float2half2_rn(-INFINITY);
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (i * TPR + lane < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) m2 = __hmax2(m2, v[i].h2[j]);
      }
    float m = fmaxf(__low2float(m2), __high2float(m2));
    m = group_reduce<TPR, true>(m, scratch);
    m2 = __float2half2_rn(m);  // exact: m is an f16 value
    // 2. e = f16(exp(f32(x - m))) with the subtract in f16; 3. s = sum f32(e)
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (i * TPR + lane < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 z = __half22float2(__hsub2(v[i].h2[j], m2));
          const __half2 e = __floats2half2_rn(__expf(z.x), __expf(z.y));
          v[i].h2[j] = e;
          const float2 ef = __half22float2(e);
          s += ef.x + ef.y;
        }
      }
    s = group_reduce<TPR, false>(s, scratch);
    // 4. y = f16(f32(e) / s), as a multiply by the row's reciprocal
    //    (qcom_hexagon_backend/lib/Transforms/DivToMulOptimizationPass.cpp:9-18)
    const float inv = __frcp_rn(s);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      int idx = i * TPR + lane;
      if (idx < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 ef = __half22float2(v[i].h2[j]);
          v[i].h2[j] = __floats2half2_rn(ef.x * inv, ef.y * inv);
        }
        yr[idx] = v[i].u;
      }
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) v[i].u = nv[i].u;
  }
}

// Any shape / alignment: one block per row, three passes over the row (it sits
// in L1/L2 after the first).
template <typename T>
__device__ __forceinline__ float ld_f(const T *p);
template <>
__device__ __forceinline__ float ld_f<__half>(const __half *p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float ld_f<float>(const float *p) { return *p; }

__global__ void __launch_bounds__(256)
softmax_f16_generic(const __half *__restrict__ x, __half *__restrict__ y, int64_t rows,
                    int64_t cols, int64_t ldx, int64_t ldy) {
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  const __half *xr = x + row * ldx;
  __half *yr = y + row * ldy;
  float m = -INFINITY;
  for (int64_t j = threadIdx.x; j < cols; j += 256) m = fmaxf(m, __half2float(xr[j]));
  m = group_reduce<256, true>(m, scratch);
  const __half mh = __float2half_rn(m);
  float s = 0.0f;
  for (int64_t j = threadIdx.x; j < cols; j += 256) {
    __half e = __float2half_rn(__expf(__half2float(__hsub(xr[j], mh))));
    s += __half2float(e);
  }
  s = group_reduce<256, false>(s, scratch);
  for (int64_t j = threadIdx.x; j < cols; j += 256) {
    __half e = __float2half_rn(__expf(__half2float(__hsub(xr[j], mh))));
    yr[j] = __float2half_rn(__fdividef(__half2float(e), s));
  }
}

__global__ void __launch_bounds__(256)
softmax_f32_generic(const float *__restrict__ x, float *__restrict__ y, int64_t rows, int64_t cols,
                    int64_t ldx, int64_t ldy) {
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  const float *xr = x + row * ldx;
  float *yr = y + row * ldy;
  float m = -INFINITY;
  for (int64_t j = threadIdx.x; j < cols; j += 256) m = fmaxf(m, xr[j]);
  m = group_reduce<256, true>(m, scratch);
  float s = 0.0f;
  for (int64_t j = threadIdx.x; j < cols; j += 256) s += expf(xr[j] - m);
  s = group_reduce<256, false>(s, scratch);
  for (int64_t j = threadIdx.x; j < cols; j += 256) yr[j] = expf(xr[j] - m) / s;
}

// ---- RMSNorm -------------------------------------------------------------------------
// Same row walk as the softmax kernel (next row's loads issued before the current row's
// reduction); the gain vector is fetched once per thread, before the first reduction, instead of
// after it.
template <int TPR, int VPL>
__global__ void __launch_bounds__(TPR > 32 ? TPR : 256)
rmsnorm_f16_kernel(const __half *__restrict__ x, const __half *__restrict__ w,
                   __half *__restrict__ y, int64_t rows, int cols, int64_t ldx, int64_t ldy,
                   float eps) {
  __shared__ float scratch[32];
  constexpr int ROWS_PER_BLOCK = TPR > 32 ? 1 : 256 / 32;
  const int lane = TPR > 32 ? threadIdx.x : (threadIdx.x & 31);
  int64_t row = (int64_t)blockIdx.x * ROWS_PER_BLOCK + (TPR > 32 ? 0 : (threadIdx.x >> 5));
  const int64_t stride = (int64_t)gridDim.x * ROWS_PER_BLOCK;
  pdl_trigger();
  if (TPR == 32 && row >= rows) return;
  const int nvec = cols >> 3;
  const uint4 *wr = reinterpret_cast<const uint4 *>(w);
  pdl_wait();
  H8 v[VPL], nv[VPL], g[VPL];
  {
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + row * ldx);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      int idx = i * TPR + lane;
      if (idx < nvec) v[i].u = __ldg(xr + idx);
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      int idx = i * TPR + lane;
      if (idx < nvec) g[i].u = __ldg(wr + idx);
    }
  }
  const float inv_cols = 1.0f / (float)cols;
  for (; row < rows; row += stride) {
    const int64_t next = row + stride;
    if (next < rows) {
      const uint4 *xn = reinterpret_cast<const uint4 *>(x + next * ldx);
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        int idx = i * TPR + lane;
        if (idx < nvec) nv[i].u = __ldg(xn + idx);
      }
    }
    uint4 *yr = reinterpret_cast<uint4 *>(y + row * ldy);
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (i * TPR + lane < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __half22float2(v[i].h2[j]);
          ss = fmaf(f.x, f.x, ss);
          ss = fmaf(f.y, f.y, ss);
        }
      }
    ss = group_reduce<TPR, false>(ss, scratch);
    const float inv = rsqrtf(ss * inv_cols + eps);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      int idx = i * TPR + lane;
      if (idx < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __half22float2(v[i].h2[j]);
          float2 gg = __half22float2(g[i].h2[j]);
          v[i].h2[j] = __floats2half2_rn(f.x * inv * gg.x, f.y * inv * gg.y);
        }
        yr[idx] = v[i].u;
      }
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) v[i].u = nv[i].u;
  }
}

template <typename T>
__device__ __forceinline__ void st_f(T *p, float v);
template <>
__device__ __forceinline__ void st_f<__half>(__half *p, float v) { *p = __float2half_rn(v); }
template <>
__device__ __forceinline__ void st_f<float>(float *p, float v) { *p = v; }

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_generic(const T *__restrict__ x, const T *__restrict__ w, T *__restrict__ y, int64_t rows,
                int64_t cols, int64_t ldx, int64_t ldy, float eps) {
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  const T *xr = x + row * ldx;
  T *yr = y + row * ldy;
  float ss = 0.0f;
  for (int64_t j = threadIdx.x; j < cols; j += 256) {
    float f = ld_f(xr + j);
    ss = fmaf(f, f, ss);
  }
  ss = group_reduce<256, false>(ss, scratch);
  const float inv = rsqrtf(ss / (float)cols + eps);
  for (int64_t j = threadIdx.x; j < cols; j += 256)
    st_f(yr + j, ld_f(xr + j) * inv * ld_f(w + j));
}

// ---- elementwise -------------------------------------------------------------------------
// silu(x) = x / (1 + f16(exp(f32(-x)))), add and divide in f16 (test_silu.py:48)
__device__ __forceinline__ __half silu_h(__half x) {
  __half e = __float2half_rn(__expf(-__half2float(x)));
  __half d = __float2half_rn(1.0f + __half2float(e));
  return __float2half_rn(__fdividef(__half2float(x), __half2float(d)));
}

enum { EW_SILU = 0, EW_SWIGLU = 1, EW_ADD = 2 };

template <int OP>
__device__ __forceinline__ __half ew_apply(__half a, __half b) {
  if (OP == EW_SILU) return silu_h(a);
  if (OP == EW_SWIGLU) return __float2half_rn(__half2float(silu_h(a)) * __half2float(b));
  return __float2half_rn(__half2float(a) + __half2float(b));
}

// Each thread owns UNROLL 16-byte vectors, all loads issued before any math so
// that every SM keeps tens of KB in flight.
template <int OP, int UNROLL>
__global__ void __launch_bounds__(256)
ew_f16_kernel(const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ y,
              int64_t n) {
  const int64_t nvec = n >> 3;
  const int64_t base = ((int64_t)blockIdx.x * 256 * UNROLL) + threadIdx.x;
  const uint4 *av = reinterpret_cast<const uint4 *>(a);
  const uint4 *bv = reinterpret_cast<const uint4 *>(b);
  uint4 *yv = reinterpret_cast<uint4 *>(y);
  pdl_trigger();
  pdl_wait();
  H8 va[UNROLL], vb[UNROLL];
#pragma unroll
  for (int i = 0; i < UNROLL; ++i) {
    int64_t idx = base + (int64_t)i * 256;
    if (idx < nvec) {
      va[i].u = __ldg(av + idx);
      if (OP != EW_SILU) vb[i].u = __ldg(bv + idx);
    }
  }
#pragma unroll
  for (int i = 0; i < UNROLL; ++i) {
    int64_t idx = base + (int64_t)i * 256;
    if (idx < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) va[i].h[j] = ew_apply<OP>(va[i].h[j], vb[i].h[j]);
      yv[idx] = va[i].u;
    }
  }
  // ragged tail (n % 8 elements), one thread
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (int64_t j = nvec << 3; j < n; ++j)
      y[j] = ew_apply<OP>(a[j], OP != EW_SILU ? b[j] : a[j]);
}

template <int OP>
__global__ void __launch_bounds__(256)
ew_f16_scalar(const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ y,
              int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256)
    y[i] = ew_apply<OP>(a[i], OP != EW_SILU ? b[i] : a[i]);
}

__global__ void __launch_bounds__(256)
silu_f32_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    float v = x[i];
    y[i] = v / (1.0f + expf(-v));
  }
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

// Second half of the tensor-parallel block's reduction: this rank owns `rows` rows; their W
// fp16 partials sit in its receive buffer [W][rows][cols].  out = f16(sum_w f32(partial_w) +
// f32(residual)), written to the same rows of EVERY rank's output (peer stores over NVLink).
struct ReducePushParams {
  const __half *recv;
  const __half *residual;  // this rank's rows of the block input, or null
  int64_t ldres;
  __half *out[kMaxPushRanks];  // by rank: base of the [T][cols] output
  int world, rank;
  int64_t rows, cols;
};

template <int WORLD>
__global__ void __launch_bounds__(256)
reduce_rows_push_kernel(const ReducePushParams p) {
  // every thread owns UNR 16-byte pieces; all their loads are issued before any arithmetic
  constexpr int UNR = 4;
  constexpr int WMAX = WORLD > 0 ? WORLD : kMaxPushRanks;
  const int64_t vec_per_row = p.cols >> 3;
  const int64_t total = p.rows * vec_per_row;
  const int64_t slot = p.rows * p.cols;
  const int world = WORLD > 0 ? WORLD : p.world;
  for (int64_t base = ((int64_t)blockIdx.x * 256) * UNR + threadIdx.x; base < total;
       base += (int64_t)gridDim.x * 256 * UNR) {
    H8 part[UNR][WMAX], res[UNR];
    int64_t off[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int64_t i = base + (int64_t)u * 256;
      off[u] = 0;
      if (i < total) {
        const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) << 3;
        off[u] = r * p.cols + c;
#pragma unroll
        for (int w = 0; w < WMAX; ++w)
          if (w < world) part[u][w].u = *reinterpret_cast<const uint4 *>(p.recv + w * slot + off[u]);
        if (p.residual) res[u].u = __ldg(reinterpret_cast<const uint4 *>(p.residual + r * p.ldres + c));
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int64_t i = base + (int64_t)u * 256;
      if (i >= total) continue;
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
#pragma unroll
      for (int w = 0; w < WMAX; ++w)
        if (w < world) {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += __half2float(part[u][w].h[e]);
        }
      if (p.residual) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += __half2float(res[u].h[e]);
      }
      H8 o;
#pragma unroll
      for (int e = 0; e < 8; ++e) o.h[e] = __float2half_rn(acc[e]);
      const int64_t dst = p.rank * slot + off[u];
      // peers first: their stores cross NVLink and take longest to drain
#pragma unroll
      for (int w = 0; w < WMAX; ++w)
        if (w < world && w != p.rank) *reinterpret_cast<uint4 *>(p.out[w] + dst) = o.u;
      *reinterpret_cast<uint4 *>(p.out[p.rank] + dst) = o.u;
    }
  }
}

// All-reduce of one rank's slice through the NVSwitch's multicast addresses: `mc_in` and `mc_out`
// are multicast mappings of a buffer every rank of the group holds at the same offset.  One
// multimem.ld_reduce returns the SUM over all ranks' copies of 8 fp16 values (added in fp32 inside
// the switch, rounded once); one multimem.st writes the result into every rank's copy.  A rank
// reduces only its own slice, so per GPU 1/world of the buffer comes in and 1/world goes out —
// against (world-1)/world each way for exchanges through peer loads and stores.
__global__ void __launch_bounds__(256)
allreduce_multimem_kernel(const uint4 *__restrict__ mc_in, uint4 *__restrict__ mc_out, int64_t nvec) {
  constexpr int UNR = 4;
  const int64_t nthr = blockDim.x;
  for (int64_t base = ((int64_t)blockIdx.x * nthr) * UNR + threadIdx.x; base < nvec;
       base += (int64_t)gridDim.x * nthr * UNR) {
    uint32_t v[UNR][4];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int64_t i = base + (int64_t)u * nthr;
      if (i < nvec)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[u][0]), "=r"(v[u][1]), "=r"(v[u][2]), "=r"(v[u][3])
                     : "l"(mc_in + i)
                     : "memory");
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int64_t i = base + (int64_t)u * nthr;
      if (i < nvec)
        asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_out + i), "r"(v[u][0]),
                     "r"(v[u][1]), "r"(v[u][2]), "r"(v[u][3])
                     : "memory");
    }
  }
}

// The same all-reduce with the two rendezvous of the ranks inside the launch (no barrier kernels
// around it).  Every rank's copy of the buffer holds 16 flag words: [r] = the launch number at
// which rank r's partial was complete, [8 + r] = the launch number whose sums rank r has written
// everywhere.  A rank stores its flag into every peer's copy with plain release stores over NVLink
// (one thread per peer; a store through the multicast address costs a trip through the switch
// and back and measured three times the latency) and polls its own copy.  `state` is local:
// [0] launches finished, [1] CTAs finished.
//  entry: CTA 0 stores "arrived", every CTA waits until all ranks have arrived;
//  body:  this rank's slice, as above;
//  exit:  the last CTA to finish stores "written" and waits for every rank's "written", so the
//         launch ends only when this rank's copy holds every slice and nobody still reads it.
// Every wait is bounded; one that runs out records {site 48, late rank} and the launch returns.
struct PeerFlags {
  uint32_t *f[kMaxPushRanks];  // the flag words of every rank's copy, as this rank addresses them
};
__device__ __forceinline__ void flag_store_all(const PeerFlags &pf, int world, int slot, uint32_t v) {
  const int r = threadIdx.x;
  if (r < world) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf.f[r] + slot), "r"(v) : "memory");
}
__device__ __forceinline__ bool flags_reached(const uint32_t *flags, int world, uint32_t epoch, int *status, int site) {
  const int r = threadIdx.x;
  bool ok = true;
  if (r < world) {
    const long long t0 = clock64();
    for (;;) {
      uint32_t v;
      asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if (*(volatile int *)status != 0 || clock64() - t0 > 2000000000LL) {
        if (atomicCAS(status, 0, site) == 0) status[1] = r;
        ok = false;
        break;
      }
      __nanosleep(32);
    }
    __threadfence_system();  // what the other ranks wrote before their flags is visible from here on
  }
  return ok;
}

// A barrier of the ranks as a launch of its own: one warp; thread r tells rank r (a release store of
// this barrier's launch number into the flag word [slot * 8 + rank] of rank r's copy, over NVLink)
// and waits, bounded, for rank r's word in the local copy.  `state[2 + slot]` keeps the launch
// number on the device (graph replay).  Two slots, so that the barrier before and the one after an
// all-reduce never share a word.  A wait that runs out records {site 49, late rank}.
__global__ void __launch_bounds__(32)
rank_barrier_kernel(const PeerFlags pf, int world, int rank, int slot, uint32_t *state, int *status) {
  const uint32_t epoch = *(volatile uint32_t *)(state + 2 + slot) + 1;
  __syncwarp();
  const int r = threadIdx.x;
  if (r < world) {
    // what this rank wrote before the barrier was written by launches that have completed: the flag
    // needs no fence of its own in front of it
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(pf.f[r] + slot * 8 + rank), "r"(epoch) : "memory");
    const uint32_t *mine = pf.f[rank] + slot * 8 + r;
    const long long t0 = clock64();
    for (;;) {
      uint32_t v;
      asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if (*(volatile int *)status != 0 || clock64() - t0 > 2000000000LL) {
        if (atomicCAS(status, 0, 49) == 0) status[1] = r;
        break;
      }
    }
    __threadfence_system();  // what the other ranks wrote before their flags is visible to the launches that follow
  }
  __syncwarp();
  if (threadIdx.x == 0) state[2 + slot] = epoch;
}

__global__ void __launch_bounds__(256)
allreduce_multimem_sync_kernel(const uint4 *__restrict__ mc_in, uint4 *__restrict__ mc_out, int64_t nvec,
                               const PeerFlags pf, int world, int rank, uint32_t *state, int *status,
                               int exit_rendezvous) {
  const uint32_t *local_flags = pf.f[rank];
  const uint32_t epoch = *(volatile uint32_t *)state + 1;
  // the partial, written by the launch before this one, is complete: one CTA says so (CTA 0 is
  // among the first dispatched; CTAs that start later find the flags set)
  if (blockIdx.x == 0) flag_store_all(pf, world, rank, epoch);
  if (threadIdx.x < 32) flags_reached(local_flags, world, epoch, status, 48);
  __syncthreads();

  constexpr int UNR = 4;
  const int64_t nthr = blockDim.x;
  for (int64_t base = ((int64_t)blockIdx.x * nthr) * UNR + threadIdx.x; base < nvec;
       base += (int64_t)gridDim.x * nthr * UNR) {
    uint32_t v[UNR][4];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int64_t i = base + (int64_t)u * nthr;
      if (i < nvec)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[u][0]), "=r"(v[u][1]), "=r"(v[u][2]), "=r"(v[u][3])
                     : "l"(mc_in + i)
                     : "memory");
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int64_t i = base + (int64_t)u * nthr;
      if (i < nvec)
        asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_out + i), "r"(v[u][0]),
                     "r"(v[u][1]), "r"(v[u][2]), "r"(v[u][3])
                     : "memory");
    }
  }

  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    // this CTA's sums are on their way to every copy before it counts as finished (with the exit
    // rendezvous left to the caller's barrier, the end of the launch does that)
    if (exit_rendezvous) __threadfence_system();
    else __threadfence();
    s_last = atomicAdd(&state[1], 1u) == gridDim.x - 1;
    if (s_last) {
      if (exit_rendezvous) __threadfence_system();
      state[1] = 0;
    }
  }
  __syncthreads();
  if (s_last) {
    if (exit_rendezvous) {
      flag_store_all(pf, world, 8 + rank, epoch);  // release stores: after every CTA's sums (fence + counter above)
      if (threadIdx.x < 32) flags_reached(local_flags + 8, world, epoch, status, 48);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      state[0] = epoch;
      __threadfence();
    }
  }
}

template <int OP>
int launch_ew(const __half *a, const __half *b, __half *y, int64_t n, const char *what) {
  B200_TRY(ensure_ready());
  if (n <= 0) return 0;
  cudaStream_t s = ctx().stream;
  if (aligned16(a) && aligned16(y) && (OP == EW_SILU || aligned16(b))) {
    constexpr int UNROLL = 4;
    int64_t nvec = n >> 3;
    int64_t blocks = (nvec + 256 * UNROLL - 1) / (256 * UNROLL);
    if (blocks < 1) blocks = 1;
    launch_pdl(ew_f16_kernel<OP, UNROLL>, dim3((unsigned)blocks), dim3(256), 0, s, a, b, y, n);
  } else {
    int64_t blocks = (n + 255) / 256;
    int64_t cap = (int64_t)ctx().sm_count * 16;
    if (blocks > cap) blocks = cap;
    ew_f16_scalar<OP><<<(unsigned)blocks, 256, 0, s>>>(a, b, y, n);
  }
  return check_launch(what);
}

}  // namespace

// Grid of a row kernel.  `rows` row groups are wanted (one per row, rows_per_block per block).
// Option rowKernelWalk: 0 = one group per row (every load of the launch in flight at once);
// k > 0 = at most k resident blocks per SM and the groups walk the rows (loads of the next row
// under the arithmetic and the stores of the current one); -1 = the measured choice per kernel
// (`auto_walk`): softmax is fastest with one group per row at every shape tried (4096x1024 5.05 us
// against 5.4-7.8 walking; bytes in flight matter more than the overlap), RMSNorm gains from a
// walk (2048x4096: 7.6 us at 6 blocks per SM against 8.5; 4096x1024: 5.3 at 2 against 5.9).
static unsigned row_grid(int64_t rows, int rows_per_block, int block_threads, int auto_walk) {
  const int64_t want = (rows + rows_per_block - 1) / rows_per_block;
  int walk = (int)ctx().opt.row_kernel_walk;
  if (walk < 0) walk = auto_walk;
  if (walk == 0) return (unsigned)want;
  const int resident = 2048 / block_threads;  // blocks of this size an SM holds
  const int per_sm = walk > resident ? resident : walk;
  const int64_t cap = (int64_t)ctx().sm_count * per_sm;
  if ((int)ctx().opt.row_kernel_walk < 0 && want > cap * 8) return (unsigned)want;  // deep launches: the plain form is at the roofline
  return (unsigned)(want < cap ? want : cap);
}

#define ROW_DISPATCH(KERNEL, WALK_WARP, WALK_BLOCK, ...)                                                        \
  do {                                                                                   \
    if (cols <= 256) {                                                                   \
      launch_pdl(KERNEL<32, 1>, dim3(row_grid(rows, 8, 256, WALK_WARP)), dim3(256), 0, s, __VA_ARGS__);             \
    } else if (cols <= 512) {                                                            \
      launch_pdl(KERNEL<32, 2>, dim3(row_grid(rows, 8, 256, WALK_WARP)), dim3(256), 0, s, __VA_ARGS__);             \
    } else if (cols <= 1024) {                                                           \
      launch_pdl(KERNEL<32, 4>, dim3(row_grid(rows, 8, 256, WALK_WARP)), dim3(256), 0, s, __VA_ARGS__);             \
    } else if (cols <= 2048) {                                                           \
      launch_pdl(KERNEL<32, 8>, dim3(row_grid(rows, 8, 256, WALK_WARP)), dim3(256), 0, s, __VA_ARGS__);             \
    } else if (cols <= 4096) {                                                           \
      launch_pdl(KERNEL<128, 4>, dim3(row_grid(rows, 1, 128, WALK_BLOCK)), dim3(128), 0, s, __VA_ARGS__);            \
    } else if (cols <= 8192) {                                                           \
      launch_pdl(KERNEL<256, 4>, dim3(row_grid(rows, 1, 256, WALK_BLOCK)), dim3(256), 0, s, __VA_ARGS__);            \
    } else if (cols <= 16384) {                                                          \
      launch_pdl(KERNEL<512, 4>, dim3(row_grid(rows, 1, 512, WALK_BLOCK)), dim3(512), 0, s, __VA_ARGS__);            \
    } else {                                                                             \
      launch_pdl(KERNEL<1024, 4>, dim3(row_grid(rows, 1, 1024, WALK_BLOCK)), dim3(1024), 0, s, __VA_ARGS__);         \
    }                                                                                    \
  } while (0)

int launch_reduce_rows_push(const __half *recv, const __half *residual, int64_t ldres, void *const *peer_out,
                            int world, int rank, int64_t rows_per_rank, int64_t cols) {
  B200_TRY(ensure_ready());
  if (world < 1 || world > kMaxPushRanks || rank < 0 || rank >= world || rows_per_rank < 1 || cols < 8 || cols % 8 ||
      !recv || !aligned16(recv) || (residual && (!aligned16(residual) || ldres % 8)))
    return set_error(B200MLIR_ERR_BAD_ARG,
                     "reduce_rows_push: bad argument (world <= 8, cols a multiple of 8, 16-byte aligned)");
  ReducePushParams p;
  p.recv = recv;
  p.residual = residual;
  p.ldres = ldres;
  for (int w = 0; w < kMaxPushRanks; ++w) {
    p.out[w] = w < world ? (__half *)peer_out[w] : nullptr;
    if (w < world && (!p.out[w] || !aligned16(p.out[w])))
      return set_error(B200MLIR_ERR_BAD_ARG, "reduce_rows_push: output pointer %d missing or unaligned", w);
  }
  p.world = world;
  p.rank = rank;
  p.rows = rows_per_rank;
  p.cols = cols;
  const int64_t total = rows_per_rank * (cols >> 3);
  int64_t blocks = (total + 256 * 4 - 1) / (256 * 4);
  const int64_t cap = (int64_t)ctx().sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const unsigned g = (unsigned)blocks;
  switch (world) {
    case 2: reduce_rows_push_kernel<2><<<g, 256, 0, ctx().stream>>>(p); break;
    case 4: reduce_rows_push_kernel<4><<<g, 256, 0, ctx().stream>>>(p); break;
    case 8: reduce_rows_push_kernel<8><<<g, 256, 0, ctx().stream>>>(p); break;
    default: reduce_rows_push_kernel<0><<<g, 256, 0, ctx().stream>>>(p); break;
  }
  return check_launch("reduce_rows_push");
}

int launch_allreduce_multimem(const void *mc_in, void *mc_out, int64_t elem_offset, int64_t count) {
  B200_TRY(ensure_ready());
  if (!mc_in || !mc_out || elem_offset < 0 || count < 0 || elem_offset % 8 || count % 8 || !aligned16(mc_in) ||
      !aligned16(mc_out))
    return set_error(B200MLIR_ERR_BAD_ARG,
                     "allreduce_multimem: multicast addresses 16-byte aligned, offset and count multiples of 8 elements");
  if (count == 0) return 0;
  const int64_t nvec = count >> 3;
  // one CTA of 128 threads per SM: the exchange is bound by the links, a few tens of KB in flight
  // per SM saturate them, and wider or deeper grids measured slower (two ranks, 16.8 MB: 43.7 us
  // against 52.5 with four CTAs of 256 threads per SM)
  const int threads = 128;
  int64_t blocks = (nvec + threads * 4 - 1) / (threads * 4);
  const int64_t cap = (int64_t)ctx().sm_count;
  if (blocks > cap) blocks = cap;
  allreduce_multimem_kernel<<<(unsigned)blocks, threads, 0, ctx().stream>>>(
      reinterpret_cast<const uint4 *>((const __half *)mc_in + elem_offset),
      reinterpret_cast<uint4 *>((__half *)mc_out + elem_offset), nvec);
  return check_launch("allreduce_multimem");
}

int launch_rank_barrier(void *const *peer_bufs, int64_t flags_elem_offset, int slot, int rank, int world, void *state) {
  B200_TRY(ensure_ready());
  if (!peer_bufs || !state || world < 2 || world > kMaxPushRanks || rank < 0 || rank >= world || slot < 0 || slot > 1 ||
      flags_elem_offset < 0 || flags_elem_offset % 8)
    return set_error(B200MLIR_ERR_BAD_ARG, "tp_barrier: the buffer's address on every rank, slot 0 or 1, 2 <= world <= %d, "
                     "a device state of four words", kMaxPushRanks);
  PeerFlags pf;
  for (int r = 0; r < kMaxPushRanks; ++r) {
    if (r < world && !peer_bufs[r]) return set_error(B200MLIR_ERR_BAD_ARG, "tp_barrier: buffer address of rank %d missing", r);
    pf.f[r] = r < world ? reinterpret_cast<uint32_t *>((__half *)peer_bufs[r] + flags_elem_offset) : nullptr;
  }
  rank_barrier_kernel<<<1, 32, 0, ctx().stream>>>(pf, world, rank, slot, (uint32_t *)state, ctx().d_status);
  return check_launch("tp_barrier");
}

int launch_allreduce_multimem_sync(void *mc_buf, void *const *peer_bufs, int64_t elem_offset, int64_t count,
                                   int64_t flags_elem_offset, int rank, int world, void *state, cudaStream_t stream,
                                   int exit_rendezvous) {
  B200_TRY(ensure_ready());
  if (!peer_bufs || world < 2 || world > kMaxPushRanks || rank < 0 || rank >= world)
    return set_error(B200MLIR_ERR_BAD_ARG, "allreduce_multimem_sync: the buffer's address on every rank, 2 <= world <= %d",
                     kMaxPushRanks);
  void *local_buf = peer_bufs[rank];
  PeerFlags pf;
  for (int r = 0; r < kMaxPushRanks; ++r) {
    if (r < world && (!peer_bufs[r] || !aligned16(peer_bufs[r])))
      return set_error(B200MLIR_ERR_BAD_ARG, "allreduce_multimem_sync: buffer address of rank %d missing or unaligned", r);
    pf.f[r] = r < world ? reinterpret_cast<uint32_t *>((__half *)peer_bufs[r] + flags_elem_offset) : nullptr;
  }
  if (!mc_buf || !local_buf || !state || elem_offset < 0 || count < 0 || elem_offset % 8 || count % 8 ||
      flags_elem_offset < 0 || flags_elem_offset % 8 || !aligned16(mc_buf) || !aligned16(local_buf) || world < 2 ||
      world > kMaxPushRanks || rank < 0 || rank >= world)
    return set_error(B200MLIR_ERR_BAD_ARG,
                     "allreduce_multimem_sync: 16-byte aligned multicast and local addresses of one buffer, offsets and "
                     "count multiples of 8 elements, 2 <= world <= %d, a device state of two words", kMaxPushRanks);
  const int64_t nvec = count >> 3;
  // one CTA of 128 threads per SM: two ranks, 16.8 MB, measured 63 us against 65-76 for wider or
  // deeper grids (the exchange is bound by the links, and every extra CTA adds a system-scope
  // fence and a flag round to the end of the launch); it also leaves the SMs to a GEMM beside it
  const int threads = 128;
  int64_t blocks = (nvec + threads * 4 - 1) / (threads * 4);
  const int64_t cap = (int64_t)ctx().sm_count;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  allreduce_multimem_sync_kernel<<<(unsigned)blocks, threads, 0, stream ? stream : ctx().stream>>>(
      reinterpret_cast<const uint4 *>((const __half *)mc_buf + elem_offset),
      reinterpret_cast<uint4 *>((__half *)mc_buf + elem_offset), nvec, pf, world, rank, (uint32_t *)state, ctx().d_status,
      exit_rendezvous);
  return check_launch("allreduce_multimem_sync");
}

static bool row_fast_path(const void *x, const void *y, int64_t cols, int64_t ldx, int64_t ldy) {
  return cols % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0 && aligned16(x) && aligned16(y) &&
         cols <= 32768;
}

int launch_softmax_f16(const __half *x, __half *y, int64_t rows, int64_t cols, int64_t ldx,
                       int64_t ldy) {
  B200_TRY(ensure_ready());
  if (rows <= 0 || cols <= 0) return 0;
  if (rows > 0x7fffffff) return set_error(B200MLIR_ERR_BAD_ARG, "softmax: too many rows");
  cudaStream_t s = ctx().stream;
  if (row_fast_path(x, y, cols, ldx, ldy)) {
    ROW_DISPATCH(softmax_f16_kernel, 0, 0, x, y, rows, (int)cols, ldx, ldy);
  } else {
    softmax_f16_generic<<<(unsigned)rows, 256, 0, s>>>(x, y, rows, cols, ldx, ldy);
  }
  return check_launch("softmax_f16");
}

int launch_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols, int64_t ldx,
                       int64_t ldy) {
  B200_TRY(ensure_ready());
  if (rows <= 0 || cols <= 0) return 0;
  if (rows > 0x7fffffff) return set_error(B200MLIR_ERR_BAD_ARG, "softmax: too many rows");
  softmax_f32_generic<<<(unsigned)rows, 256, 0, ctx().stream>>>(x, y, rows, cols, ldx, ldy);
  return check_launch("softmax_f32");
}

int launch_rmsnorm_f16(const __half *x, const __half *w, __half *y, int64_t rows, int64_t cols,
                       int64_t ldx, int64_t ldy, float eps) {
  B200_TRY(ensure_ready());
  if (rows <= 0 || cols <= 0) return 0;
  if (rows > 0x7fffffff) return set_error(B200MLIR_ERR_BAD_ARG, "rms_norm: too many rows");
  cudaStream_t s = ctx().stream;
  if (row_fast_path(x, y, cols, ldx, ldy) && aligned16(w)) {
    ROW_DISPATCH(rmsnorm_f16_kernel, 2, 6, x, w, y, rows, (int)cols, ldx, ldy, eps);
  } else {
    rmsnorm_generic<__half><<<(unsigned)rows, 256, 0, s>>>(x, w, y, rows, cols, ldx, ldy, eps);
  }
  return check_launch("rmsnorm_f16");
}

int launch_rmsnorm_f32(const float *x, const float *w, float *y, int64_t rows, int64_t cols,
                       int64_t ldx, int64_t ldy, float eps) {
  B200_TRY(ensure_ready());
  if (rows <= 0 || cols <= 0) return 0;
  if (rows > 0x7fffffff) return set_error(B200MLIR_ERR_BAD_ARG, "rms_norm: too many rows");
  rmsnorm_generic<float><<<(unsigned)rows, 256, 0, ctx().stream>>>(x, w, y, rows, cols, ldx, ldy,
                                                                   eps);
  return check_launch("rmsnorm_f32");
}

int launch_silu_f16(const __half *x, __half *y, int64_t n) {
  return launch_ew<EW_SILU>(x, x, y, n, "silu_f16");
}
int launch_swiglu_f16(const __half *g, const __half *u, __half *y, int64_t n) {
  return launch_ew<EW_SWIGLU>(g, u, y, n, "swiglu_f16");
}
int launch_add_f16(const __half *a, const __half *b, __half *y, int64_t n) {
  return launch_ew<EW_ADD>(a, b, y, n, "add_f16");
}
int launch_silu_f32(const float *x, float *y, int64_t n) {
  B200_TRY(ensure_ready());
  if (n <= 0) return 0;
  int64_t blocks = (n + 255) / 256;
  int64_t cap = (int64_t)ctx().sm_count * 16;
  if (blocks > cap) blocks = cap;
  silu_f32_kernel<<<(unsigned)blocks, 256, 0, ctx().stream>>>(x, y, n);
  return check_launch("silu_f32");
}

}  // namespace b200
