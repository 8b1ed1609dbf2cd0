// w8a16 GEMM on tcgen05 with the dequantisation done in registers on the way
// from HBM to shared memory: C[M,N] = A[M,K] · (q[K,N] · s[N]).
//
// The op is weight streaming (45 MB of int8 for the 4096 x 11008 config), so the
// kernel is arranged around the weight image, not around A:
//   * every CTA (one per SM, persistent) owns a contiguous range of output
//     channels for the WHOLE of K — no split-K, no partial sums in memory, no
//     atomics, no scratch, and the result is bit-reproducible;
//   * the weights are brought in by the converter threads themselves with
//     16-byte cp.async copies into a private shared-memory ring, seven K=128
//     steps ahead (≈66 KB in flight per SM).  Measured on B200: bulk/TMA copies
//     that miss L2 sustain only ~11 B/clk per SM (the copy engine's queue of
//     outstanding requests is short), about half of an SM's share of HBM
//     bandwidth; register prefetch does not work either, because a warp has only
//     a handful of scoreboard slots and a wait on an old load also waits for the
//     newer loads that share its slot; cp.async groups have neither limit;
//   * a converter thread owns one (channel, 16-k group) position for the whole
//     K loop: 16 bytes (stored as q+128) become 16 fp16 values with byte-permutes
//     and one subtract each, written in the 128-byte swizzled K-major layout the
//     MMA reads;
//   * operands are swapped: the weights are the MMA's "A" operand (channels on
//     the 128 rows), the activations its "B" operand (N_mma = M rows padded to
//     NM), so a decode step costs a 128 x 16 x 16 MMA per K=16 step.  A 128-row
//     MMA occupies the tensor pipe for ~48 clocks however narrow it is and
//     issuing one costs its thread about as much, so K steps alternate between
//     two issuing threads with one TMEM accumulator each;
//   * activations come through a small TMA ring (they are L2 hits); at the end
//     of K the first four converter warps read TMEM, add the two partial sums,
//     scale by s[n], round and store.
//
// Resident image, built once per weight (the analogue of the reference's
// pre-packed weight: backend/hmx_weight_prepack.py:124-212,
// lib/Dialect/Hmx/Transforms/WeightResidentPass.cpp:9-93):
//   [k-chunk = k/64][channel n][64 bytes = q[64*chunk + 0..63][n] + 128]
// i.e. the transposed weight in 64-deep chunks, so that any range of channels
// of one chunk is contiguous; positions with k >= K hold 128 (zero weight).
#include "common.h"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

using namespace ptx;

constexpr int CH_PASS = 80;          // channels per pass: 4 positions each on 320 converter threads
constexpr int CONV_W = 10;           // converter warps
constexpr int ISSUERS = 2;
constexpr int D_AHEAD = 8;           // depth of the int8 ring (K=128 steps)
constexpr int STG_BYTES = 2 * CH_PASS * 64;  // one ring slot: two [80][64 B] int8 sub-chunks, 10 KiB
constexpr int NB = 4;                // fp16 tile / activation buffers
constexpr int TILE_BYTES = 2 * CH_PASS * 128;  // two [80][64] fp16 sub-tiles (K = 128): 20 KiB
constexpr int THREADS = (CONV_W + 1 + ISSUERS) * 32;

__device__ __forceinline__ void sts128(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// two biased bytes -> two fp16 values: 0x64xx is 1024 + xx; minus 1152 gives xx - 128
__device__ __forceinline__ uint32_t dq2(uint32_t word, uint32_t selector) {
  uint32_t h, out;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(h) : "r"(word), "r"(0x64646464u), "r"(selector));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(out) : "r"(h), "r"(0x64806480u));
  return out;
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ void tmem_ld_32x32_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Region stamps for timeline debugging (the analogue of the reference's light-weight
// profiling regions, lib/Transforms/HexagonLWPInstrumentation.cpp): compiled in only
// with -DB200MLIR_W8_TRACE; CTA 3 records clock64() per role and step.
#ifdef B200MLIR_W8_TRACE
__device__ long long g_trace_buf[8 * 64];
#define TR(role, u) do { if (blockIdx.x == 3 && (u) < 64) trace_s[(role) * 64 + (u)] = clock64(); } while (0)
#else
#define TR(role, u) do { } while (0)
#endif

struct TcDecodeParams {
  const uint8_t *image;  // [k_chunks][n][64]
  const __half *scales;
  __half *c;
  int64_t ldc;
  int m, n, k_chunks;
  int *status;
};

// NM: activation rows padded to the MMA's N (16 or 64).
template <int NM>
__global__ void __launch_bounds__(THREADS, 1)
w8a16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const TcDecodeParams p) {
  constexpr int A_BYTES = 2 * NM * 128;  // two [NM][64] activation sub-tiles per K=128 step
  constexpr int TMEM_COLS = NM * ISSUERS < 32 ? 32 : NM * ISSUERS;
  constexpr uint32_t IDESC = make_idesc(/*D f32*/ 1, /*A f16*/ 0, /*B f16*/ 0, /*A K-major*/ 0,
                                        /*B K-major*/ 0, 128, NM);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // fp16 tiles first: a 128-row MMA reads 48 rows past an 80-row tile, into the next tile / the activation ring
  const uint32_t act0 = base + NB * TILE_BYTES;
  const uint32_t stg0 = act0 + NB * A_BYTES;               // int8 ring (also absorbs the last tile's over-read)
  const uint32_t ctrl = stg0 + D_AHEAD * STG_BYTES;
  const uint32_t bar_conv = ctrl;                          // NB: fp16 tile written (CONV_W arrivals)
  const uint32_t bar_act = ctrl + 8 * NB;                  // NB: activation sub-tiles landed (TMA)
  const uint32_t bar_free = ctrl + 16 * NB;                // NB: MMAs of the buffer done (commit)
  const uint32_t bar_afull = ctrl + 24 * NB;               // accumulators complete (ISSUERS commits)
  const uint32_t bar_aempty = bar_afull + 8;               // accumulators read out (CONV_W arrivals)
  const uint32_t tmem_slot = bar_aempty + 8;
  uint8_t *ctrl_gen = smem_raw + (ctrl - smem_u32(smem_raw));
  const int misc = 24 * NB + 16;
  volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(ctrl_gen + misc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ctrl_gen + misc + 4);

#ifdef B200MLIR_W8_TRACE
  __shared__ long long trace_s[8 * 64];
#endif
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) TR(7, 0);
  // this CTA's channels, walked in passes of at most CH_PASS
  const int c_begin = (int)((int64_t)p.n * blockIdx.x / gridDim.x);
  const int c_end = (int)((int64_t)p.n * (blockIdx.x + 1) / gridDim.x);
  const int passes = (c_end - c_begin + CH_PASS - 1) / CH_PASS;
  const int kch = p.k_chunks;
  const int steps = (kch + 1) >> 1;  // K=128 steps per pass

  if (threadIdx.x == 0) {
    for (int b = 0; b < NB; ++b) {
      mbar_init(bar_conv + 8 * b, CONV_W);
      mbar_init(bar_act + 8 * b, 1);
      mbar_init(bar_free + 8 * b, 1);
    }
    mbar_init(bar_afull, ISSUERS);
    mbar_init(bar_aempty, CONV_W);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
  }
  if (warp == CONV_W + 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, TMEM_COLS);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;
  if (threadIdx.x == 0) TR(7, 1);

  // Every CTA needs the same activation tile for a given k chunk; each CTA starts
  // at its own step so that they do not all ask one L2 slice for the same lines at
  // once (owning all of K, the order of the sum is free).
  const int rot = (int)((blockIdx.x * 19u) % (unsigned)steps);

  if (warp == CONV_W) {
    // ---------------- producer: the activation sub-tiles of each K=128 step ----------------
    if (lane == 0) {
      int t = 0;
      for (int pass = 0; pass < passes; ++pass) {
        int st = rot;
        for (int j = 0; j < steps; ++j, ++t) {
          const int b = t % NB;
          TR(6, t);
          if (!mbar_wait(bar_free + 8 * b, (uint32_t)(((t / NB) & 1) ^ 1), abort_flag, p.status, 21, t)) goto done;
          const uint32_t full = bar_act + 8 * b;
          const uint32_t dst = act0 + b * A_BYTES;
          mbar_expect_tx(full, A_BYTES);
          tma_load_2d(dst, &tmA, full, st * 128, 0);                  // k chunk 2*st (zero fill past K)
          tma_load_2d(dst + NM * 128, &tmA, full, st * 128 + 64, 0);  // k chunk 2*st + 1
          if (++st == steps) st = 0;
        }
      }
    }
  } else if (warp > CONV_W) {
    // ---------------- MMA issuer g: steps t = g, g+2, ... ----------------
    if (lane == 0) {
      const int g = warp - (CONV_W + 1);
      const uint32_t d_tmem = tmem_base + (uint32_t)(g * NM);
      int t = 0;
      for (int pass = 0; pass < passes; ++pass) {
        if (pass > 0 && !mbar_wait(bar_aempty, (uint32_t)((pass & 1) ^ 1), abort_flag, p.status, 22, pass)) goto done;
        uint32_t accumulate = 0;
        for (int j = 0; j < steps; ++j, ++t) {
          if ((t % ISSUERS) != g) continue;
          const int b = t % NB;
          const uint32_t ph = (uint32_t)((t / NB) & 1);
          TR(3, t);
          if (!mbar_wait(bar_conv + 8 * b, ph, abort_flag, p.status, 23, t)) goto done;
          if (!mbar_wait(bar_act + 8 * b, ph, abort_flag, p.status, 24, t)) goto done;
          tc_fence_after_sync();
          TR(4, t);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            const uint64_t adesc = smem_desc_sw128(base + b * TILE_BYTES + sub * (CH_PASS * 128), 16, 1024);
            const uint64_t bdesc = smem_desc_sw128(act0 + b * A_BYTES + sub * (NM * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              mma_f16_ss(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), IDESC, accumulate);
              accumulate = 1;
            }
          }
          mma_commit(bar_free + 8 * b);  // the fp16 tile and the activation buffer may be rewritten
          TR(5, t);
        }
        mma_commit(bar_afull);
      }
    }
  } else {
    // ---------------- converters (warps 0..9); read-out by warps 0..3 ----------------
    const int tid = threadIdx.x;       // position: channel = tid / 4, 16-k group = tid % 4
    const int row = tid >> 2, jj = tid & 3;
    const int q = warp & 3;            // TMEM lane quadrant this warp may read
    // where this position lands in a sub-tile: two 16-byte chunks of the channel's 128-byte row
    const uint32_t off0 = (uint32_t)(row * 128 + (((2 * jj) ^ (row & 7)) << 4));
    const uint32_t off1 = (uint32_t)(row * 128 + (((2 * jj + 1) ^ (row & 7)) << 4));
    const int64_t chunk_stride = (int64_t)p.n * 4;  // uint4 per k chunk
    int t = 0;
    for (int pass = 0; pass < passes; ++pass) {
      const int ch0 = c_begin + pass * CH_PASS;
      const int ch = min(CH_PASS, c_end - ch0);
      const bool mine = row < ch;
      const uint4 *src = reinterpret_cast<const uint4 *>(p.image) + ((int64_t)(ch0 + row) * 4 + jj);
      // zero weight is the byte 128: used for k chunks past the end of the image
      const uint4 zero = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
      const uint32_t my_stg = stg0 + (uint32_t)tid * 16;  // this thread's 16 bytes inside a sub-chunk
      // copies of step j (rotated) into ring slot j % D_AHEAD; always one commit per call
      auto issue = [&](int j) {
        if (j < steps && mine) {
          int st = j + rot;
          if (st >= steps) st -= steps;
          const int kc = 2 * st;
          const uint32_t dst = my_stg + (uint32_t)((j % D_AHEAD) * STG_BYTES);
          if (kc < kch) cp_async16(dst, src + (int64_t)kc * chunk_stride);
          if (kc + 1 < kch) cp_async16(dst + CH_PASS * 64, src + (int64_t)(kc + 1) * chunk_stride);
        }
        cp_async_commit();
      };
      for (int d = 0; d < D_AHEAD - 1; ++d) issue(d);
      for (int j = 0; j < steps; ++j, ++t) {
        const int b = t % NB;
        if (tid == 0) TR(0, t);
        cp_async_wait<D_AHEAD - 2>();  // this thread's copies of step j have landed
        if (tid == 0) TR(1, t);
        bool ok = mbar_wait(bar_free + 8 * b, (uint32_t)(((t / NB) & 1) ^ 1), abort_flag, p.status, 27, t);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) goto done;
        if (tid == 0) TR(2, t);
        if (mine) {
          int st = j + rot;
          if (st >= steps) st -= steps;
          const int kc = 2 * st;
          const uint32_t slot = my_stg + (uint32_t)((j % D_AHEAD) * STG_BYTES);
          const uint32_t tile = base + b * TILE_BYTES;
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            const uint4 v = (kc + sub < kch) ? lds128(slot + sub * (CH_PASS * 64)) : zero;
            const uint32_t tb = tile + sub * (CH_PASS * 128);
            sts128(tb + off0, dq2(v.x, 0x5140u), dq2(v.x, 0x5342u), dq2(v.y, 0x5140u), dq2(v.y, 0x5342u));
            sts128(tb + off1, dq2(v.z, 0x5140u), dq2(v.z, 0x5342u), dq2(v.w, 0x5140u), dq2(v.w, 0x5342u));
          }
        }
        issue(j + D_AHEAD - 1);  // refills the slot this thread read one step ago
        fence_async_smem();      // generic-proxy writes must be visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_conv + 8 * b);
      }
      if (tid == 0) TR(7, 2);
      cp_async_wait<0>();
      // end of K for this pass: read the accumulators out, add them, scale, round, store
      {
        bool ok = mbar_wait(bar_afull, (uint32_t)(pass & 1), abort_flag, p.status, 25, pass);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) goto done;
        tc_fence_after_sync();
        if (tid == 0) TR(7, 3);
        if (warp < 4) {
          const int chl = q * 32 + lane;  // channel = TMEM lane
          const bool live = chl < ch;
          const float sc = live ? __half2float(p.scales[ch0 + chl]) : 0.0f;
          const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
          const int used = min(ISSUERS, steps);  // accumulators that received an MMA
#pragma unroll 1
          for (int m0 = 0; m0 < NM; m0 += 16) {
            if (m0 >= p.m) break;  // uniform across the warp
            float acc[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[e] = 0.0f;
#pragma unroll 1
            for (int a = 0; a < used; ++a) {
              uint32_t rr[16];
              tmem_ld_32x32_x16(t_row + (uint32_t)(a * NM + m0), rr);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 16; ++e) acc[e] += __uint_as_float(rr[e]);
            }
            if (live) {
#pragma unroll
              for (int e = 0; e < 16; ++e)
                if (m0 + e < p.m) p.c[(int64_t)(m0 + e) * p.ldc + ch0 + chl] = __float2half_rn(acc[e] * sc);
            }
          }
        }
        if (tid == 0) TR(7, 4);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_aempty);
      }
    }
  }
done:
  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
#ifdef B200MLIR_W8_TRACE
  if (blockIdx.x == 3) for (int i = threadIdx.x; i < 8 * 64; i += blockDim.x) g_trace_buf[i] = trace_s[i];
#endif
  if (warp == CONV_W + 1) {
    if (*abort_flag)
      for (int i = 0; i < 64; ++i) __nanosleep(1000);  // bounded grace for copies / MMAs in flight
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// row-major int8 [K,N] -> [k/64][n][64 bytes]; one 16-byte piece (16 consecutive k of one channel) per thread
__global__ void __launch_bounds__(256)
w8a16_image_kernel(const int8_t *__restrict__ wq, uint4 *__restrict__ image, int K, int N, int k_chunks) {
  const int64_t total = (int64_t)k_chunks * N * 4;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    // consecutive threads take consecutive channels so that the reads of wq coalesce
    const int n = (int)(i % N);
    const int64_t r = i / N;
    const int j = (int)(r & 3);
    const int kc = (int)(r >> 2);
    uint32_t words[4];
#pragma unroll
    for (int wv = 0; wv < 4; ++wv) {
      uint32_t w = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int k = kc * 64 + j * 16 + wv * 4 + e;
        const int qv = k < K ? (int)wq[(int64_t)k * N + n] : 0;
        w |= (uint32_t)((qv + 128) & 0xff) << (8 * e);
      }
      words[wv] = w;
    }
    image[((int64_t)kc * N + n) * 4 + j] = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

int make_a_map(CUtensorMap *map, const void *a, int64_t m, int64_t k, int64_t lda, int box_rows) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return set_error(B200MLIR_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available");
    fn = (EncodeTiledFn)ptr;
  }
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
  cuuint64_t strides[1] = {(cuuint64_t)lda * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(a), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(B200MLIR_ERR_CUDA, "cuTensorMapEncodeTiled(A) failed: %d", (int)r);
  return 0;
}

template <int NM>
int launch_tc(const CUtensorMap &tmA, const TcDecodeParams &p) {
  Context &cx = ctx();
  constexpr int smem = NB * TILE_BYTES + NB * 2 * NM * 128 + D_AHEAD * STG_BYTES + 24 * NB + 64 + 1024;
  static_assert(smem <= 227 * 1024, "w8a16 tensor-core kernel exceeds shared memory");
  auto kern = w8a16_tc_kernel<NM>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set = true;
  }
  int grid = cx.sm_count;
  if (grid > p.n) grid = p.n;
  kern<<<grid, THREADS, smem, cx.stream>>>(tmA, p);
  return check_launch("w8a16_tc");
}

}  // namespace

#ifdef B200MLIR_W8_TRACE
extern "C" __attribute__((visibility("default"))) int b200mlir_debug_get_trace(long long *host) {
  return (int)cudaMemcpyFromSymbol(host, g_trace_buf, sizeof(long long) * 8 * 64);
}
#endif

int w8a16_build_block_image(const int8_t *wq_dev, int64_t k, int64_t n, void **image, size_t *bytes) {
  B200_TRY(ensure_ready());
  const int k_chunks = (int)((k + 63) / 64);
  const size_t sz = (size_t)k_chunks * n * 64;
  void *img = nullptr;
  B200_CUDA(cudaMalloc(&img, sz));
  int64_t total = (int64_t)(sz / 16);
  int64_t blocks = (total + 255) / 256;
  int64_t cap = (int64_t)ctx().sm_count * 32;
  if (blocks > cap) blocks = cap;
  w8a16_image_kernel<<<(unsigned)blocks, 256, 0, ctx().stream>>>(wq_dev, (uint4 *)img, (int)k, (int)n, k_chunks);
  int rc = check_launch("w8a16_image");
  if (rc) {
    cudaFree(img);
    return rc;
  }
  *image = img;
  *bytes = sz;
  return 0;
}

// Up to 64 rows per call (the caller loops over row passes).
int launch_w8a16_decode(const __half *a, const void *block_image, const __half *scales_dev, int64_t k,
                        int64_t n, __half *c, int64_t m, int64_t lda, int64_t ldc) {
  B200_TRY(ensure_ready());
  if (m < 1 || m > 64) return set_error(B200MLIR_ERR_BAD_ARG, "w8a16 tensor-core pass takes 1..64 rows");
  if (n > 0x7fffffff || k > 0x7fffffff) return set_error(B200MLIR_ERR_UNSUPPORTED, "w8a16: extent too large");
  TcDecodeParams p;
  p.k_chunks = (int)((k + 63) / 64);
  const int nm = m <= 16 ? 16 : 64;
  CUtensorMap tmA;
  B200_TRY(make_a_map(&tmA, a, m, k, lda, nm));
  p.image = (const uint8_t *)block_image;
  p.scales = scales_dev;
  p.c = c;
  p.ldc = ldc;
  p.m = (int)m;
  p.n = (int)n;
  p.status = ctx().d_status;
  return nm == 16 ? launch_tc<16>(tmA, p) : launch_tc<64>(tmA, p);
}

}  // namespace b200
