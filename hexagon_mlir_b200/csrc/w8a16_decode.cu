// w8a16 GEMM on tcgen05 with the dequantisation done on the way through shared
// memory: C[M,N] = A[M,K] · (q[K,N] · s[N]).
//
// The op is weight streaming (45 MB of int8 for the 4096 x 11008 config), so the
// kernel is arranged around the weight image, not around A:
//   * every CTA (one per SM, persistent) owns a contiguous range of output
//     channels for the WHOLE of K — no split-K, no partial sums, no atomics, no
//     scratch, and the result is bit-reproducible;
//   * operands are swapped: the weights are the MMA's "A" operand (up to 128
//     channels per instruction, K-major), the activations its "B" operand
//     (N_mma = M rows padded to NM), so an M=1..16 decode step costs a
//     128 x 16 x 16 MMA (8 clocks) per K=16 step;
//   * one producer thread keeps a deep ring of stages full: one bulk copy of the
//     CTA's channels x 64 k of int8 plus one TMA tile of activations per stage;
//   * eight converter warps turn each stage's bytes (stored as q+128) into fp16
//     with a byte-permute and one subtract and write them in the 128-byte
//     swizzled K-major layout the MMA reads (three 16 KiB buffers);
//   * one thread issues the MMAs into a TMEM accumulator [channel][row]; at the
//     end of K the converter warps read it out, scale by s[n], round and store.
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

constexpr int CH_MAX = 128;                 // channels per pass = MMA M

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
  return v;
}
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
__device__ __forceinline__ void tmem_ld_32x32_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

struct TcDecodeParams {
  const uint8_t *image;  // [k_chunks][n][64]
  const __half *scales;
  __half *c;
  int64_t ldc;
  int m, n, k_chunks;
  int *status;
};

#ifdef W8_TRACE
__device__ long long g_trace_buf[8 * 64];
#define TR(role, u) do { if (blockIdx.x == 3 && (u) < 64) trace_s[(role) * 64 + (u)] = clock64(); } while (0)
#else
#define TR(role, u) do { } while (0)
#endif

struct TcLayout {
  int n_slots;     // ring depth (<= MAX_SLOTS)
  int slot_bytes;  // activation tile + this launch's widest int8 slab, multiple of 1024
  int tile_bytes;  // fp16 weight tile: channels rounded up to 8 rows of 128 bytes, multiple of 1024
};
constexpr int MAX_SLOTS = 32;

// NM: activation rows padded to the MMA's N (16..256, multiple of 16).
// G: independent convert->MMA pipelines.  The costs that shape this (measured on
// B200): a 128-row MMA occupies the tensor pipe for at least ~48 clocks however
// narrow it is, issuing one costs its thread about as much, a commit-to-wake
// round trip is ~200 clocks and a converter group needs a few hundred clocks per
// K=64 step — while HBM delivers a step's bytes every ~200 clocks.  So K steps
// are dealt round-robin to G pipelines, each with two converter warps, two fp16
// tiles, one issuing thread and one TMEM accumulator; one producer thread feeds
// all of them through a deep ring of int8 slots (that ring, not the fp16 tiles,
// is what keeps ~100 KB per SM in flight).  The read-out adds the G partial sums.
template <int NM, int G>
__global__ void __launch_bounds__((2 * G + 1 + G) * 32, 1)
w8a16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const TcDecodeParams p, const TcLayout lay) {
  constexpr int A_BYTES = NM * 128;
  constexpr int NB = 2 * G;           // fp16 tiles
  constexpr int CONV_W = 2 * G;       // converter warps
  constexpr int TMEM_COLS = NM * G < 32 ? 32 : NM * G;
  static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns");
  constexpr uint32_t IDESC = make_idesc(/*D f32*/ 1, /*A f16*/ 0, /*B f16*/ 0, /*A K-major*/ 0,
                                        /*B K-major*/ 0, 128, NM);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // fp16 tiles first: a 128-row MMA reads past a shorter tile into the next tile / the ring
  const uint32_t ring = base + NB * lay.tile_bytes;
  const uint32_t ctrl = ring + lay.n_slots * lay.slot_bytes;
  const uint32_t bar_full = ctrl;                          // MAX_SLOTS
  const uint32_t bar_empty = ctrl + 8 * MAX_SLOTS;         // MAX_SLOTS
  const uint32_t bar_conv = ctrl + 16 * MAX_SLOTS;         // NB
  const uint32_t bar_cempty = bar_conv + 8 * NB;           // NB
  const uint32_t bar_afull = bar_cempty + 8 * NB;          // 1
  const uint32_t bar_aempty = bar_afull + 8;               // 1
  const uint32_t tmem_slot = bar_aempty + 8;
  uint8_t *ctrl_gen = smem_raw + (ctrl - smem_u32(smem_raw));
  const int misc = 16 * MAX_SLOTS + 16 * NB + 16;
  volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(ctrl_gen + misc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ctrl_gen + misc + 4);

#ifdef W8_TRACE
  __shared__ long long trace_s[8 * 64];
#endif
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // this CTA's channels, walked in passes of at most CH_MAX
  const int c_begin = (int)((int64_t)p.n * blockIdx.x / gridDim.x);
  const int c_end = (int)((int64_t)p.n * (blockIdx.x + 1) / gridDim.x);
  const int passes = (c_end - c_begin + CH_MAX - 1) / CH_MAX;
  const int kch = p.k_chunks;
  const int ns = lay.n_slots;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ns; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < NB; ++b) {
      mbar_init(bar_conv + 8 * b, 2);  // the two converter warps of the pipeline
      mbar_init(bar_cempty + 8 * b, 1);
    }
    mbar_init(bar_afull, G);
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

  if (warp == CONV_W) {
    // ---------------- producer: one bulk copy + one activation tile per K=64 step ----------------
    if (lane == 0) {
      // Every CTA needs the same activation tile for a given k chunk; each CTA
      // starts at its own chunk so that they do not all ask one L2 slice for the
      // same lines at once (owning all of K, the order of the sum is free).
      const int rot = (int)((blockIdx.x * 37u) % (unsigned)kch);
      int slot = 0;
      uint32_t phase = 0;
      for (int pass = 0; pass < passes; ++pass) {
        const int ch0 = c_begin + pass * CH_MAX;
        const int ch = min(CH_MAX, c_end - ch0);
        const uint8_t *src = p.image + (int64_t)ch0 * 64;
        int kc = rot;
        for (int j = 0; j < kch; ++j) {
          TR(0, j);
          if (!mbar_wait(bar_empty + 8 * slot, phase ^ 1u, abort_flag, p.status, 21, j)) goto done;
          TR(1, j);
          const uint32_t full = bar_full + 8 * slot;
          const uint32_t dst = ring + slot * lay.slot_bytes;
          mbar_expect_tx(full, (uint32_t)(ch * 64 + A_BYTES));
          tma_load_2d(dst, &tmA, full, kc * 64, 0);
          bulk_load(dst + A_BYTES, src + (int64_t)kc * p.n * 64, (uint32_t)(ch * 64), full);
          if (++kc == kch) kc = 0;
          if (++slot == ns) {
            slot = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp > CONV_W) {
    // ---------------- MMA issuer of pipeline g: steps u = g, g+G, ... ----------------
    if (lane == 0) {
      const int g = warp - (CONV_W + 1);
      const uint32_t d_tmem = tmem_base + (uint32_t)(g * NM);
      const int units = passes * kch;
      int slot = g % ns;
      uint32_t sphase = (uint32_t)((g / ns) & 1);
      int t = 0;  // this pipeline's step count
      int u = g;
      for (int pass = 0; pass < passes; ++pass) {
        const int u_end = (pass + 1) * kch;
        if (pass > 0 && !mbar_wait(bar_aempty, (pass & 1) ^ 1u, abort_flag, p.status, 22, pass)) goto done;
        uint32_t accumulate = 0;
        for (; u < u_end && u < units; u += G, ++t) {
          const int b = g + G * (t & 1);
          TR(5, u);
          if (!mbar_wait(bar_conv + 8 * b, (uint32_t)((t >> 1) & 1), abort_flag, p.status, 23, u)) goto done;
          tc_fence_after_sync();
          TR(6, u);
          const uint64_t adesc = smem_desc_sw128(base + b * lay.tile_bytes, 16, 1024);   // fp16 weights [<=128][64]
          const uint64_t bdesc = smem_desc_sw128(ring + slot * lay.slot_bytes, 16, 1024);  // activations [NM][64]
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            mma_f16_ss(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), IDESC, accumulate);
            accumulate = 1;
          }
          mma_commit(bar_empty + 8 * slot);   // the slot (activation tile) may be refilled
          mma_commit(bar_cempty + 8 * b);     // the fp16 tile may be rewritten
          TR(7, u);
          slot += G;
          while (slot >= ns) {
            slot -= ns;
            sphase ^= 1u;
          }
        }
        mma_commit(bar_afull);
      }
      (void)sphase;
    }
  } else {
    // ---------------- converters: pipeline g = warps 2g, 2g+1; read-out by warps 0..3 ----------------
    const int g = warp >> 1;
    const int tid = (warp & 1) * 32 + lane;  // 0..63 inside the pipeline
    const int q = warp & 3;                  // TMEM lane quadrant this warp may read
    const int units = passes * kch;
    int slot = g % ns;
    uint32_t sphase = (uint32_t)((g / ns) & 1);
    int t = 0;
    int u = g;
    for (int pass = 0; pass < passes; ++pass) {
      const int ch0 = c_begin + pass * CH_MAX;
      const int ch = min(CH_MAX, c_end - ch0);
      const int u_end = (pass + 1) * kch;
      for (; u < u_end && u < units; u += G, ++t) {
        const int b = g + G * (t & 1);
        if (tid == 0) TR(2, u);
        bool ok = mbar_wait(bar_full + 8 * slot, sphase, abort_flag, p.status, 26, u) &&
                  mbar_wait(bar_cempty + 8 * b, (uint32_t)(((t >> 1) & 1) ^ 1), abort_flag, p.status, 27, u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) goto done;
        if (tid == 0) TR(3, u);
        const uint32_t src = ring + slot * lay.slot_bytes + A_BYTES;
        const uint32_t dst = base + b * lay.tile_bytes;
        // task = (channel, 16-k group): 16 bytes in, two 16-byte chunks of the channel's row out
        for (int task = tid; task < ch * 4; task += 64) {
          const int row = task >> 2, jj = task & 3;
          const uint4 w = lds128(src + (uint32_t)task * 16);
          const uint32_t rbase = dst + (uint32_t)row * 128;
          const uint32_t c0 = (uint32_t)(((2 * jj) ^ (row & 7)) << 4), c1 = (uint32_t)(((2 * jj + 1) ^ (row & 7)) << 4);
          sts128(rbase + c0, dq2(w.x, 0x5140u), dq2(w.x, 0x5342u), dq2(w.y, 0x5140u), dq2(w.y, 0x5342u));
          sts128(rbase + c1, dq2(w.z, 0x5140u), dq2(w.z, 0x5342u), dq2(w.w, 0x5140u), dq2(w.w, 0x5342u));
        }
        fence_async_smem();  // generic-proxy writes must be visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_conv + 8 * b);
        if (tid == 0) TR(4, u);
        slot += G;
        while (slot >= ns) {
          slot -= ns;
          sphase ^= 1u;
        }
      }
      // end of K for this pass: read the accumulators out, add them, scale, round, store
      {
        bool ok = mbar_wait(bar_afull, pass & 1, abort_flag, p.status, 25, pass);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) goto done;
        tc_fence_after_sync();
        if (warp < 4) {
          const int chl = q * 32 + lane;  // channel = TMEM lane
          const bool live = chl < ch;
          const float sc = live ? __half2float(p.scales[ch0 + chl]) : 0.0f;
          const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
          const int used = min(G, kch);  // accumulators that received an MMA
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
#ifdef W8_TRACE
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

template <int NM, int G>
int launch_tc(const CUtensorMap &tmA, const TcDecodeParams &p) {
  Context &cx = ctx();
  int grid = cx.sm_count;
  if (grid > p.n) grid = p.n;
  // widest channel range any CTA gets in one pass
  int ch_max = (p.n + grid - 1) / grid;
  if (ch_max > CH_MAX) ch_max = CH_MAX;
  TcLayout lay;
  lay.tile_bytes = ((((ch_max + 7) / 8) * 8 * 128) + 1023) / 1024 * 1024;
  lay.slot_bytes = (NM * 128 + ch_max * 64 + 1023) / 1024 * 1024;
#ifdef W8_TRACE
  const int ctrl_bytes = 16 * MAX_SLOTS + 16 * 2 * G + 64 + 8192;
#else
  const int ctrl_bytes = 16 * MAX_SLOTS + 16 * 2 * G + 64;
#endif
  const int budget = 227 * 1024 - 1024 - ctrl_bytes - 2 * G * lay.tile_bytes;
  lay.n_slots = budget / lay.slot_bytes;
  if (lay.n_slots > MAX_SLOTS) lay.n_slots = MAX_SLOTS;
  if (lay.n_slots < G + 1)
    return set_error(B200MLIR_ERR_UNSUPPORTED, "w8a16: shared memory too small for %d rows", NM);
  const int smem = 2 * G * lay.tile_bytes + lay.n_slots * lay.slot_bytes + ctrl_bytes + 1024;
  auto kern = w8a16_tc_kernel<NM, G>;
  static bool attr_set = false;
  if (!attr_set) {
#ifdef W8_TRACE
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 8192));
#else
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
#endif
    attr_set = true;
  }
  kern<<<grid, (3 * G + 1) * 32, smem, cx.stream>>>(tmA, p, lay);
  return check_launch("w8a16_tc");
}

}  // namespace

#ifdef W8_TRACE
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

// Up to 256 rows per call (the caller loops over row passes).
int launch_w8a16_decode(const __half *a, const void *block_image, const __half *scales_dev, int64_t k,
                        int64_t n, __half *c, int64_t m, int64_t lda, int64_t ldc) {
  B200_TRY(ensure_ready());
  if (m < 1 || m > 256) return set_error(B200MLIR_ERR_BAD_ARG, "w8a16 tensor-core pass takes 1..256 rows");
  if (n > 0x7fffffff || k > 0x7fffffff) return set_error(B200MLIR_ERR_UNSUPPORTED, "w8a16: extent too large");
  TcDecodeParams p;
  p.k_chunks = (int)((k + 63) / 64);
  const int nm = m <= 16 ? 16 : (m <= 64 ? 64 : 256);
  CUtensorMap tmA;
  B200_TRY(make_a_map(&tmA, a, m, k, lda, nm));
  p.image = (const uint8_t *)block_image;
  p.scales = scales_dev;
  p.c = c;
  p.ldc = ldc;
  p.m = (int)m;
  p.n = (int)n;
  p.status = ctx().d_status;
  if (nm == 16) return launch_tc<16, 4>(tmA, p);
  if (nm == 64) return launch_tc<64, 4>(tmA, p);
  return launch_tc<256, 2>(tmA, p);
}

}  // namespace b200
