// Attention block (QK · softmax · PV) as one tcgen05 kernel.
//
// What it computes is the reference's flash-attention kernel
// (test/python/triton/test_flash_attention.py:43-113 loop over key blocks, :116-195 set-up and
// final division): per block of keys, S = Q·Kᵀ; m' = max(m, rowmax(S)·c); P = exp2(S·c − m');
// l = l·exp2(m − m') + ΣP; O = O·exp2(m − m') + P·V; at the end O / l, with c = sm_scale·log2(e).
// Q, K, V and P are fp16 operands of the tensor cores, every sum is fp32.
//
// The kernel keeps m lazily: O lives in TMEM scaled by exp2(-m) and m moves only when the row
// maximum has grown by more than 2^8, in which case O and l are rescaled; O / l is the same.
//
// One CTA owns TILES tiles of 128 queries of one (batch, head); key blocks of 64.  Roles:
//   warps [4t, 4t+4)     softmax group of tile t: thread = one query row.  Reads the row of S from
//                        TMEM once, takes the maximum, writes P as packed fp16 back to TMEM.
//   warp 4·TILES + t     lane 0 issues tile t's score products S = Q·Kᵀ (both operands in shared
//                        memory), two blocks ahead of the softmax group.
//   warp 5·TILES + t     lane 0 issues tile t's O += P·V (P from TMEM, V from shared memory).
//   warp 6·TILES         lane 0 loads Q once and the K and V blocks into two rings with TMA.
// TMEM per tile (256 columns): S0, S1 [128 x 64] fp32; head size 64: P0, P1 (32 columns each) and
// O [128 x 64] fp32; head size 128: O [128 x 128] fp32 and P(i) written over the read half of S(i).
// Short problems share a tile's key blocks among several CTAs (partial O, m, l per row; merged by
// attention_combine_kernel); the causal form skips the blocks past a tile's diagonal and masks
// the two blocks on it.
// Every wait is bounded; a wait that runs out sets the CTA's abort flag and the device status.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cmath>

#include "common.h"
#include "gemm_tc_common.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {
using namespace ptx;

constexpr int ATT_BM = 128;

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two fp32 lanes per instruction (sm_100): {d0, d1} = {a0, a1} * {b, b} + {c, c}, and a packed add.
__device__ __forceinline__ void fma2(float &d0, float &d1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float &d0, float &d1, float a0, float a1) {
  asm("{\n\t.reg .b64 ra, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\t"
      "add.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait_all() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] · B[smem descriptor]
__device__ __forceinline__ void mma_f16_ts_att(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

struct AttParams {
  void *out;              // fp16 or fp32, same strides as the inputs
  int64_t so_z, so_h, so_n;  // output strides in elements
  int n_ctx, n_blocks;    // keys, and key blocks of BN
  float scale2;           // sm_scale · log2(e)
  int *status;
  // Short problems: the key blocks are split over `splits` CTAs per tile; each writes its
  // unnormalised O (fp32) and its (m, l) per row, and attention_combine_kernel merges them.
  int splits, rows_pad;   // rows_pad: rows of a (batch, head) rounded up to whole CTAs
  int causal;             // query i sees keys 0..i only (one tile per CTA, no key splits)
  int split_blk[17];      // key-block boundaries of the splits (splits <= 16), so that no CTA divides
  float *part_o;          // [z][h][split][rows_pad][D]
  float *part_ml;         // [z][h][split][rows_pad][2]
};

// Region stamps for timeline debugging (the analogue of the reference's light-weight profiling
// regions, lib/Transforms/HexagonLWPInstrumentation.cpp): compiled in only with
// -DB200MLIR_ATT_TRACE; CTA (0,0,0) records clock64() per role and key block.
#ifdef B200MLIR_ATT_TRACE
__device__ long long g_att_trace[8 * 32];
#define ATR(role, u) do { if ((blockIdx.x | blockIdx.y | blockIdx.z) == 0 && (u) < 32) trace_s[(role) * 32 + (u)] = clock64(); } while (0)
#else
#define ATR(role, u) do { } while (0)
#endif

// status sites of this kernel
constexpr int ATT_SITE = 60;

// Block: TILES softmax warpgroups, then per tile one warp that issues the score products and one
// that issues P·V, then the load warp.
constexpr int att_threads(int tiles) { return 32 * (6 * tiles + 1); }
constexpr int ATT_BN = 64;  // keys per block

// Pipeline of one tile (block i, S buffer b = i & 1):
//   score warp: QK(0), QK(1);  then per i:  wait P(i) -> QK(i+2) into buffer b
//   P·V warp:   per i:  wait P(i) -> O += P(i)·V(i)
//   softmax:   wait S(i) -> max -> (rarely: rescale O in TMEM) -> exponentials, P(i) -> signal
// O accumulates in TMEM over all blocks (P·V with accumulate), so the softmax thread holds only
// the row's scores; the next S is complete before the softmax group asks for it, and the group
// never waits for the tensor cores in steady state.
template <int D, int TILES, int KST, int VST, bool OUT32>
__global__ void __launch_bounds__(att_threads(TILES), 1)
    attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const AttParams p) {
  static_assert(D == 64 || D == 128, "head size");
  constexpr int BN = ATT_BN;
  constexpr bool ALIAS = D == 128;         // P(i) overwrites the first half of S(i) instead of its own columns
  constexpr int SLABS = D / 64;            // 64-column (128-byte) slabs of a tile row
  constexpr int Q_SLAB = ATT_BM * 128;     // bytes of one slab of a Q tile
  constexpr int Q_BYTES = SLABS * Q_SLAB;
  constexpr int KV_SLAB = BN * 128;
  constexpr int KV_BYTES = SLABS * KV_SLAB;
  // TMEM columns of one tile: S0 [0,64), S1 [64,128); D=64: P0 [128,160), P1 [160,192), PV [192,256);
  // D=128: PV [128,256)
  constexpr int TCOLS = 256;
  constexpr int COL_P = 128, COL_PV = ALIAS ? 128 : 192;
  constexpr int TMEM_COLS = TILES * TCOLS;
  constexpr int QK_WARP0 = 4 * TILES, PV_WARP0 = 5 * TILES, LOAD_WARP = 6 * TILES;
  constexpr uint32_t IDESC_QK = make_idesc(/*D f32*/ 1, /*A f16*/ 0, /*B f16*/ 0, /*A K-major*/ 0,
                                           /*B K-major*/ 0, ATT_BM, BN);
  constexpr uint32_t IDESC_PV = make_idesc(/*D f32*/ 1, /*A f16*/ 0, /*B f16*/ 0, /*A K-major*/ 0,
                                           /*B MN-major*/ 1, ATT_BM, D);

  extern __shared__ uint8_t smem_raw[];
#ifdef B200MLIR_ATT_TRACE
  __shared__ long long trace_s[8 * 32];
#endif
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base;
  const uint32_t k_smem = q_smem + TILES * Q_BYTES;
  const uint32_t v_smem = k_smem + KST * KV_BYTES;
  const uint32_t ctrl = v_smem + VST * KV_BYTES;
  const uint32_t bar_qfull = ctrl;            // [tile] Q tile landed
  const uint32_t bar_kfull = ctrl + 16;       // [stage] K block landed
  const uint32_t bar_kempty = ctrl + 48;      // [stage] every tile's QK product of the block is complete
  const uint32_t bar_vfull = ctrl + 80;       // [stage]
  const uint32_t bar_vempty = ctrl + 112;     // [stage] every tile's P·V of the block is complete
  const uint32_t bar_sfull = ctrl + 144;      // [tile][buffer] S complete
  const uint32_t bar_pfull = ctrl + 176;      // [tile][block parity] P written (and S read), 4 warps
  const uint32_t bar_pvfull = ctrl + 208;     // [tile][block parity] O += P·V of a block complete
  const uint32_t tmem_slot = ctrl + 240;
  uint8_t *ctrl_ptr = smem_raw + (ctrl - smem_u32(smem_raw));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ctrl_ptr + 244);
  static_assert(KST <= 4 && KST >= 2 && VST <= 4 && VST >= 2, "barrier table; K(i), K(i+1) are resident together");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // (divisions are kept off this path: the first loads wait for these numbers)
  const int mt = p.splits == 1 ? (int)blockIdx.x : (int)blockIdx.x / p.splits;
  const int split = (int)blockIdx.x - mt * p.splits;
  // causal: the last tiles have the most key blocks, so they are handed out first
  const int m0 = (p.causal ? (int)gridDim.x / p.splits - 1 - mt : mt) * (TILES * ATT_BM);
  const int hh = blockIdx.y, zz = blockIdx.z;
  // causal: the tile's last row m0 + 127 sees keys up to itself, later blocks are skipped altogether
  const int nb_tile = p.causal ? min(p.n_blocks, (m0 + TILES * ATT_BM - 1) / ATT_BN + 1) : p.n_blocks;
  const int blk0 = p.splits == 1 ? 0 : p.split_blk[split];           // this CTA's key blocks: [blk0, blk0 + nb)
  const int nb = (p.splits == 1 ? nb_tile : p.split_blk[split + 1]) - blk0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int t = 0; t < TILES; ++t) {
      mbar_init(bar_qfull + 8 * t, 1);
      mbar_init(bar_sfull + 16 * t, 1);
      mbar_init(bar_sfull + 16 * t + 8, 1);
      mbar_init(bar_pfull + 16 * t, 4);
      mbar_init(bar_pfull + 16 * t + 8, 4);
      mbar_init(bar_pvfull + 16 * t, 1);
      mbar_init(bar_pvfull + 16 * t + 8, 1);
    }
    for (int s = 0; s < KST; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, TILES);
    }
    for (int s = 0; s < VST; ++s) {
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, TILES);
    }
    fence_barrier_init();
  }
  if (warp == QK_WARP0) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(ctrl_ptr + 240);

  if (warp < 4 * TILES) {
    // ---------------- softmax group of tile t: one thread per query row ----------------
    const int t = warp >> 2, q4 = warp & 3;
    const uint32_t t_row = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(t * TCOLS);
    const uint32_t t_o = t_row + COL_PV;
    const float c2 = p.scale2;
    // O accumulates in TMEM across blocks, scaled by exp2(-m): m follows the row maximum lazily.
    // It moves only when the maximum has grown by more than kSlack (then P would leave fp16's
    // comfortable range): O and l are multiplied by exp2(m_old - m_new).  O / l does not depend
    // on which m was used, so the result is the reference's up to rounding.
    constexpr float kSlack = 8.0f;
    float m = -1.0e30f, l = 0.0f;
    bool ok = true;
    for (int i = 0; i < nb; ++i) {
      const int b = i & 1;
      ok = mbar_wait_parked(bar_sfull + 16 * t + 8 * b, (uint32_t)((i >> 1) & 1), abort_flag, p.status, ATT_SITE + 2, i);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (threadIdx.x == 0) ATR(4, i);
      tc_fence_after_sync();
      const uint32_t t_s = t_row + (uint32_t)(b * 64);
      const uint32_t t_p = ALIAS ? t_s : t_row + (uint32_t)(COL_P + b * 32);
      // the row's 64 scores stay in registers for both passes
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(t_s, s0);
      tmem_ld_32x32(t_s + 32, s1);
      tmem_ld_wait();
      const int n_valid = p.n_ctx - (blk0 + i) * BN;  // keys of this block that exist (the last block may be short)
      if (n_valid < BN) {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          if (e >= n_valid) s0[e] = 0xff800000u;  // -inf: no weight
          if (32 + e >= n_valid) s1[e] = 0xff800000u;
        }
      }
      if (p.causal && (blk0 + i) * BN + BN > m0) {
        // a block on the diagonal: keys after the thread's own row carry no weight
        const int over = m0 + t * ATT_BM + q4 * 32 + lane - (blk0 + i) * BN;  // last key offset this row may see
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          if (e > over) s0[e] = 0xff800000u;
          if (32 + e > over) s1[e] = 0xff800000u;
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 32; e += 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) mx[j] = max3(mx[j], __uint_as_float(s0[e + j]), __uint_as_float(s1[e + j]));
      }
      const float cur = max3(mx[0], mx[1], fmaxf(mx[2], mx[3])) * c2;
      if (__any_sync(0xffffffffu, cur > m + kSlack)) {
        const float m_new = fmaxf(m, cur);
        const float alpha = ex2(m - m_new);  // 0 on the first block, 1 for a row whose maximum stayed
        l *= alpha;
        m = m_new;
        if (i > 0) {
          // O must hold every product issued so far before it is rescaled
          ok = mbar_wait_parked(bar_pvfull + 16 * t + 8 * ((i - 1) & 1), (uint32_t)(((i - 1) >> 1) & 1), abort_flag, p.status,
                         ATT_SITE + 1, i);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_o + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st_x32(t_o + c * 32, r);
          }
        }
      }
      if (i >= 2) {
        // P(i) goes where P(i-2) was: the product that read it, two blocks old, is complete.  Every
        // barrier of this kernel belongs to a block parity, so its next phase cannot start before
        // each of its waiters has seen this one.
        ok = mbar_wait_parked(bar_pvfull + 16 * t + 8 * b, (uint32_t)(((i - 2) >> 1) & 1), abort_flag, p.status, ATT_SITE + 9, i);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (threadIdx.x == 0) ATR(6, i);
      }
      const float neg_m = -m;
      float ls[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float a0, a1;
          fma2(a0, a1, __uint_as_float(s0[2 * e]), __uint_as_float(s0[2 * e + 1]), c2, neg_m);
          a0 = ex2(a0);
          a1 = ex2(a1);
          add2(ls[0], ls[1], a0, a1);
          pk[e] = pack_h2(a0, a1);
        }
        tmem_st_x16(t_p, pk);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float a0, a1;
          fma2(a0, a1, __uint_as_float(s1[2 * e]), __uint_as_float(s1[2 * e + 1]), c2, neg_m);
          a0 = ex2(a0);
          a1 = ex2(a1);
          add2(ls[2], ls[3], a0, a1);
          pk[e] = pack_h2(a0, a1);
        }
        tmem_st_x16(t_p + 16, pk);
      }
      tmem_st_wait_all();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull + 16 * t + 8 * b);
      if (threadIdx.x == 0) ATR(5, i);
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
    }
    if (ok) {
      ok = mbar_wait_parked(bar_pvfull + 16 * t + 8 * ((nb - 1) & 1), (uint32_t)(((nb - 1) >> 1) & 1), abort_flag, p.status,
                     ATT_SITE + 3, 0);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const int row = m0 + t * ATT_BM + q4 * 32 + lane;
      const int64_t off = (int64_t)zz * p.so_z + (int64_t)hh * p.so_h + (int64_t)row * p.so_n;
      if (p.splits > 1) {
        // partial result of this key range: O as it stands (scaled by exp2(-m)), and (m, l)
        const int64_t prow = (((int64_t)zz * gridDim.y + hh) * p.splits + split) * p.rows_pad + row;
        float4 *dst = reinterpret_cast<float4 *>(p.part_o + prow * D);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_o + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 8; ++e)
            dst[c * 8 + e] = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]),
                                         __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
        }
        *reinterpret_cast<float2 *>(p.part_ml + prow * 2) = make_float2(m, l);
      } else {
      const float inv_l = 1.0f / l;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_o + c * 32, r);
        tmem_ld_wait();
        float o[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = __uint_as_float(r[e]) * inv_l;
        if (row < p.n_ctx) {
          if (OUT32) {
            float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + off + c * 32);
#pragma unroll
            for (int e = 0; e < 8; ++e) dst[e] = make_float4(o[4 * e], o[4 * e + 1], o[4 * e + 2], o[4 * e + 3]);
          } else {
            uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(p.out) + off + c * 32);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              dst[e] = make_uint4(pack_h2(o[8 * e], o[8 * e + 1]), pack_h2(o[8 * e + 2], o[8 * e + 3]),
                                  pack_h2(o[8 * e + 4], o[8 * e + 5]), pack_h2(o[8 * e + 6], o[8 * e + 7]));
          }
        }
      }
      }
    }
  } else if (warp >= QK_WARP0 && warp < QK_WARP0 + TILES) {
    // ---------------- score products of tile t: S(i+2) = Q·K(i+2)ᵀ as soon as S(i) is read ----------------
    if (lane == 0) {
      const int t = warp - QK_WARP0;
      const uint32_t tm = tmem_base + (uint32_t)(t * TCOLS);
      bool ok = mbar_wait_parked(bar_qfull + 8 * t, 0u, abort_flag, p.status, ATT_SITE + 4, t);
      // descriptors of the ring's first stage; a stage or a K=16 step adds a constant to the address field
      const uint64_t qdesc = smem_desc_sw128(q_smem + t * Q_BYTES, 16, 1024);
      const uint64_t kdesc0 = smem_desc_sw128(k_smem, 16, 1024);
      int ks = 0;
      uint32_t kph = 0;
      auto issue_qk = [&](int buf, int blk) -> bool {
        if (!mbar_wait_parked(bar_kfull + 8 * ks, kph, abort_flag, p.status, ATT_SITE + 5, blk)) return false;
        tc_fence_after_sync();
        const uint64_t kd = kdesc0 + (uint64_t)((ks * KV_BYTES) >> 4);
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
          // both operands K-major: 8-row groups 1024 B apart, a K=16 step is 32 bytes inside the swizzle row
          const uint64_t qo = (uint64_t)(((j >> 2) * Q_SLAB + (j & 3) * 32) >> 4);
          const uint64_t ko = (uint64_t)(((j >> 2) * KV_SLAB + (j & 3) * 32) >> 4);
          mma_f16_ss(tm + (uint32_t)(buf * 64), qdesc + qo, kd + ko, IDESC_QK, j ? 1u : 0u);
        }
        mma_commit(bar_sfull + 16 * t + 8 * buf);
        mma_commit(bar_kempty + 8 * ks);
        if (++ks == KST) {
          ks = 0;
          kph ^= 1u;
        }
        return true;
      };
      if (ok) ok = issue_qk(0, 0);
      if (ok && nb > 1) ok = issue_qk(1, 1);
      for (int i = 0; i + 2 < nb && ok; ++i) {
        const int b = i & 1;
        const uint32_t ph = (uint32_t)((i >> 1) & 1);
        ok = mbar_wait_parked(bar_pfull + 16 * t + 8 * b, ph, abort_flag, p.status, ATT_SITE + 8, i);
        if (ok && ALIAS)  // P(i) lives in the S buffer this product overwrites: P·V(i) must have read it
          ok = mbar_wait_parked(bar_pvfull + 16 * t + 8 * b, ph, abort_flag, p.status, ATT_SITE + 7, i);
        if (!ok) break;
        if (t == 0) ATR(3, i);
        ok = issue_qk(b, i + 2);
        if (t == 0) ATR(2, i);
      }
    }
  } else if (warp >= PV_WARP0 && warp < PV_WARP0 + TILES) {
    // ---------------- O += P(i)·V(i) of tile t ----------------
    if (lane == 0) {
      const int t = warp - PV_WARP0;
      const uint32_t tm = tmem_base + (uint32_t)(t * TCOLS);
      const uint64_t vdesc0 = smem_desc_sw128(v_smem, KV_SLAB, 1024);
      int vs = 0;
      uint32_t vph = 0;
      bool ok = true;
      for (int i = 0; i < nb && ok; ++i) {
        const int b = i & 1;
        ok = mbar_wait_parked(bar_pfull + 16 * t + 8 * b, (uint32_t)((i >> 1) & 1), abort_flag, p.status, ATT_SITE + 12, i);
        if (ok) ok = mbar_wait_parked(bar_vfull + 8 * vs, vph, abort_flag, p.status, ATT_SITE + 6, i);
        if (!ok) break;
        if (t == 0) ATR(0, i);
        tc_fence_after_sync();
        const uint32_t a_tmem = tm + (uint32_t)(ALIAS ? b * 64 : COL_P + b * 32);
        const uint64_t vd = vdesc0 + (uint64_t)((vs * KV_BYTES) >> 4);
#pragma unroll
        for (int j = 0; j < BN / 16; ++j) {
          // V is MN-major: 64-column slabs KV_SLAB apart, 8-key groups 1024 B apart, a K=16 step is 16 rows
          mma_f16_ts_att(tm + COL_PV, a_tmem + (uint32_t)(j * 8), vd + (uint64_t)(j * 128), IDESC_PV, (i | j) ? 1u : 0u);
        }
        mma_commit(bar_pvfull + 16 * t + 8 * b);
        mma_commit(bar_vempty + 8 * vs);
        if (++vs == VST) {
          vs = 0;
          vph ^= 1u;
        }
        if (t == 0) ATR(1, i);
      }
    }
  } else if (warp == LOAD_WARP) {
    // ---------------- TMA producer: Q, then K(0), K(1), V(0), K(2), V(1), K(3), ... ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      for (int t = 0; t < TILES; ++t) {
        mbar_expect_tx(bar_qfull + 8 * t, Q_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(q_smem + t * Q_BYTES + s * Q_SLAB, &tmQ, bar_qfull + 8 * t, s * 64, m0 + t * ATT_BM, hh, zz);
      }
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      bool ok = true;
      auto load_k = [&](int blk) {
        ok = mbar_wait_parked(bar_kempty + 8 * ks, kph ^ 1u, abort_flag, p.status, ATT_SITE + 10, blk);
        if (!ok) return;
        mbar_expect_tx(bar_kfull + 8 * ks, KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(k_smem + ks * KV_BYTES + s * KV_SLAB, &tmK, bar_kfull + 8 * ks, s * 64, (blk0 + blk) * BN, hh, zz);
        if (++ks == KST) {
          ks = 0;
          kph ^= 1u;
        }
      };
      load_k(0);
      if (ok && nb > 1) load_k(1);
      for (int i = 0; i < nb && ok; ++i) {
        ok = mbar_wait_parked(bar_vempty + 8 * vs, vph ^ 1u, abort_flag, p.status, ATT_SITE + 11, i);
        if (!ok) break;
        mbar_expect_tx(bar_vfull + 8 * vs, KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(v_smem + vs * KV_BYTES + s * KV_SLAB, &tmV, bar_vfull + 8 * vs, s * 64, (blk0 + i) * BN, hh, zz);
        if (++vs == VST) {
          vs = 0;
          vph ^= 1u;
        }
        if (i + 2 < nb) load_k(i + 2);
      }
    }
  }
  // every role ends here; the accumulators are read, so TMEM can go back
  tc_fence_before_sync();
  __syncthreads();
#ifdef B200MLIR_ATT_TRACE
  if ((blockIdx.x | blockIdx.y | blockIdx.z) == 0)
    for (int i = threadIdx.x; i < 8 * 32; i += blockDim.x) g_att_trace[i] = trace_s[i];
#endif
  if (warp == QK_WARP0) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Merges the partial results of a split attention: per row M = max_s m_s,
// out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).  One thread per (row, 8 columns).
template <bool OUT32>
__global__ void attention_combine_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, void *out,
                                         int64_t total, int splits, int rows_pad, int n_ctx, int d, int h,
                                         int64_t so_z, int64_t so_h, int64_t so_n) {
  const int groups = d / 8;
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int g = (int)(idx % groups);
  const int64_t rr = idx / groups;
  const int row = (int)(rr % n_ctx);
  const int64_t zh = rr / n_ctx;
  const int64_t base = zh * splits * rows_pad + row;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_ml[(base + (int64_t)s * rows_pad) * 2]);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, lsum = 0.0f;
  for (int s = 0; s < splits; ++s) {
    const int64_t pr = base + (int64_t)s * rows_pad;
    const float w = exp2f(part_ml[pr * 2] - mx);
    lsum = fmaf(part_ml[pr * 2 + 1], w, lsum);
    const float4 a = *reinterpret_cast<const float4 *>(part_o + pr * d + g * 8);
    const float4 b = *reinterpret_cast<const float4 *>(part_o + pr * d + g * 8 + 4);
    acc[0] = fmaf(a.x, w, acc[0]); acc[1] = fmaf(a.y, w, acc[1]); acc[2] = fmaf(a.z, w, acc[2]); acc[3] = fmaf(a.w, w, acc[3]);
    acc[4] = fmaf(b.x, w, acc[4]); acc[5] = fmaf(b.y, w, acc[5]); acc[6] = fmaf(b.z, w, acc[6]); acc[7] = fmaf(b.w, w, acc[7]);
  }
  const float inv = 1.0f / lsum;
  const int64_t off = (zh / h) * so_z + (zh % h) * so_h + (int64_t)row * so_n + g * 8;
  if (OUT32) {
    float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + off);
    dst[0] = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    dst[1] = make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
  } else {
    *reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(out) + off) =
        make_uint4(pack_h2(acc[0] * inv, acc[1] * inv), pack_h2(acc[2] * inv, acc[3] * inv),
                   pack_h2(acc[4] * inv, acc[5] * inv), pack_h2(acc[6] * inv, acc[7] * inv));
  }
}

// fp32 [z,h,n,d] with the caller's strides -> contiguous fp16 (round to nearest even, as the
// engine's pack leaf does: bin/runtime/hmx/src/HMXLayout.c:257-264).
__global__ void attention_cast_kernel(const float *__restrict__ q, const float *__restrict__ k,
                                      const float *__restrict__ v, __half *__restrict__ dst, int64_t total4, int d4,
                                      int n, int h, int64_t sz, int64_t sh, int64_t sn) {
  // blockIdx.y picks the operand; the three results are stored one after the other
  const float *src = blockIdx.y == 0 ? q : blockIdx.y == 1 ? k : v;
  dst += (int64_t)blockIdx.y * total4 * 4;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % d4);
    int64_t r = i / d4;
    const int row = (int)(r % n);
    r /= n;
    const int hh = (int)(r % h);
    const int64_t zz = r / h;
    const float4 x = *reinterpret_cast<const float4 *>(src + zz * sz + hh * sh + (int64_t)row * sn + c * 4);
    uint2 o;
    o.x = pack_h2(x.x, x.y);
    o.y = pack_h2(x.z, x.w);
    *reinterpret_cast<uint2 *>(dst + i * 4) = o;
  }
}

// fp16 tensor [z, h, n, d] (d contiguous) as a 4-D map; box = {64 columns, box_rows rows}.
int make_map_qkv(CUtensorMap *map, const void *base, int64_t z, int64_t h, int64_t n, int64_t d, int64_t sz,
                 int64_t sh, int64_t sn, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(B200MLIR_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available");
  // a dimension of extent 1 is never stepped: give it a stride the encoder accepts
  if (h == 1) sh = n * sn;
  if (z == 1) sz = h * sh > n * sn ? h * sh : n * sn;
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)n, (cuuint64_t)h, (cuuint64_t)z};
  cuuint64_t strides[3] = {(cuuint64_t)sn * 2, (cuuint64_t)sh * 2, (cuuint64_t)sz * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(B200MLIR_ERR_CUDA, "attention: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

struct AttShape {
  int64_t z, h, n, d, sz, sh, sn;
};

template <int D, int TILES, int KST, int VST, bool OUT32>
int launch_attention_variant(const void *q, const void *k, const void *v, void *out, const AttShape &in,
                             const AttShape &os, double sm_scale, bool causal) {
  constexpr int BN = ATT_BN;
  constexpr int SMEM = TILES * (D / 64) * ATT_BM * 128 + (KST + VST) * (D / 64) * BN * 128 + 256 + 1024;
  static bool attr_set = false;
  auto kern = attention_kernel<D, TILES, KST, VST, OUT32>;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    attr_set = true;
  }
  CUtensorMap tmQ, tmK, tmV;
  B200_TRY(make_map_qkv(&tmQ, q, in.z, in.h, in.n, in.d, in.sz, in.sh, in.sn, ATT_BM));
  B200_TRY(make_map_qkv(&tmK, k, in.z, in.h, in.n, in.d, in.sz, in.sh, in.sn, BN));
  B200_TRY(make_map_qkv(&tmV, v, in.z, in.h, in.n, in.d, in.sz, in.sh, in.sn, BN));
  AttParams p;
  p.out = out;
  p.so_z = os.sz;
  p.so_h = os.sh;
  p.so_n = os.sn;
  p.n_ctx = (int)in.n;
  p.n_blocks = (int)((in.n + BN - 1) / BN);
  p.scale2 = (float)(sm_scale * 1.44269504);  // the kernel source's own constant for 1/ln 2
  p.status = ctx().d_status;
  // Few tiles and many key blocks: split the keys so that more SMs work.  Two CTAs fit an SM, so
  // there are 2 x SMs places; a split keeps at least four blocks, and problems with fewer than 16
  // blocks are not worth the merge (measured: 1x1x1024x64 14.4 -> 10.3 us, 1x2x4096x64 46.6 -> 23.4,
  // 2x8x512x64 9.3 -> 10.3 when split).  Option attentionSplits overrides (0 = this rule).
  const int grid_m = (int)((in.n + TILES * ATT_BM - 1) / (TILES * ATT_BM));
  const int64_t ctas = (int64_t)grid_m * in.h * in.z;
  int splits = 1;
  if (ctas * 2 <= ctx().sm_count && p.n_blocks >= 16)
    splits = (int)std::min<int64_t>(std::min<int64_t>(p.n_blocks / 4, 2 * ctx().sm_count / ctas), 8);
  if (ctx().opt.attention_splits >= 1) splits = (int)std::min<double>(ctx().opt.attention_splits, (double)p.n_blocks);
  p.causal = causal ? 1 : 0;
  if (causal) splits = 1;  // the tiles of a causal problem have different numbers of key blocks
  if (splits > 16) splits = 16;
  p.splits = splits;
  for (int i = 0; i <= 16; ++i) p.split_blk[i] = i <= splits ? (int)((int64_t)p.n_blocks * i / splits) : p.n_blocks;
  p.rows_pad = grid_m * TILES * ATT_BM;
  p.part_o = nullptr;
  p.part_ml = nullptr;
  if (splits > 1) {
    const size_t rows = (size_t)in.z * in.h * splits * p.rows_pad;
    void *ws = nullptr;
    B200_TRY(workspace2(rows * (D + 2) * sizeof(float), &ws));
    p.part_o = (float *)ws;
    p.part_ml = p.part_o + rows * D;
  }
  dim3 grid((unsigned)(grid_m * splits), (unsigned)in.h, (unsigned)in.z);
  kern<<<grid, att_threads(TILES), SMEM, ctx().stream>>>(tmQ, tmK, tmV, p);
  if (splits > 1) {
    B200_TRY(check_launch("attention_kernel"));
    const int64_t total = (int64_t)in.z * in.h * in.n * (D / 8);
    attention_combine_kernel<OUT32><<<(unsigned)((total + 127) / 128), 128, 0, ctx().stream>>>(
        p.part_o, p.part_ml, out, total, splits, p.rows_pad, (int)in.n, D, (int)in.h, os.sz, os.sh, os.sn);
    return check_launch("attention_combine_kernel");
  }
  return check_launch("attention_kernel");
}

}  // namespace

#ifdef B200MLIR_ATT_TRACE
extern "C" __attribute__((visibility("default"))) int b200mlir_debug_get_att_trace(long long *host) {
  return (int)cudaMemcpyFromSymbol(host, g_att_trace, sizeof(long long) * 8 * 32);
}
#endif

int launch_attention(const void *q, const void *k, const void *v, void *out, bool f32, int64_t z, int64_t h,
                     int64_t n, int64_t d, int64_t sz, int64_t sh, int64_t sn, int64_t soz, int64_t soh,
                     int64_t son, double sm_scale, bool causal) {
  Context &c = ctx();
  if (d != 64 && d != 128) return set_error(B200MLIR_ERR_UNSUPPORTED, "attention: head size %lld (64 or 128)", (long long)d);
  if (z < 1 || h < 1 || n < 1 || h > 65535 || z > 65535 || n > (1 << 30))
    return set_error(B200MLIR_ERR_BAD_ARG, "attention: bad extents z=%lld h=%lld n=%lld", (long long)z, (long long)h, (long long)n);
  if (!(sm_scale > 0.0) || !std::isfinite(sm_scale))
    return set_error(B200MLIR_ERR_BAD_ARG, "attention: sm_scale must be positive and finite");
  if (sn < d || sn % 8 || (h > 1 && sh % 8) || (z > 1 && sz % 8) || son < d || son % 8 || (h > 1 && soh % 8) ||
      (z > 1 && soz % 8))
    return set_error(B200MLIR_ERR_BAD_ARG, "attention: strides must be multiples of 8 elements and rows at least d_head apart");
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
    return set_error(B200MLIR_ERR_BAD_ARG, "attention: tensors must be 16-byte aligned");
  AttShape in{z, h, n, d, sz, sh, sn}, os{z, h, n, d, soz, soh, son};
  if (f32) {
    // quantise the three operands once into the workspace, contiguous [z,h,n,d]
    const size_t each = (size_t)z * h * n * d;
    void *ws = nullptr;
    B200_TRY(workspace(3 * each * sizeof(__half), &ws));
    __half *dst = (__half *)ws;
    const int64_t total4 = (int64_t)each / 4;
    const int blocks = (int)std::min<int64_t>((total4 + 255) / 256, (int64_t)c.sm_count * 8);
    attention_cast_kernel<<<dim3(blocks, 3), 256, 0, c.stream>>>((const float *)q, (const float *)k, (const float *)v,
                                                                 dst, total4, (int)(d / 4), (int)n, (int)h, sz, sh, sn);
    B200_TRY(check_launch("attention_cast_kernel"));
    q = dst;
    k = dst + each;
    v = dst + 2 * each;
    in = AttShape{z, h, n, d, h * n * d, n * d, d};
  }
  // One tile per CTA and two CTAs per SM measured as fast as or faster than two tiles in one CTA
  // at both head sizes (4 x 16 x 4096: 679 against 597 TFLOP/s at 64, 1075 against 1062 at 128);
  // option attentionTiles = 2 selects the two-tile form.
  const int two = c.opt.attention_tiles == 2 && !causal ? 1 : 0;  // (causal: one tile per CTA)
#define ATT_GO(D_, T_, K_, V_, O_) launch_attention_variant<D_, T_, K_, V_, O_>(q, k, v, out, in, os, sm_scale, causal)
  if (d == 64) {
    if (two) return f32 ? ATT_GO(64, 2, 4, 4, true) : ATT_GO(64, 2, 4, 4, false);
    return f32 ? ATT_GO(64, 1, 4, 4, true) : ATT_GO(64, 1, 4, 4, false);
  }
  if (two) return f32 ? ATT_GO(128, 2, 3, 3, true) : ATT_GO(128, 2, 3, 3, false);
  return f32 ? ATT_GO(128, 1, 2, 2, true) : ATT_GO(128, 1, 2, 2, false);
#undef ATT_GO
}

}  // namespace b200
