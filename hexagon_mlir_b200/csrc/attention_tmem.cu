// Attention block (QK · softmax · PV) as one tcgen05 kernel.
//
// What it computes is the reference's flash-attention kernel
// (test/python/triton/test_flash_attention.py:43-113 loop over key blocks, :116-195 set-up and
// final division): per block of keys, S = Q·Kᵀ; m' = max(m, rowmax(S)·c); P = exp2(S·c − m');
// l = l·exp2(m − m') + ΣP; O = O·exp2(m − m') + P·V; at the end O / l, with c = sm_scale·log2(e).
// Q, K, V and P are fp16 operands of the tensor cores, every sum is fp32.
//
// One CTA owns TILES tiles of 128 queries of one (batch, head).  Roles:
//   warps [4t, 4t+4)   softmax group of tile t: thread = one query row.  Reads S from TMEM twice
//                      (row maximum, then exponentials), writes P as packed fp16 back to TMEM, and
//                      keeps the row's O[D] in registers: O = O·alpha + (P·V read from TMEM).
//   warp 4·TILES       lane 0 issues every MMA: S_t = Q_t·Kᵀ (operands in shared memory) and
//                      PV_t = P_t·V (P from TMEM, V from shared memory), in the order
//                      PV(t,i), QK(t,i+1) so that a group's next S is on its way while the other
//                      group computes.
//   warp 4·TILES+1     lane 0 loads Q once and the K and V blocks into two rings with TMA.
// TMEM per tile: S [128 x BN] fp32, P [128 x BN] fp16 (BN/2 columns), PV [128 x D] fp32.
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
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
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
};

// status sites of this kernel
constexpr int ATT_SITE = 60;

template <int D, int BN, int TILES, int STAGES, bool OUT32>
__global__ void __launch_bounds__(128 * TILES + 64, 1)
    attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const AttParams p) {
  static_assert(D == 64 || D == 128, "head size");
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 128, "key block");
  constexpr int SLABS = D / 64;            // 64-column (128-byte) slabs of a tile row
  constexpr int Q_SLAB = ATT_BM * 128;     // bytes of one slab of a Q tile
  constexpr int Q_BYTES = SLABS * Q_SLAB;
  constexpr int KV_SLAB = BN * 128;
  constexpr int KV_BYTES = SLABS * KV_SLAB;
  constexpr int TCOLS = BN + BN / 2 + D;   // TMEM columns of one tile: S, P, PV
  constexpr int TMEM_COLS = TILES * TCOLS <= 256 ? 256 : 512;
  static_assert(TILES * TCOLS <= 512, "TMEM budget");
  constexpr int MMA_WARP = 4 * TILES, LOAD_WARP = 4 * TILES + 1;
  constexpr uint32_t IDESC_QK = make_idesc(/*D f32*/ 1, /*A f16*/ 0, /*B f16*/ 0, /*A K-major*/ 0,
                                           /*B K-major*/ 0, ATT_BM, BN);
  constexpr uint32_t IDESC_PV = make_idesc(/*D f32*/ 1, /*A f16*/ 0, /*B f16*/ 0, /*A K-major*/ 0,
                                           /*B MN-major*/ 1, ATT_BM, D);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base;
  const uint32_t k_smem = q_smem + TILES * Q_BYTES;
  const uint32_t v_smem = k_smem + STAGES * KV_BYTES;
  const uint32_t ctrl = v_smem + STAGES * KV_BYTES;
  const uint32_t bar_qfull = ctrl;            // TILES: Q tile landed
  const uint32_t bar_kfull = ctrl + 16;       // STAGES: K block landed
  const uint32_t bar_kempty = ctrl + 48;      // STAGES: every QK product that reads the stage is complete
  const uint32_t bar_vfull = ctrl + 80;       // STAGES
  const uint32_t bar_vempty = ctrl + 112;     // STAGES
  const uint32_t bar_sfull = ctrl + 144;      // TILES: S of the tile complete
  const uint32_t bar_pfull = ctrl + 160;      // TILES: P written (and S no longer needed), 4 warps
  const uint32_t bar_pvfull = ctrl + 176;     // TILES: P·V complete
  const uint32_t bar_pvfree = ctrl + 192;     // TILES: P·V read out, 4 warps
  const uint32_t tmem_slot = ctrl + 208;
  uint8_t *ctrl_ptr = smem_raw + (ctrl - smem_u32(smem_raw));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ctrl_ptr + 212);
  static_assert(STAGES <= 4, "barrier table");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * (TILES * ATT_BM);
  const int hh = blockIdx.y, zz = blockIdx.z;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int t = 0; t < TILES; ++t) {
      mbar_init(bar_qfull + 8 * t, 1);
      mbar_init(bar_sfull + 8 * t, 1);
      mbar_init(bar_pfull + 8 * t, 4);
      mbar_init(bar_pvfull + 8 * t, 1);
      mbar_init(bar_pvfree + 8 * t, 4);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, 1);
    }
    fence_barrier_init();
  }
  if (warp == MMA_WARP) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(ctrl_ptr + 208);

  if (warp < 4 * TILES) {
    // ---------------- softmax group of tile t: one thread per query row ----------------
    const int t = warp >> 2, q4 = warp & 3;
    const uint32_t t_s = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(t * TCOLS);
    const uint32_t t_p = t_s + BN;
    const uint32_t t_pv = t_p + BN / 2;
    const float c2 = p.scale2;
    float o[D];
#pragma unroll
    for (int e = 0; e < D; ++e) o[e] = 0.0f;
    float m = -1.0e30f, l = 0.0f, alpha_prev = 0.0f;
    bool ok = true;
    for (int i = 0; i < p.n_blocks; ++i) {
      const uint32_t par = (uint32_t)(i & 1);
      if (i > 0) {
        // P·V of the previous block: it was issued before this block's S, so it is complete first
        ok = mbar_wait(bar_pvfull + 8 * t, par ^ 1u, abort_flag, p.status, ATT_SITE + 1, i);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_pv + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[c * 32 + e] = fmaf(o[c * 32 + e], alpha_prev, __uint_as_float(r[e]));
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pvfree + 8 * t);
      }
      ok = mbar_wait(bar_sfull + 8 * t, par, abort_flag, p.status, ATT_SITE + 2, i);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int n_valid = p.n_ctx - i * BN;  // keys of this block that exist (the last block may be short)
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_s + c * 32, r);
        tmem_ld_wait();
        if (n_valid >= BN) {
#pragma unroll
          for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (c * 32 + e < n_valid) mx = fmaxf(mx, __uint_as_float(r[e]));
        }
      }
      const float m_new = fmaxf(m, mx * c2);
      const float alpha = ex2(m - m_new);
      float lsum = 0.0f;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_s + c * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float e0 = ex2(fmaf(__uint_as_float(r[2 * e]), c2, -m_new));
          float e1 = ex2(fmaf(__uint_as_float(r[2 * e + 1]), c2, -m_new));
          if (n_valid < BN) {
            if (c * 32 + 2 * e >= n_valid) e0 = 0.0f;
            if (c * 32 + 2 * e + 1 >= n_valid) e1 = 0.0f;
          }
          lsum += e0 + e1;
          pk[e] = pack_h2(e0, e1);
        }
        tmem_st_x16(t_p + c * 16, pk);
      }
      tmem_st_wait_all();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull + 8 * t);
      l = fmaf(l, alpha, lsum);
      alpha_prev = alpha;
      m = m_new;
    }
    if (ok) {
      ok = mbar_wait(bar_pvfull + 8 * t, (uint32_t)((p.n_blocks - 1) & 1), abort_flag, p.status, ATT_SITE + 3, 0);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const int row = m0 + t * ATT_BM + q4 * 32 + lane;
      const int64_t off = (int64_t)zz * p.so_z + (int64_t)hh * p.so_h + (int64_t)row * p.so_n;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_pv + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c * 32 + e] = fmaf(o[c * 32 + e], alpha_prev, __uint_as_float(r[e])) / l;
        if (row < p.n_ctx) {
          if (OUT32) {
            float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + off + c * 32);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              dst[e] = make_float4(o[c * 32 + 4 * e], o[c * 32 + 4 * e + 1], o[c * 32 + 4 * e + 2],
                                   o[c * 32 + 4 * e + 3]);
          } else {
            uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(p.out) + off + c * 32);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              dst[e] = make_uint4(pack_h2(o[c * 32 + 8 * e], o[c * 32 + 8 * e + 1]),
                                  pack_h2(o[c * 32 + 8 * e + 2], o[c * 32 + 8 * e + 3]),
                                  pack_h2(o[c * 32 + 8 * e + 4], o[c * 32 + 8 * e + 5]),
                                  pack_h2(o[c * 32 + 8 * e + 6], o[c * 32 + 8 * e + 7]));
          }
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      bool ok = true;
      for (int t = 0; t < TILES && ok; ++t)
        ok = mbar_wait(bar_qfull + 8 * t, 0u, abort_flag, p.status, ATT_SITE + 4, t);
      auto issue_qk = [&](int t, int stage) {
        const uint32_t qa = q_smem + t * Q_BYTES, ka = k_smem + stage * KV_BYTES;
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
          // both operands K-major: 8-row groups 1024 B apart, one K=16 step is 32 bytes inside the swizzle row
          const uint32_t in_row = (uint32_t)((j & 3) * 32);
          const uint64_t adesc = smem_desc_sw128(qa + (j >> 2) * Q_SLAB + in_row, 16, 1024);
          const uint64_t bdesc = smem_desc_sw128(ka + (j >> 2) * KV_SLAB + in_row, 16, 1024);
          mma_f16_ss(tmem_base + (uint32_t)(t * TCOLS), adesc, bdesc, IDESC_QK, j ? 1u : 0u);
        }
        mma_commit(bar_sfull + 8 * t);
      };
      auto issue_pv = [&](int t, int stage) {
        const uint32_t va = v_smem + stage * KV_BYTES;
        const uint32_t t_p = tmem_base + (uint32_t)(t * TCOLS + BN);
#pragma unroll
        for (int j = 0; j < BN / 16; ++j) {
          // V is MN-major: 64-column slabs KV_SLAB apart, 8-key groups 1024 B apart, one K=16 step is 16 rows
          const uint64_t bdesc = smem_desc_sw128(va + j * 2048, KV_SLAB, 1024);
          mma_f16_ts_att(t_p + BN / 2, t_p + (uint32_t)(j * 8), bdesc, IDESC_PV, j ? 1u : 0u);
        }
        mma_commit(bar_pvfull + 8 * t);
      };
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      if (ok) ok = mbar_wait(bar_kfull, 0u, abort_flag, p.status, ATT_SITE + 5, 0);
      if (ok) {
        tc_fence_after_sync();
        for (int t = 0; t < TILES; ++t) issue_qk(t, 0);
        mma_commit(bar_kempty);
        if (++ks == STAGES) {
          ks = 0;
          kph ^= 1u;
        }
      }
      for (int i = 0; i < p.n_blocks && ok; ++i) {
        const bool more = i + 1 < p.n_blocks;
        ok = mbar_wait(bar_vfull + 8 * vs, vph, abort_flag, p.status, ATT_SITE + 6, i);
        if (ok && more) ok = mbar_wait(bar_kfull + 8 * ks, kph, abort_flag, p.status, ATT_SITE + 7, i);
        for (int t = 0; t < TILES && ok; ++t) {
          ok = mbar_wait(bar_pfull + 8 * t, (uint32_t)(i & 1), abort_flag, p.status, ATT_SITE + 8, i);
          if (ok && i > 0)
            ok = mbar_wait(bar_pvfree + 8 * t, (uint32_t)((i - 1) & 1), abort_flag, p.status, ATT_SITE + 9, i);
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv(t, vs);
          if (more) issue_qk(t, ks);
        }
        if (!ok) break;
        mma_commit(bar_vempty + 8 * vs);
        if (++vs == STAGES) {
          vs = 0;
          vph ^= 1u;
        }
        if (more) {
          mma_commit(bar_kempty + 8 * ks);
          if (++ks == STAGES) {
            ks = 0;
            kph ^= 1u;
          }
        }
      }
    }
  } else if (warp == LOAD_WARP) {
    // ---------------- TMA producer ----------------
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
      int st = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int i = 0; i < p.n_blocks; ++i) {
        ok = mbar_wait(bar_kempty + 8 * st, ph ^ 1u, abort_flag, p.status, ATT_SITE + 10, i);
        if (!ok) break;
        mbar_expect_tx(bar_kfull + 8 * st, KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(k_smem + st * KV_BYTES + s * KV_SLAB, &tmK, bar_kfull + 8 * st, s * 64, i * BN, hh, zz);
        ok = mbar_wait(bar_vempty + 8 * st, ph ^ 1u, abort_flag, p.status, ATT_SITE + 11, i);
        if (!ok) break;
        mbar_expect_tx(bar_vfull + 8 * st, KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(v_smem + st * KV_BYTES + s * KV_SLAB, &tmV, bar_vfull + 8 * st, s * 64, i * BN, hh, zz);
        if (++st == STAGES) {
          st = 0;
          ph ^= 1u;
        }
      }
    }
  }
  // every role ends here; the accumulators are read, so TMEM can go back
  tc_fence_before_sync();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// fp32 [z,h,n,d] with the caller's strides -> contiguous fp16 (round to nearest even, as the
// engine's pack leaf does: bin/runtime/hmx/src/HMXLayout.c:257-264).
__global__ void attention_cast_kernel(const float *__restrict__ src, __half *__restrict__ dst, int64_t total4,
                                      int d4, int n, int h, int64_t sz, int64_t sh, int64_t sn) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % d4);
    int64_t r = i / d4;
    const int row = (int)(r % n);
    r /= n;
    const int hh = (int)(r % h);
    const int64_t zz = r / h;
    const float4 v = *reinterpret_cast<const float4 *>(src + zz * sz + hh * sh + (int64_t)row * sn + c * 4);
    uint2 o;
    o.x = pack_h2(v.x, v.y);
    o.y = pack_h2(v.z, v.w);
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

template <int D, int BN, int TILES, int STAGES, bool OUT32>
int launch_attention_variant(const void *q, const void *k, const void *v, void *out, const AttShape &in,
                             const AttShape &os, double sm_scale) {
  constexpr int SMEM = TILES * (D / 64) * ATT_BM * 128 + 2 * STAGES * (D / 64) * BN * 128 + 256 + 1024;
  static bool attr_set = false;
  auto kern = attention_kernel<D, BN, TILES, STAGES, OUT32>;
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
  dim3 grid((unsigned)((in.n + TILES * ATT_BM - 1) / (TILES * ATT_BM)), (unsigned)in.h, (unsigned)in.z);
  kern<<<grid, 128 * TILES + 64, SMEM, ctx().stream>>>(tmQ, tmK, tmV, p);
  count_launch();
  return check_launch("attention_kernel");
}

}  // namespace

int launch_attention(const void *q, const void *k, const void *v, void *out, bool f32, int64_t z, int64_t h,
                     int64_t n, int64_t d, int64_t sz, int64_t sh, int64_t sn, int64_t soz, int64_t soh,
                     int64_t son, double sm_scale) {
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
    const void *src[3] = {q, k, v};
    __half *dst = (__half *)ws;
    const int64_t total4 = (int64_t)each / 4;
    const int blocks = (int)std::min<int64_t>((total4 + 255) / 256, (int64_t)c.sm_count * 8);
    for (int i = 0; i < 3; ++i) {
      attention_cast_kernel<<<blocks, 256, 0, c.stream>>>((const float *)src[i], dst + i * each, total4, (int)(d / 4),
                                                          (int)n, (int)h, sz, sh, sn);
      count_launch();
    }
    B200_TRY(check_launch("attention_cast_kernel"));
    q = dst;
    k = dst + each;
    v = dst + 2 * each;
    in = AttShape{z, h, n, d, h * n * d, n * d, d};
  }
  const int64_t tiles = z * h * ((n + ATT_BM - 1) / ATT_BM);
  int two = tiles > c.sm_count ? 1 : 0;
  if (c.opt.attention_tiles == 1) two = 0;
  if (c.opt.attention_tiles == 2) two = 1;
#define ATT_GO(D_, BN_, T_, O_) launch_attention_variant<D_, BN_, T_, 3, O_>(q, k, v, out, in, os, sm_scale)
  if (d == 64) {
    if (two) return f32 ? ATT_GO(64, 128, 2, true) : ATT_GO(64, 128, 2, false);
    return f32 ? ATT_GO(64, 128, 1, true) : ATT_GO(64, 128, 1, false);
  }
  if (two) return f32 ? ATT_GO(128, 64, 2, true) : ATT_GO(128, 64, 2, false);
  return f32 ? ATT_GO(128, 64, 1, true) : ATT_GO(128, 64, 1, false);
#undef ATT_GO
}

}  // namespace b200
