// fp16 GEMM over SM pairs for grids that do not fill the machine: the 256 x 256 pair kernel with
// the K dimension of its tiles dealt out evenly ("stream-K").
//
// Why: with whole tiles per pair, a problem of T tiles on P pairs takes ceil(T / P) rounds — 43
// tiles leave 31 of 74 pairs idle, 86 tiles cost two rounds for 1.16 rounds of work.  Here the
// unit of work is one 64-deep k-block of one tile; the T * KB units are cut into P contiguous,
// equal ranges, so a pair's range is: the tail of one tile, whole tiles, the head of another.
//
// A tile cut between pairs needs its partial sums combined.  The reference combines K segments in
// fp32 after the engine's read-out (hmx/src/HMXLayout.c:880-901; the span count of a tiling,
// backend/hmx_search.py:221-232); here every contributor of a cut tile stores its fp32 partial
// (as it lies in TMEM: column-major per 32-row slab, so the stores coalesce) into its own slot of
// a resident workspace, then bumps the slab's arrival counter; whichever contributor arrives LAST
// sums all partials — its own included, re-read from the workspace — in contributor order and
// runs the fused read-out.  Nobody waits for anybody (no spin, nothing to time out), and because
// the order of the sum is fixed by the partition, not by arrival, results are bit-reproducible
// run to run.  The counters return to zero before the kernel ends.
//
// Roles, barriers and the operand path are those of the pair kernel (gemm_tcgen05_2cta.cu).
#include <cstdlib>
#include <cstring>

#include "common.h"
#include "gemm_tc2_common.cuh"

namespace b200 {
namespace {

using namespace ptx;

constexpr int SK_STAGES = 6;
constexpr int SK_TILE_ROWS = 256, SK_TILE_COLS = 256;
constexpr int SK_MAX_TILES = 8192;                                   // arrival counters: 8 per tile
constexpr size_t SK_COUNTER_BYTES = (size_t)SK_MAX_TILES * 8 * sizeof(int);
constexpr size_t SK_SLAB_FLOATS = 32 * 256;                          // one warp's 32 rows x 256 accumulator columns
constexpr size_t SK_CTA_FLOATS = 4 * SK_SLAB_FLOATS;                 // 128 rows
constexpr size_t SK_SLOT_FLOATS = 2 * SK_CTA_FLOATS;                 // both CTAs of the pair: 256 KiB of fp32

struct SkParams {
  TcParams t;
  int units_q, units_r;   // pair p owns units [p*q + min(p, r), (p+1)*q + min(p+1, r))
  int *counters;          // [tile][cta rank][lane quadrant]
  float *partials;        // [pair][slot 0/1][cta rank][quadrant][column][lane]
};

__device__ __forceinline__ int sk_unit_begin(int p, int q, int r) { return p * q + min(p, r); }
__device__ __forceinline__ int sk_pair_of_unit(int u, int q, int r) {
  const int wide = (q + 1) * r;  // the first r pairs own q + 1 units each
  return u < wide ? u / (q + 1) : r + (u - wide) / q;
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS2, 1)
gemm_tc2_streamk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmB2, const SkParams sp) {
  const TcParams &p = sp.t;
  constexpr int BN_MMA = 256;
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? 128 : 256;
  constexpr int TMEM_COLS = 512;
  constexpr uint32_t IDESC = make_idesc(/*D=f32*/ 1, /*A=f16*/ 0, /*B=f16*/ 0, /*A K-major*/ 0, /*B MN-major*/ 1, 256,
                                        BN_MMA);
  constexpr int STAGES = SK_STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ctrl = smem_base + STAGES * STAGE2_BYTES;
  const uint32_t bar_full = ctrl;
  const uint32_t bar_empty = ctrl + 8 * STAGES;
  const uint32_t bar_tfull = ctrl + 16 * STAGES;
  const uint32_t bar_tempty = ctrl + 16 * STAGES + 16;
  const uint32_t tmem_slot = ctrl + 16 * STAGES + 32;
  uint8_t *ctrl_gen = smem_raw + (ctrl - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(ctrl_gen + 16 * STAGES + 32);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ctrl_gen + 16 * STAGES + 36);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int KB = p.k_blocks;
  const int u_begin = sk_unit_begin(pair, sp.units_q, sp.units_r);
  const int u_end = sk_unit_begin(pair + 1, sp.units_q, sp.units_r);
  pdl_trigger();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 2);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (EPI == EPI_SWIGLU) tma_prefetch_desc(&tmB2);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = u_begin; ok && u < u_end;) {
        const int tile = u / KB, kb0 = u - tile * KB;
        const int kb1 = min(KB, kb0 + (u_end - u));
        int m_blk, n_blk;
        tile_coords(tile, p.m_blocks, p.n_blocks, p.group_m, m_blk, n_blk);
        const int m0 = m_blk * 256 + (int)rank * BM2;
        const int n0 = n_blk * BN_OUT;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, 41, tile)) {
            ok = false;
            break;
          }
          const uint32_t full = map_to_cta(bar_full + 8 * stage, 0);
          remote_expect_tx(full, STAGE2_BYTES);
          const uint32_t sa = smem_base + stage * STAGE2_BYTES;
          const uint32_t sb = sa + A2_BYTES;
          const int k0 = kb * BK2;
          tma_load_2d_pair(sa, &tmA, full, k0, m0);
          if (EPI == EPI_SWIGLU) {
            const CUtensorMap *mb = leader ? &tmB : &tmB2;  // gate half / up half
            tma_load_2d_pair(sb, mb, full, n0, k0);
            tma_load_2d_pair(sb + SLAB_BYTES, mb, full, n0 + 64, k0);
          } else {
            const int nb = n0 + (int)rank * 128;
            tma_load_2d_pair(sb, &tmB, full, nb, k0);
            tma_load_2d_pair(sb + SLAB_BYTES, &tmB, full, nb + 64, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        u += kb1 - kb0;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only): one accumulator stage per segment ----------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = u_begin; ok && u < u_end;) {
        const int tile = u / KB, kb0 = u - tile * KB;
        const int kb1 = min(KB, kb0 + (u_end - u));
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, 42, tile)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN_MMA);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, 43, tile)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * STAGE2_BYTES;
          const uint32_t sb = sa + A2_BYTES;
          const uint64_t adesc = smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = smem_desc_sw128(sb, SLAB_BYTES, 1024);
#pragma unroll
          for (int k = 0; k < BK2 / 16; ++k)
            mma_f16_pair(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 128), IDESC,
                         (kb != kb0 || k != 0) ? 1u : 0u);
          mma_commit_pair(bar_empty + 8 * stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        mma_commit_pair(bar_tfull + 8 * acc);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
        u += kb1 - kb0;
      }
    }
  } else {
    // ---------------- read-out (warps 2..5): this CTA's 128 rows ----------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    int seg = 0;
    for (int u = u_begin; u < u_end; ++seg) {
      const int tile = u / KB, kb0 = u - tile * KB;
      const int kb1 = min(KB, kb0 + (u_end - u));
      u += kb1 - kb0;
      int m_blk, n_blk;
      tile_coords(tile, p.m_blocks, p.n_blocks, p.group_m, m_blk, n_blk);
      const int m0 = m_blk * 256 + (int)rank * BM2, n0 = n_blk * BN_OUT;
      bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, 44, tile);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN_MMA);
      const bool whole = kb0 == 0 && kb1 == KB;
      if (whole) {
#pragma unroll 1
        for (int c = 0; c < BN_OUT / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          uint32_t r2[32];
          if (EPI == EPI_SWIGLU) tmem_ld_32x32(t_row + BN_OUT + c * 32, r2);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (!row_ok || col0 >= p.n) continue;
          epilogue_store_chunk<EPI>(r, r2, row, col0, p);
        }
      } else {
        // this pair's partial of the tile, all 256 accumulator columns of the slab, as it lies in
        // TMEM: element (column j, lane l) at j*32 + l, so the 32 lanes of a store are contiguous
        float *mine = sp.partials + ((size_t)pair * 2 + (seg == 0 ? 0 : 1)) * SK_SLOT_FLOATS + (size_t)rank * SK_CTA_FLOATS +
                      (size_t)q * SK_SLAB_FLOATS;
#pragma unroll 1
        for (int c = 0; c < BN_MMA / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) __stcg(mine + (c * 32 + j) * 32 + lane, __uint_as_float(r[j]));
        }
      }
      // the accumulator stage is free once it has been read (the partial lives in memory now)
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) remote_arrive(map_to_cta(bar_tempty + 8 * acc, 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
      if (whole) continue;
      // ---- arrival: the last contributor of this 32-row slab combines and reads out ----
      const int t_first = tile * KB;
      const int p_first = sk_pair_of_unit(t_first, sp.units_q, sp.units_r);
      const int p_last = sk_pair_of_unit(t_first + KB - 1, sp.units_q, sp.units_r);
      const int contributors = p_last - p_first + 1;
      int *counter = sp.counters + ((size_t)tile * 2 + rank) * 4 + q;
      __threadfence();  // the partial is visible device-wide before the arrival is
      __syncwarp();
      int arrived = 0;
      if (lane == 0) arrived = atomicAdd(counter, 1);
      arrived = __shfl_sync(0xffffffffu, arrived, 0);
      if (arrived != contributors - 1) continue;
      __threadfence();
      if (lane == 0) *counter = 0;  // clean for the next launch; nobody else touches it any more
      // contributor c is pair p_first + c; every contributor after the first began its range inside
      // this tile, so its partial is in its slot 0; the first one's is in slot 0 only if its range
      // begins exactly with this tile
      const bool first_in_slot0 = sk_unit_begin(p_first, sp.units_q, sp.units_r) >= t_first;
#pragma unroll 1
      for (int c = 0; c < BN_OUT / 32; ++c) {
        float s[32], s2[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) s[j] = s2[j] = 0.0f;
        for (int ci = 0; ci < contributors; ++ci) {
          const int slot = (ci == 0 && !first_in_slot0) ? 1 : 0;
          const float *src = sp.partials + ((size_t)(p_first + ci) * 2 + slot) * SK_SLOT_FLOATS +
                             (size_t)rank * SK_CTA_FLOATS + (size_t)q * SK_SLAB_FLOATS;
#pragma unroll
          for (int j = 0; j < 32; ++j) s[j] += __ldcg(src + (c * 32 + j) * 32 + lane);
          if (EPI == EPI_SWIGLU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) s2[j] += __ldcg(src + (BN_OUT + c * 32 + j) * 32 + lane);
          }
        }
        const int col0 = n0 + c * 32;
        if (!row_ok || col0 >= p.n) continue;
        uint32_t r[32], r2[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          r[j] = __float_as_uint(s[j]);
          r2[j] = __float_as_uint(s2[j]);
        }
        epilogue_store_chunk<EPI>(r, r2, row, col0, p);
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1 && *abort_flag)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  cluster_sync();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

constexpr int kSmemSk = SK_STAGES * STAGE2_BYTES + 16 * SK_STAGES + 64 + 1024;

template <int EPI>
int launch_streamk(const GemmArgs &g) {
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? 128 : 256;
  Context &c = ctx();
  CUtensorMap tmA, tmB, tmB2;
  B200_TRY(make_map_2d(&tmA, g.a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.k, g.m, g.lda, BK2, BM2));
  B200_TRY(make_map_2d(&tmB, g.b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.n, g.k, g.ldb, 64, BK2));
  if (EPI == EPI_SWIGLU)
    B200_TRY(make_map_2d(&tmB2, g.b2, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.n, g.k, g.ldb, 64, BK2));
  else
    tmB2 = tmB;
  SkParams sp;
  TcParams &p = sp.t;
  p.c = g.c;
  p.res = g.res;
  p.ldc = g.ldc;
  p.ldres = g.ldres;
  p.m = (int)g.m;
  p.n = (int)g.n;
  p.k = (int)g.k;
  p.m_blocks = (int)((g.m + 255) / 256);
  p.n_blocks = (int)((g.n + BN_OUT - 1) / BN_OUT);
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.k_blocks = (int)((g.k + BK2 - 1) / BK2);
  p.group_m = ctx().opt.gemm_group_m >= 1 ? (int)ctx().opt.gemm_group_m : GROUP_M;
  p.seg_kb = 1;
  set_push_params(p, g);
  p.status = c.d_status;
  auto kern = gemm_tc2_streamk_kernel<EPI>;
  static int max_pairs = 0;  // one per template instantiation
  if (max_pairs == 0) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemSk));
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2 * (c.sm_count / 2));
    q.blockDim = dim3(THREADS2);
    q.dynamicSmemBytes = kSmemSk;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &q) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = c.sm_count / 2 - 4;
    }
    max_pairs = clusters < c.sm_count / 2 ? clusters : c.sm_count / 2;
  }
  const long long units = (long long)p.num_tiles * p.k_blocks;
  const int pairs = (int)(units < max_pairs ? units : max_pairs);
  sp.units_q = (int)(units / pairs);
  sp.units_r = (int)(units % pairs);
  void *ws = nullptr;
  B200_TRY(splitk_workspace(SK_COUNTER_BYTES + (size_t)max_pairs * 2 * SK_SLOT_FLOATS * sizeof(float), &ws));
  sp.counters = (int *)ws;
  sp.partials = (float *)((char *)ws + SK_COUNTER_BYTES);
  B200_CUDA(launch_maybe_dependent(c.opt.gemm_dependent_launch != 0, kern, dim3((unsigned)(2 * pairs)), dim3(THREADS2),
                                   (size_t)kSmemSk, c.stream, tmA, tmB, tmB2, sp));
  return check_launch("tc256x256x64_2cta_streamk");
}

}  // namespace

// What the variant needs beyond the pair kernel's own legality: its counters cover 8192 tiles and
// the unit index must fit an int.
bool streamk_shape_ok(const GemmArgs &g) {
  const int bn_out = g.epilogue == EPI_SWIGLU ? 128 : 256;
  const long long tiles = ((g.m + 255) / 256) * ((g.n + bn_out - 1) / bn_out);
  const long long kb = (g.k + BK2 - 1) / BK2;
  return tiles <= SK_MAX_TILES && tiles * kb < 0x7fffffffLL;
}

int launch_gemm_tc_streamk(const GemmArgs &g) {
  switch (g.epilogue) {
    case EPI_F16: return launch_streamk<EPI_F16>(g);
    case EPI_F32_RES: return launch_streamk<EPI_F32_RES>(g);
    case EPI_F16_RES16: return launch_streamk<EPI_F16_RES16>(g);
    case EPI_PUSH16: return launch_streamk<EPI_PUSH16>(g);
    case EPI_SWIGLU: return launch_streamk<EPI_SWIGLU>(g);
    default: return set_error(B200MLIR_ERR_UNSUPPORTED, "stream-K gemm: epilogue %d not built", g.epilogue);
  }
}

}  // namespace b200
