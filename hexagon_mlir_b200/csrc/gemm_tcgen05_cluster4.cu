// fp16 GEMM for SMALL problems: a cluster of four CTAs per 256 x 128 output tile — two SM pairs,
// each issuing tcgen05.mma.cta_group::2 over ONE HALF of K, the halves added through distributed
// shared memory.
//
// Why: a problem like 1024^3 has too few large tiles to fill the machine, and with small tiles it
// is bound by what one SM can pull in — a 128 x 64 tile fetches 24 KiB per 64-deep k-block, 384 KiB
// per CTA over K = 1024, and an SM sustained ~38 B/clock on cold operands.  Here a CTA fetches its
// 128 rows of A and its 64 columns of B (24 KiB per k-block, like before) for a 256 x 128 tile —
// four times the flops per byte — and only for half of K: 192 KiB per CTA at K = 1024, on the same
// 128 SMs.  The price is the exchange of one fp32 partial tile per cluster, which never leaves the
// SMs: the pair that owns the upper half of K stores its accumulators straight into the shared
// memory of the pair that owns the lower half (st.shared::cluster), which adds them to its own
// before the fused read-out.  The order of the sum is fixed (lower half + upper half), so results
// are bit-reproducible.  Reference analogue: K segments accumulated in fp32 after the engine's
// read-out (hmx/src/HMXLayout.c:880-901).
//
// One tile per cluster, no tile loop (the variant is for problems of at most a wave or two of
// clusters).  Roles per CTA (192 threads) as in the pair kernel: warp 0 lane 0 TMA producer, warp 1
// TMEM owner and — in each pair's leader — MMA issuer, warps 2-5 read-out.  Cluster ranks: pair =
// rank >> 1 (K half), side = rank & 1 (rows m0 + 128*side, columns n0 + 64*side of B's tile).
#include <cstdlib>
#include <cstring>

#include "common.h"
#include "gemm_tc2_common.cuh"

namespace b200 {
namespace {

using namespace ptx;

constexpr int C4_STAGES = 5;
constexpr int C4_BN = 128;                             // tile columns (64 per CTA of a pair)
constexpr int C4_STAGE_BYTES = A2_BYTES + SLAB_BYTES;  // 16 KiB of A + 8 KiB of B
constexpr int C4_RECV_BYTES = 128 * C4_BN * 4;         // the other pair's partial of this CTA's 128 rows: 64 KiB
constexpr int C4_TMEM_COLS = 128;
constexpr long long C4_WAIT_LIMIT = 2000000000LL;

__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
__device__ __forceinline__ void fence_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
// commit to the barrier at this offset in both CTAs of THIS pair (cluster ranks base, base + 1)
__device__ __forceinline__ void mma_commit_pair_of(uint32_t bar, uint32_t pair_base_rank) {
  const uint16_t mask = (uint16_t)(3u << pair_base_rank);
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(4, 1, 1) __launch_bounds__(THREADS2, 1)
gemm_c4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcParams p) {
  constexpr uint32_t IDESC = make_idesc(/*D=f32*/ 1, /*A=f16*/ 0, /*B=f16*/ 0, /*A K-major*/ 0, /*B MN-major*/ 1, 256, C4_BN);
  constexpr int STAGES = C4_STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t recv = smem_base + STAGES * C4_STAGE_BYTES;  // [column][row] fp32, written by the other pair
  const uint32_t ctrl = recv + C4_RECV_BYTES;
  const uint32_t bar_full = ctrl;                  // STAGES (used in the pair's leader)
  const uint32_t bar_empty = ctrl + 8 * STAGES;    // STAGES (both CTAs of the pair)
  const uint32_t bar_tfull = ctrl + 16 * STAGES;   // accumulator complete (both CTAs of the pair)
  const uint32_t bar_recv = bar_tfull + 8;         // the other pair's partial has landed (lower-half pair only)
  const uint32_t tmem_slot = bar_tfull + 16;
  uint8_t *gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(gen + (tmem_slot - smem_base));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + (tmem_slot - smem_base) + 4);
  const float *recv_gen = reinterpret_cast<const float *>(gen + (recv - smem_base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const uint32_t pair = rank >> 1, side = rank & 1u, pair_base = rank & ~1u;
  const bool leader = side == 0;
  const int tile = blockIdx.x >> 2;
  const int m_blk = tile % p.m_blocks, n_blk = tile / p.m_blocks;
  const int m0 = m_blk * 256 + (int)side * BM2, n0 = n_blk * C4_BN;
  // this pair's half of the k-blocks (the lower half takes the odd one)
  const int kb_half = (p.k_blocks + 1) >> 1;
  const int kb0 = pair == 0 ? 0 : kb_half, kb1 = pair == 0 ? kb_half : p.k_blocks;
  pdl_trigger();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 2);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_recv, 4);  // the four read-out warps of the sending CTA
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc_pair(tmem_slot, C4_TMEM_COLS);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();  // every CTA's barriers exist before anything is signalled on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's 128 rows of A and 64 columns of B ----------------
    if (lane == 0) {
      pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, 51, tile)) break;
        const uint32_t full = map_to_cta(bar_full + 8 * stage, pair_base);  // the pair leader's barrier
        remote_expect_tx(full, C4_STAGE_BYTES);
        const uint32_t sa = smem_base + stage * C4_STAGE_BYTES;
        tma_load_2d_pair(sa, &tmA, full, kb * BK2, m0);
        tma_load_2d_pair(sa + A2_BYTES, &tmB, full, n0 + (int)side * 64, kb * BK2);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (each pair's leader) ----------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, 53, tile)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = smem_base + stage * C4_STAGE_BYTES;
        const uint64_t adesc = smem_desc_sw128(sa, 16, 1024);
        const uint64_t bdesc = smem_desc_sw128(sa + A2_BYTES, SLAB_BYTES, 1024);
#pragma unroll
        for (int k = 0; k < BK2 / 16; ++k)
          mma_f16_pair(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 128), IDESC, (kb != kb0 || k != 0) ? 1u : 0u);
        mma_commit_pair_of(bar_empty + 8 * stage, pair_base);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) mma_commit_pair_of(bar_tfull, pair_base);
    }
  } else {
    // ---------------- read-out (warps 2..5): this CTA's 128 rows x 128 columns ----------------
    const int q = warp & 3;
    bool ok = mbar_wait(bar_tfull, 0, abort_flag, p.status, 54, tile);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
      const int row_in_cta = q * 32 + lane;
      if (pair == 1) {
        // upper half of K: hand the partial to the same rows' CTA of the lower-half pair
        const uint32_t dst = map_to_cta(recv, rank - 2u);
#pragma unroll 1
        for (int c = 0; c < C4_BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            st_cluster_f32(dst + (uint32_t)(((c * 32 + j) * 128 + row_in_cta) * 4), __uint_as_float(r[j]));
        }
        fence_cluster();  // the stores are performed before the arrival is observed
        __syncwarp();
        if (lane == 0) remote_arrive(map_to_cta(bar_recv, rank - 2u));
      } else {
        // lower half of K: wait for the other pair's partial, add (own + theirs), read out
        bool got = mbar_wait(bar_recv, 0, abort_flag, p.status, 55, tile, C4_WAIT_LIMIT);
        got = __all_sync(0xffffffffu, got);
        if (got) {
          fence_cluster();
          const int row = m0 + row_in_cta;
          const bool row_ok = row < p.m;
#pragma unroll 1
          for (int c = 0; c < C4_BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              r[j] = __float_as_uint(__uint_as_float(r[j]) + recv_gen[(c * 32 + j) * 128 + row_in_cta]);
            const int col0 = n0 + c * 32;
            if (!row_ok || col0 >= p.n) continue;
            epilogue_store_chunk<EPI>(r, r, row, col0, p);
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1 && *abort_flag)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  cluster_sync();  // nobody leaves while a peer may still write its shared memory or signal its barriers
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, C4_TMEM_COLS);
  }
}

constexpr int kSmemC4 = C4_STAGES * C4_STAGE_BYTES + C4_RECV_BYTES + 16 * C4_STAGES + 64 + 1024;

template <int EPI>
int launch_c4(const GemmArgs &g) {
  Context &c = ctx();
  CUtensorMap tmA, tmB;
  B200_TRY(make_map_2d(&tmA, g.a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.k, g.m, g.lda, BK2, BM2));
  B200_TRY(make_map_2d(&tmB, g.b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.n, g.k, g.ldb, 64, BK2));
  TcParams p;
  p.c = g.c;
  p.res = g.res;
  p.ldc = g.ldc;
  p.ldres = g.ldres;
  p.m = (int)g.m;
  p.n = (int)g.n;
  p.k = (int)g.k;
  p.m_blocks = (int)((g.m + 255) / 256);
  p.n_blocks = (int)((g.n + C4_BN - 1) / C4_BN);
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.k_blocks = (int)((g.k + BK2 - 1) / BK2);
  p.group_m = GROUP_M;
  p.seg_kb = 1;
  set_push_params(p, g);
  p.status = c.d_status;
  auto kern = gemm_c4_kernel<EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemC4));
    attr_set = true;
  }
  B200_CUDA(launch_maybe_dependent(c.opt.gemm_dependent_launch != 0, kern, dim3((unsigned)(4 * p.num_tiles)), dim3(THREADS2),
                                   (size_t)kSmemC4, c.stream, tmA, tmB, p));
  return check_launch("tc256x128x64_cluster4_splitk2");
}

}  // namespace

int cluster4_variant_smem_bytes() { return kSmemC4; }

// K must give both pairs at least one k-block; the grid is one cluster per tile
bool cluster4_shape_ok(const GemmArgs &g) {
  const long long tiles = ((g.m + 255) / 256) * ((g.n + C4_BN - 1) / C4_BN);
  return g.k > BK2 && tiles <= 16384;
}

int launch_gemm_tc_cluster4(const GemmArgs &g) {
  switch (g.epilogue) {
    case EPI_F16: return launch_c4<EPI_F16>(g);
    case EPI_F32_RES: return launch_c4<EPI_F32_RES>(g);
    case EPI_F16_RES16: return launch_c4<EPI_F16_RES16>(g);
    default: return set_error(B200MLIR_ERR_UNSUPPORTED, "cluster split-K gemm: epilogue %d not built", g.epilogue);
  }
}

}  // namespace b200
