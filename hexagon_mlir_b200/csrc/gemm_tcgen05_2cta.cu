// fp16 GEMM, 2-CTA form: a pair of CTAs on two SMs (a cluster of 2) works on one
// 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// Why: with one CTA per 128 x 256 tile every K=64 step pulls 48 KiB through the
// L2 -> SM path and reads 12 KiB of shared memory per MMA; pairing two SMs halves
// the B traffic of each — CTA r loads its own 128 rows of A and only its half
// (128 columns) of B, and the tensor cores of both SMs read both halves.  No
// TMA multicast is used anywhere: every CTA issues plain tiled loads (with the
// cta_group::2 form, whose only effect is that the completion may be signalled
// on the leader CTA's mbarrier).
//
// Roles per CTA (192 threads): warp 0 lane 0 = TMA producer for this CTA's
// operands; warp 1 = TMEM owner, and in the leader CTA (cluster rank 0) lane 0
// issues the MMAs for the pair; warps 2-5 = epilogue of this CTA's 128 rows.
// Barriers: full[s] lives in the leader and counts both producers; empty[s] and
// tmem_full[a] are signalled in both CTAs by a multicast tcgen05.commit;
// tmem_empty[a] lives in the leader and counts the epilogue warps of both CTAs.
#include <cstdlib>
#include <cstring>

#include "common.h"
#include "gemm_tc2_common.cuh"

namespace b200 {
namespace {

using namespace ptx;

#ifdef G2_TRACE
__device__ long long g2_trace_buf[2 * 6 * 64];
#define TR2(role, i) do { if (pair == 1 && (i) < 64) trace_s[(role) * 64 + (i)] = clock64(); } while (0)
#else
#define TR2(role, i) do { } while (0)
#endif

// EPI_SWIGLU: the pair's MMA N = 256 is [gate 128 | up 128]; CTA 0 loads the Wg tile,
// CTA 1 the Wu tile, and each CTA's accumulator rows hold both halves.
// NSUB: 64-deep K sub-tiles per stage (one barrier round trip and one commit per stage).
// K-looped form (EPI_KLOOP_F16): one accumulator stage per K segment of p.seg_kb stages, started
// with accumulate off; eight read-out warps per CTA (two per TMEM lane quadrant, 128 columns each)
// round every segment to fp16 and keep the row's fp32 running sums in registers
// (test/python/triton/test_matmul_kloop.py:87-98).
constexpr int pair_threads(int epi) { return epi == EPI_KLOOP_F16 ? 320 : THREADS2; }
// BKB: B is the K-blocked image [k/64][N][64] (GemmArgs::b_kblocked): a K-major operand whose tile
// of one k-block is contiguous in HBM; loaded and described like the int8 form's transposed B.
template <int STAGES, int NSUB, int EPI, bool BKB = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair_threads(EPI), 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmB2, const TcParams p) {
  constexpr int BN_MMA = 256;
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? 128 : 256;
  constexpr int TMEM_COLS = 512;  // two accumulator stages of 256 columns
  // int8 form (EPI_I32): both operands K-major (B arrives transposed, this CTA loads its 128 rows
  // of it), 128 int8 per swizzle row and K = 32 per instruction: the fp16 form's bytes per stage
  constexpr bool I8 = EPI == EPI_I32;
  constexpr bool BKM = I8 || BKB;  // B arrives K-major
  constexpr uint32_t IDESC = I8 ? make_idesc(/*D=s32*/ 2, /*A=s8*/ 1, /*B=s8*/ 1, 0, /*B K-major*/ 0, 256, BN_MMA)
                                : make_idesc(/*D=f32*/ 1, /*A=f16*/ 0, /*B=f16*/ 0, /*A K-major*/ 0,
                                             /*B MN-major unless K-blocked*/ BKB ? 0 : 1, 256, BN_MMA);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int STAGE_BYTES = NSUB * STAGE2_BYTES;
  constexpr int BKS = NSUB * BK2;  // K per stage
  const uint32_t ctrl = smem_base + STAGES * STAGE_BYTES;
  const uint32_t bar_full = ctrl;                       // STAGES (used in the leader)
  const uint32_t bar_empty = ctrl + 8 * STAGES;         // STAGES (both CTAs)
  const uint32_t bar_tfull = ctrl + 16 * STAGES;        // 2 (both CTAs)
  const uint32_t bar_tempty = ctrl + 16 * STAGES + 16;  // 2 (used in the leader)
  const uint32_t tmem_slot = ctrl + 16 * STAGES + 32;
  uint8_t *ctrl_gen = smem_raw + (ctrl - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(ctrl_gen + 16 * STAGES + 32);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ctrl_gen + 16 * STAGES + 36);

#ifdef G2_TRACE
  __shared__ long long trace_s[6 * 64];
#endif
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  // A programmatic dependent of the previous kernel in the stream: our own successor may start
  // now; what the predecessor wrote is touched only after the producers' griddepcontrol.wait
  // (every other access of the pair is ordered after it through the mbarriers).
  pdl_trigger();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 2);   // one arrive.expect_tx per CTA of the pair
      mbar_init(bar_empty + 8 * s, 1);  // the multicast commit
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, EPI == EPI_KLOOP_F16 ? 16 : 8);  // the read-out warps of both CTAs
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
  cluster_sync();  // the peer's barriers exist before anything is signalled on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's 128 rows of A and 128 columns of B ----------------
    if (lane == 0) {
      pdl_wait();  // (see the note at the kernel's top)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.num_tiles; tile += num_pairs) {
        int m_blk, n_blk;
        tile_coords(tile, p.m_blocks, p.n_blocks, p.group_m, m_blk, n_blk);
        const int m0 = m_blk * 256 + (int)rank * BM2;
        const int n0 = n_blk * BN_OUT;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, 31, tile)) {
            ok = false;
            break;
          }
          const uint32_t full = map_to_cta(bar_full + 8 * stage, 0);  // the leader's barrier
          remote_expect_tx(full, STAGE_BYTES);
#pragma unroll
          for (int sub = 0; sub < NSUB; ++sub) {
            const uint32_t sa = smem_base + stage * STAGE_BYTES + sub * STAGE2_BYTES;
            const uint32_t sb = sa + A2_BYTES;
            const int k0 = (kb * NSUB + sub) * (I8 ? 128 : BK2);  // in elements
            tma_load_2d_pair(sa, &tmA, full, k0, m0);
            if (I8) {
              tma_load_2d_pair(sb, &tmB, full, k0, n0 + (int)rank * 128);  // 128 rows of Bᵀ x 128 bytes
            } else if (BKB) {
              // rows (k-block, n) of the image: this CTA's 128 columns of the block, 16 KiB contiguous
              tma_load_2d_pair(sb, &tmB, full, 0, (kb * NSUB + sub) * p.n + n0 + (int)rank * 128);
            } else if (EPI == EPI_SWIGLU) {
              const CUtensorMap *mb = leader ? &tmB : &tmB2;  // gate half / up half
              tma_load_2d_pair(sb, mb, full, n0, k0);
              tma_load_2d_pair(sb + SLAB_BYTES, mb, full, n0 + 64, k0);
            } else {
              const int nb = n0 + (int)rank * 128;
              tma_load_2d_pair(sb, &tmB, full, nb, k0);
              tma_load_2d_pair(sb + SLAB_BYTES, &tmB, full, nb + 64, k0);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      int tord = 0;
      if constexpr (EPI == EPI_KLOOP_F16) {
      for (int tile = pair; ok && tile < p.num_tiles; tile += num_pairs, ++tord) {
        TR2(0, tord);
        // (position inside the K segment by counting: a division costs the lone issuing thread ~300 clocks)
        for (int kb = 0, in_seg = 0; kb < p.k_blocks; ++kb) {
          const bool seg_start = EPI == EPI_KLOOP_F16 ? in_seg == 0 : kb == 0;
          if (seg_start) {
            if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, 32, tile)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            TR2(1, tord);
          }
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN_MMA);
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, 33, tile)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < NSUB; ++sub) {
            const uint32_t sa = smem_base + stage * STAGE_BYTES + sub * STAGE2_BYTES;
            const uint32_t sb = sa + A2_BYTES;
            const uint64_t adesc = smem_desc_sw128(sa, 16, 1024);
            const uint64_t bdesc = BKM ? smem_desc_sw128(sb, 16, 1024) : smem_desc_sw128(sb, SLAB_BYTES, 1024);
#pragma unroll
            for (int k = 0; k < BK2 / 16; ++k) {
              const uint32_t accum = (seg_start && sub == 0 && k == 0) ? 0u : 1u;
              if (I8)
                mma_i8_pair(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), IDESC, accum);
              else
                mma_f16_pair(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(BKB ? k * 2 : k * 128), IDESC, accum);
            }
          }
          mma_commit_pair(bar_empty + 8 * stage);  // both producers may refill the stage
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
          if (++in_seg == p.seg_kb) in_seg = 0;
          const bool seg_end = EPI == EPI_KLOOP_F16 ? (in_seg == 0 || kb + 1 == p.k_blocks)
                                                    : kb + 1 == p.k_blocks;
          if (seg_end) {
            mma_commit_pair(bar_tfull + 8 * acc);  // accumulators complete in both CTAs
            if (++acc == 2) {
              acc = 0;
              acc_phase ^= 1u;
            }
          }
        }
        TR2(2, tord);
      }
      } else {
      for (int tile = pair; ok && tile < p.num_tiles; tile += num_pairs, ++tord) {
        TR2(0, tord);
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, 32, tile)) break;
        tc_fence_after_sync();
        TR2(1, tord);
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN_MMA);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, 33, tile)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < NSUB; ++sub) {
            const uint32_t sa = smem_base + stage * STAGE_BYTES + sub * STAGE2_BYTES;
            const uint32_t sb = sa + A2_BYTES;
            const uint64_t adesc = smem_desc_sw128(sa, 16, 1024);
            const uint64_t bdesc = BKM ? smem_desc_sw128(sb, 16, 1024) : smem_desc_sw128(sb, SLAB_BYTES, 1024);
#pragma unroll
            for (int k = 0; k < BK2 / 16; ++k) {
              if (I8)
                mma_i8_pair(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), IDESC,
                            (kb | sub | k) != 0 ? 1u : 0u);
              else
                mma_f16_pair(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(BKB ? k * 2 : k * 128), IDESC,
                             (kb | sub | k) != 0 ? 1u : 0u);
            }
          }
          mma_commit_pair(bar_empty + 8 * stage);  // both producers may refill the stage
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        mma_commit_pair(bar_tfull + 8 * acc);  // accumulators complete in both CTAs
        TR2(2, tord);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5, K-looped form 2..9): this CTA's 128 rows ----------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    int tord = 0;
    for (int tile = pair; tile < p.num_tiles; tile += num_pairs, ++tord) {
      int m_blk, n_blk;
      tile_coords(tile, p.m_blocks, p.n_blocks, p.group_m, m_blk, n_blk);
      const int m0 = m_blk * 256 + (int)rank * BM2, n0 = n_blk * BN_OUT;
      if constexpr (EPI == EPI_KLOOP_F16) {
        // this warp's half of the 256 columns: fp32 running sums of its row, every segment rounded to fp16 first
        const int half = (warp - 2) >> 2;
        const int row = m0 + q * 32 + lane;
        float sum[128];
#pragma unroll
        for (int e = 0; e < 128; ++e) sum[e] = 0.0f;
        const int segs = (p.k_blocks + p.seg_kb - 1) / p.seg_kb;
        bool ok = true;
        for (int sg = 0; sg < segs; ++sg) {
          ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, 34, tile);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN_MMA + half * 128);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e += 2)
              add_rounded2(sum[c * 32 + e], sum[c * 32 + e + 1], __uint_as_float(r[e]), __uint_as_float(r[e + 1]));
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) remote_arrive(map_to_cta(bar_tempty + 8 * acc, 0));  // the leader's barrier
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1u;
          }
        }
        if (!ok) break;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(sum[c * 32 + e]);
          const int col0 = n0 + half * 128 + c * 32;
          if (row < p.m && col0 < p.n) epilogue_store_chunk<EPI_F16>(r, r, row, col0, p);
        }
        continue;
      }
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.m;
      ResChunk rc, rc_next;
      residual_prefetch<EPI>(rc, row, n0, row_ok, p);  // under the tile's main loop
      bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, 34, tile);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if (threadIdx.x == 64) TR2(3, tord);
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN_MMA);
#pragma unroll 1
      for (int c = 0; c < BN_OUT / 32; ++c) {
        if (c + 1 < BN_OUT / 32) residual_prefetch<EPI>(rc_next, row, n0 + (c + 1) * 32, row_ok, p);
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        uint32_t r2[32];
        if (EPI == EPI_SWIGLU) tmem_ld_32x32(t_row + BN_OUT + c * 32, r2);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row_ok && col0 < p.n) epilogue_store_chunk<EPI>(r, r2, row, col0, p, rc);
        if (EPI == EPI_F16_RES16 || EPI == EPI_F32_RES) rc = rc_next;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (threadIdx.x == 64) TR2(4, tord);
      if (lane == 0) remote_arrive(map_to_cta(bar_tempty + 8 * acc, 0));  // the leader's barrier
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  // Neither CTA may leave (or free TMEM) while the other can still signal its
  // barriers or have MMAs of the pair in flight.
  if (warp == 1 && *abort_flag)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  cluster_sync();
#ifdef G2_TRACE
  if (pair == 1) for (int i = threadIdx.x; i < 6 * 64; i += blockDim.x) g2_trace_buf[rank * 6 * 64 + i] = trace_s[i];
#endif
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

constexpr int kSmem2 = 6 * STAGE2_BYTES + 16 * 6 + 64 + 1024;  // the same ring bytes for (6 x 64) and (3 x 128)

template <int STAGES, int NSUB, int EPI, bool BKB = false>
int launch_pair(const GemmArgs &g, const char *name) {
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? 128 : 256;
  Context &c = ctx();
  CUtensorMap tmA, tmB, tmB2;
  B200_TRY(make_map_2d(&tmA, g.a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.k, g.m, g.lda, BK2, BM2));
  if (BKB)  // the image as rows of 64 fp16: [ceil(K/64) * N][64], boxes of 128 rows
    B200_TRY(make_map_2d(&tmB, g.b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, 64, ((g.k + 63) / 64) * g.n, 64, 64, 128));
  else
    B200_TRY(make_map_2d(&tmB, g.b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.n, g.k, g.ldb, 64, BK2));
  if (EPI == EPI_SWIGLU)
    B200_TRY(make_map_2d(&tmB2, g.b2, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.n, g.k, g.ldb, 64, BK2));
  else
    tmB2 = tmB;
  TcParams p;
  p.c = g.c;
  p.res = g.res;
  p.ldc = g.ldc;
  p.ldres = g.ldres;
  p.res_mod = g.res_mod;
  p.res_rem = g.res_rem;
  p.m = (int)g.m;
  p.n = (int)g.n;
  p.k = (int)g.k;
  p.m_blocks = (int)((g.m + 255) / 256);
  p.n_blocks = (int)((g.n + BN_OUT - 1) / BN_OUT);
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.k_blocks = (int)((g.k + NSUB * BK2 - 1) / (NSUB * BK2));
  p.group_m = ctx().opt.gemm_group_m >= 1 ? (int)ctx().opt.gemm_group_m : GROUP_M;
  p.seg_kb = (EPI == EPI_KLOOP_F16 && g.block_k >= NSUB * BK2) ? g.block_k / (NSUB * BK2) : 1;
  set_push_params(p, g);
  p.status = c.d_status;
  auto kern = gemm_tc2_kernel<STAGES, NSUB, EPI, BKB>;
  static int max_pairs = 0;  // one per template instantiation
  if (max_pairs == 0) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2));
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2 * (c.sm_count / 2));
    q.blockDim = dim3(pair_threads(EPI));
    q.dynamicSmemBytes = kSmem2;
    int clusters = 0;
    // SMs pair up inside a GPC only: ask how many pairs can be resident at once
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &q) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = c.sm_count / 2 - 4;
    }
    max_pairs = clusters < c.sm_count / 2 ? clusters : c.sm_count / 2;
    if (getenv("B200MLIR_DEBUG")) fprintf(stderr, "[b200mlir] 2-CTA gemm: %d resident pairs (occupancy query %d)\n", max_pairs, clusters);
  }
  int pairs = p.num_tiles < max_pairs ? p.num_tiles : max_pairs;
  B200_CUDA(launch_maybe_dependent(c.opt.gemm_dependent_launch != 0, kern, dim3((unsigned)(2 * pairs)), dim3(pair_threads(EPI)),
                                   (size_t)kSmem2, c.stream, tmA, tmB, tmB2, p));
  return check_launch(name);
}

}  // namespace

int pair_variant_smem_bytes() { return kSmem2; }

#ifdef G2_TRACE
extern "C" __attribute__((visibility("default"))) int b200mlir_debug_get_trace2(long long *host) {
  return (int)cudaMemcpyFromSymbol(host, g2_trace_buf, sizeof(long long) * 2 * 6 * 64);
}
#endif

template <int STAGES, int NSUB>
int launch_pair_epi(const GemmArgs &g, const char *name) {
  if (g.b_kblocked) {
    if constexpr (NSUB == 1) {
      if (g.epilogue == EPI_F16) return launch_pair<STAGES, NSUB, EPI_F16, true>(g, name);
    }
    return set_error(B200MLIR_ERR_UNSUPPORTED, "a K-blocked B is built for the plain fp16 read-out and 64-deep stages");
  }
  switch (g.epilogue) {
    case EPI_F16: return launch_pair<STAGES, NSUB, EPI_F16>(g, name);
    case EPI_F32_RES: return launch_pair<STAGES, NSUB, EPI_F32_RES>(g, name);
    case EPI_F16_RES16: return launch_pair<STAGES, NSUB, EPI_F16_RES16>(g, name);
    case EPI_PUSH16: return launch_pair<STAGES, NSUB, EPI_PUSH16>(g, name);
    case EPI_SWIGLU: return launch_pair<STAGES, NSUB, EPI_SWIGLU>(g, name);
    case EPI_KLOOP_F16:
      if constexpr (NSUB == 1) return launch_pair<STAGES, NSUB, EPI_KLOOP_F16>(g, name);
      return set_error(B200MLIR_ERR_UNSUPPORTED, "k-looped read-out is built for 64-deep stages");
    default: return set_error(B200MLIR_ERR_UNSUPPORTED, "2-CTA gemm: epilogue %d not built", g.epilogue);
  }
}

// int8 x int8 -> int32 over SM pairs; bt is B transposed, [N,K] row-major
int launch_gemm_i8_tc_pair(const int8_t *a, const int8_t *bt, int32_t *c, int64_t m, int64_t n, int64_t k, int64_t lda,
                           int64_t ldbt, int64_t ldc) {
  B200_TRY(ensure_ready());
  constexpr int STAGES = 6, NSUB = 1;
  Context &cx = ctx();
  CUtensorMap tmA, tmB;
  B200_TRY(make_map_2d(&tmA, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k, m, lda, 128, BM2));
  B200_TRY(make_map_2d(&tmB, bt, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k, n, ldbt, 128, 128));
  TcParams p;
  p.c = c;
  p.res = nullptr;
  p.ldc = ldc;
  p.ldres = 0;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.m_blocks = (int)((m + 255) / 256);
  p.n_blocks = (int)((n + 255) / 256);
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.k_blocks = (int)((k + 127) / 128);
  p.group_m = GROUP_M;
  p.seg_kb = 1;
  GemmArgs none;
  set_push_params(p, none);
  p.status = cx.d_status;
  auto kern = gemm_tc2_kernel<STAGES, NSUB, EPI_I32>;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2));
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2 * (cx.sm_count / 2));
    q.blockDim = dim3(THREADS2);
    q.dynamicSmemBytes = kSmem2;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &q) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = cx.sm_count / 2 - 4;
    }
    max_pairs = clusters < cx.sm_count / 2 ? clusters : cx.sm_count / 2;
  }
  const int pairs = p.num_tiles < max_pairs ? p.num_tiles : max_pairs;
  B200_CUDA(launch_maybe_dependent(false, kern, dim3((unsigned)(2 * pairs)), dim3(THREADS2), (size_t)kSmem2, cx.stream,
                                   tmA, tmB, tmB, p));
  return check_launch("gemm_tc2_i8_256x256");
}

// deep_k: 128-deep stages (three of them) instead of six 64-deep ones
int launch_gemm_tc_pair(const GemmArgs &g, bool deep_k) {
  return deep_k ? launch_pair_epi<3, 2>(g, "tc256x256x128_2cta") : launch_pair_epi<6, 1>(g, "tc256x256x64_2cta");
}

}  // namespace b200
