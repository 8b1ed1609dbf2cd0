// fp16 GEMM over SM pairs for grids that do not fill the machine evenly: the 256 x 256 pair
// kernel with the K dimension of its LAST tiles dealt out in k-blocks ("stream-K").
//
// Why: with whole tiles per pair, T tiles on P pairs take ceil(T / P) rounds — 43 tiles leave 31
// of 74 pairs idle, 86 tiles cost two rounds for 1.16 rounds of work.  Here whole rounds of P tiles
// are handed out exactly as the pair kernel does (pairs that run together work on neighbouring
// tiles, which is what keeps their operand panels in L2); the tiles of the last, part-filled round
// (plus one full round's when the remainder is below P/2; all tiles when T < P) are cut into
// 64-deep k-blocks, and those units are dealt out in P contiguous, equal ranges.  A pair's range
// is then the tail of one tile, possibly a whole tile, and the head of another.
//
// A tile cut between pairs needs its partial sums combined.  The reference combines K segments in
// fp32 after the engine's read-out (hmx/src/HMXLayout.c:880-901; the span count of a tiling,
// backend/hmx_search.py:221-232).  Here the pair that holds a tile's FIRST k-blocks combines: every
// other contributor reaches its piece as the first thing in its range, stores the fp32 partial
// (as it lies in TMEM: column-major per 32-row slab, so the stores coalesce) into its slot of a
// resident workspace and bumps the slab's arrival counter; the combining pair reaches the tile as
// the last thing in its range, waits (bounded, with the library's status word) until the others
// have arrived — they did long ago — and adds their partials to its own accumulators in
// contributor order before the fused read-out.  The order of the sum is fixed by the partition,
// not by arrival, so results are bit-reproducible run to run.  Nothing a contributor does before
// it arrives depends on another pair, so the wait cannot deadlock while all pairs are resident
// (the grid never exceeds the number of resident pairs).  Counters return to zero in the kernel.
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
constexpr int SK_MAX_TILES = 8192;                                   // arrival counters: 8 per tile
constexpr size_t SK_COUNTER_BYTES = (size_t)SK_MAX_TILES * 8 * sizeof(int);
constexpr size_t SK_SLAB_FLOATS = 32 * 256;                          // one warp's 32 rows x 256 accumulator columns
constexpr size_t SK_CTA_FLOATS = 4 * SK_SLAB_FLOATS;                 // 128 rows
constexpr size_t SK_SLOT_FLOATS = 2 * SK_CTA_FLOATS;                 // both CTAs of a pair: 256 KiB of fp32
constexpr long long SK_ARRIVAL_LIMIT = 2000000000LL;                 // clocks the combining pair waits at most (~1 s)
constexpr int SK_FAST_OTHERS = 3;                                    // contributors (beside the combining pair) the bulk-copy path holds
constexpr uint32_t SK_STEP_BYTES = 16384;                            // one contributor's share of one combine step: 128 columns x 32 lanes fp32

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void bulk_load_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

struct SkParams {
  TcParams t;
  int dp_tiles;           // tiles [0, dp_tiles) are handed out whole, round by round (a multiple of the pair count)
  int units_q, units_r;   // the k-blocks of the other tiles: pair p owns units [p*q + min(p, r), (p+1)*q + min(p+1, r))
  int *counters;          // [tile][cta rank][lane quadrant]
  float *partials;        // [pair][cta rank][quadrant][column][lane]: the partial of the one cut tile a pair does not combine itself
};

__device__ __forceinline__ int sk_unit_begin(int p, int q, int r) { return p * q + min(p, r); }
__device__ __forceinline__ int sk_pair_of_unit(int u, int q, int r) {
  const int wide = (q + 1) * r;  // the first r pairs own q + 1 units each
  return u < wide ? u / (q + 1) : r + (u - wide) / q;
}

// The pieces of work of one pair, in order: whole tiles pair, pair + P, ... below dp_tiles, then
// its range of k-blocks of the remaining tiles.  Every role of the CTA walks the same sequence.
struct SkWalk {
  int dp_tile, dp_tiles, stride, KB, u, u_end;
  __device__ SkWalk(const SkParams &sp, int pair, int num_pairs)
      : dp_tile(pair), dp_tiles(sp.dp_tiles), stride(num_pairs), KB(sp.t.k_blocks),
        u(sk_unit_begin(pair, sp.units_q, sp.units_r)), u_end(sk_unit_begin(pair + 1, sp.units_q, sp.units_r)) {}
  __device__ bool next(int &tile, int &kb0, int &kb1) {
    if (dp_tile < dp_tiles) {
      tile = dp_tile;
      kb0 = 0;
      kb1 = KB;
      dp_tile += stride;
      return true;
    }
    if (u >= u_end) return false;
    const int t = u / KB;  // (a division costs a lone thread ~300 clocks: once per piece, not per k-block)
    kb0 = u - t * KB;
    kb1 = min(KB, kb0 + (u_end - u));
    u += kb1 - kb0;
    tile = dp_tiles + t;
    return true;
  }
};

template <int EPI, bool BKB = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS2, 1)
gemm_tc2_streamk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmB2, const SkParams sp) {
  const TcParams &p = sp.t;
  constexpr int BN_MMA = 256;
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? 128 : 256;
  constexpr int TMEM_COLS = 512;
  // (BKB: B is the K-blocked image, a K-major operand; see the pair kernel)
  constexpr uint32_t IDESC = make_idesc(/*D=f32*/ 1, /*A=f16*/ 0, /*B=f16*/ 0, /*A K-major*/ 0, /*B MN-major*/ BKB ? 0 : 1,
                                        256, BN_MMA);
  constexpr int STAGES = SK_STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ctrl = smem_base + STAGES * STAGE2_BYTES;
  const uint32_t bar_full = ctrl;
  const uint32_t bar_empty = ctrl + 8 * STAGES;
  const uint32_t bar_tfull = ctrl + 16 * STAGES;
  const uint32_t bar_tempty = ctrl + 16 * STAGES + 16;
  const uint32_t tmem_slot = ctrl + 16 * STAGES + 32;
  const uint32_t bar_fix = ctrl + 16 * STAGES + 64;  // 4: one per read-out warp, for the copies of the combine step
  uint8_t *ctrl_gen = smem_raw + (ctrl - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(ctrl_gen + 16 * STAGES + 32);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ctrl_gen + 16 * STAGES + 36);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int KB = p.k_blocks;
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
    for (int s = 0; s < 4; ++s) mbar_init(bar_fix + 8 * s, 1);
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
      SkWalk walk(sp, pair, num_pairs);
      int tile, kb0, kb1;
      while (ok && walk.next(tile, kb0, kb1)) {
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
          if (BKB) {
            tma_load_2d_pair(sb, &tmB, full, 0, kb * p.n + n0 + (int)rank * 128);
          } else if (EPI == EPI_SWIGLU) {
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
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only): one accumulator stage per piece ----------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      SkWalk walk(sp, pair, num_pairs);
      int tile, kb0, kb1;
      while (ok && walk.next(tile, kb0, kb1)) {
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
          const uint64_t bdesc = BKB ? smem_desc_sw128(sb, 16, 1024) : smem_desc_sw128(sb, SLAB_BYTES, 1024);
#pragma unroll
          for (int k = 0; k < BK2 / 16; ++k)
            mma_f16_pair(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(BKB ? k * 2 : k * 128), IDESC,
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
      }
    }
  } else {
    // ---------------- read-out (warps 2..5): this CTA's 128 rows ----------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    SkWalk walk(sp, pair, num_pairs);
    int tile, kb0, kb1;
    while (walk.next(tile, kb0, kb1)) {
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
      const size_t slab = (size_t)rank * SK_CTA_FLOATS + (size_t)q * SK_SLAB_FLOATS;
      int *counter = sp.counters + ((size_t)tile * 2 + rank) * 4 + q;
      if (kb0 > 0) {
        // ---- a later piece of a cut tile: hand the partial to the pair that combines ----
        // all 256 accumulator columns of the slab as they lie in TMEM: element (column j, lane l)
        // at j*32 + l, so the 32 lanes of one store are contiguous
        float *mine = sp.partials + (size_t)pair * SK_SLOT_FLOATS + slab;
#pragma unroll 1
        for (int c = 0; c < BN_MMA / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) __stcg(mine + (c * 32 + j) * 32 + lane, __uint_as_float(r[j]));
        }
        // the partial is visible device-wide, to plain loads and to bulk copies alike, before the arrival is
        fence_proxy_async_all();
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(counter, 1);
      } else {
        // ---- a whole tile, or the first piece of a cut one: read out, adding the others' partials ----
        int others = 0, p_first = pair;
        if (kb1 < KB) {
          const int t_first = (tile - sp.dp_tiles) * KB;
          p_first = sk_pair_of_unit(t_first, sp.units_q, sp.units_r);  // == pair
          others = sk_pair_of_unit(t_first + KB - 1, sp.units_q, sp.units_r) - p_first;
          // the other contributors reached this tile first thing in their ranges; wait for their arrival
          int seen = 0;
          if (lane == 0) {
            const long long t0 = clock64();
            volatile int *vc = counter;
            while ((seen = *vc) != others) {
              if (*abort_flag) break;
              if (clock64() - t0 > SK_ARRIVAL_LIMIT) {
                *abort_flag = 1;
                if (atomicCAS(p.status, 0, 45) == 0) p.status[1] = tile;
                break;
              }
              __nanosleep(64);
            }
            if (seen == others) *vc = 0;  // clean for the next launch; every contributor has arrived
          }
          seen = __shfl_sync(0xffffffffu, seen, 0);
          if (seen != others) break;
          __threadfence();
        }
        if (others >= 1 && others <= SK_FAST_OTHERS) {
          // The others' partials come in through bulk copies (tens of KB in flight per warp; plain
          // loads keep 4 KB in flight and the combine step, which nothing overlaps, would be bound
          // by L2 latency).  The operand ring is idle by now — a cut tile's first piece is the last
          // thing in a pair's range and its MMAs have completed — so each read-out warp borrows
          // 48 KiB of it: per step, 16 KiB (128 accumulator columns of its slab; for the SwiGLU
          // form 64 gate and the matching 64 up columns) from each contributor.
          const uint32_t fx = smem_base + (uint32_t)q * (SK_FAST_OTHERS * SK_STEP_BYTES);
          const uint32_t fbar = bar_fix + 8 * q;
          const float *fx_gen = reinterpret_cast<const float *>(smem_raw + (fx - smem_u32(smem_raw)));
          fence_proxy_async_all();
          bool fine = true;
#pragma unroll 1
          for (int step = 0; step < 2 && fine; ++step) {
            if (lane == 0) {
              mbar_expect_tx(fbar, (uint32_t)others * SK_STEP_BYTES);
              for (int ci = 1; ci <= others; ++ci) {
                const float *src = sp.partials + (size_t)(p_first + ci) * SK_SLOT_FLOATS + slab;
                const uint32_t dst = fx + (uint32_t)(ci - 1) * SK_STEP_BYTES;
                if (EPI == EPI_SWIGLU) {
                  bulk_load_g2s(dst, src + (size_t)step * 64 * 32, SK_STEP_BYTES / 2, fbar);
                  bulk_load_g2s(dst + SK_STEP_BYTES / 2, src + (size_t)(BN_OUT + step * 64) * 32, SK_STEP_BYTES / 2, fbar);
                } else {
                  bulk_load_g2s(dst, src + (size_t)step * 128 * 32, SK_STEP_BYTES, fbar);
                }
              }
            }
            fine = mbar_wait(fbar, (uint32_t)step & 1u, abort_flag, p.status, 46, tile);
            fine = __all_sync(0xffffffffu, fine);
            if (!fine) break;
            constexpr int CH = (EPI == EPI_SWIGLU) ? 2 : 4;  // output chunks per step
#pragma unroll 1
            for (int cc = 0; cc < CH; ++cc) {
              const int c = step * CH + cc;
              ResChunk rc;
              residual_prefetch<EPI>(rc, row, n0 + c * 32, row_ok, p);  // lands under the loads and sums below
              uint32_t r[32];
              tmem_ld_32x32(t_row + c * 32, r);
              uint32_t r2[32];
              if (EPI == EPI_SWIGLU) tmem_ld_32x32(t_row + BN_OUT + c * 32, r2);
              tmem_ld_wait();
              // own accumulators first, then the contributors in the order of their k ranges
              for (int ci = 1; ci <= others; ++ci) {
                const float *buf = fx_gen + (size_t)(ci - 1) * (SK_STEP_BYTES / 4);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  r[j] = __float_as_uint(__uint_as_float(r[j]) + buf[(cc * 32 + j) * 32 + lane]);
                if (EPI == EPI_SWIGLU) {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    r2[j] = __float_as_uint(__uint_as_float(r2[j]) + buf[(64 + cc * 32 + j) * 32 + lane]);
                }
              }
              const int col0 = n0 + c * 32;
              if (!row_ok || col0 >= p.n) continue;
              epilogue_store_chunk<EPI>(r, r2, row, col0, p, rc);
            }
            __syncwarp();
            fence_proxy_async_all();  // the buffers were read; the next step's copies may overwrite them
          }
          if (!fine) break;
        } else {
#pragma unroll 1
        for (int c = 0; c < BN_OUT / 32; ++c) {
          ResChunk rc;
          residual_prefetch<EPI>(rc, row, n0 + c * 32, row_ok, p);  // lands under the loads and sums below
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          uint32_t r2[32];
          if (EPI == EPI_SWIGLU) tmem_ld_32x32(t_row + BN_OUT + c * 32, r2);
          tmem_ld_wait();
          // own accumulators first, then the contributors in the order of their k ranges
          for (int ci = 1; ci <= others; ++ci) {
            const float *src = sp.partials + (size_t)(p_first + ci) * SK_SLOT_FLOATS + slab;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __ldcg(src + (c * 32 + j) * 32 + lane);
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + v[j]);
            if (EPI == EPI_SWIGLU) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __ldcg(src + (BN_OUT + c * 32 + j) * 32 + lane);
#pragma unroll
              for (int j = 0; j < 32; ++j) r2[j] = __float_as_uint(__uint_as_float(r2[j]) + v[j]);
            }
          }
          const int col0 = n0 + c * 32;
          if (!row_ok || col0 >= p.n) continue;
          epilogue_store_chunk<EPI>(r, r2, row, col0, p, rc);
        }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) remote_arrive(map_to_cta(bar_tempty + 8 * acc, 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
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

constexpr int kSmemSk = SK_STAGES * STAGE2_BYTES + 16 * SK_STAGES + 64 + 32 + 1024;

template <int EPI, bool BKB = false>
int launch_streamk(const GemmArgs &g) {
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? 128 : 256;
  Context &c = ctx();
  CUtensorMap tmA, tmB, tmB2;
  B200_TRY(make_map_2d(&tmA, g.a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.k, g.m, g.lda, BK2, BM2));
  if (BKB)
    B200_TRY(make_map_2d(&tmB, g.b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, 64, ((g.k + 63) / 64) * g.n, 64, 64, 128));
  else
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
  p.res_mod = g.res_mod;
  p.res_rem = g.res_rem;
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
  auto kern = gemm_tc2_streamk_kernel<EPI, BKB>;
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
  // whole tiles round by round; the tiles of the last, part-filled round in k-blocks — together
  // with one more full round's when that remainder is below half the pairs (each cut tile would
  // otherwise have four or more contributors); below P tiles, all of them
  const int T = p.num_tiles;
  int pairs = max_pairs, dp_tiles = 0;
  if (T >= max_pairs) {
    const int rem = T % max_pairs;
    if (rem == 0) dp_tiles = T;
    else if (2 * rem >= max_pairs) dp_tiles = T - rem;
    else dp_tiles = T - rem - max_pairs;
  } else {
    const long long units = (long long)T * p.k_blocks;
    pairs = (int)(units < max_pairs ? units : max_pairs);
  }
  const long long units = (long long)(T - dp_tiles) * p.k_blocks;
  sp.dp_tiles = dp_tiles;
  sp.units_q = (int)(units / pairs);
  sp.units_r = (int)(units % pairs);
  void *ws = nullptr;
  B200_TRY(splitk_workspace(SK_COUNTER_BYTES + (size_t)max_pairs * SK_SLOT_FLOATS * sizeof(float), &ws));
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
  if (g.b_kblocked) {
    if (g.epilogue == EPI_F16) return launch_streamk<EPI_F16, true>(g);
    return set_error(B200MLIR_ERR_UNSUPPORTED, "a K-blocked B is built for the plain fp16 read-out");
  }
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
