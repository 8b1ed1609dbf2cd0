// fp16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// What this replaces in the reference, piece by piece:
//   * hmx_pack_act / hmx_pack_weight (hmx/src/HMXLayout.c:70-545): TMA's 128-byte
//     swizzle rearranges row-major global tiles on their way into shared memory;
//     there is no pack kernel and no packed copy of A or B in HBM.
//   * the 2-slot DMA ring of hmx-partition
//     (lib/Dialect/Hmx/Transforms/HmxPartitionPass.cpp:10-84): a STAGES-deep
//     mbarrier ring filled by one producer thread.
//   * hmx_acc_clear / hmx_mma_f16 (hmx/src/HMXAPI.c:36-55): tcgen05.mma with the
//     accumulate flag off on a tile's first K step, fp32 accumulators in TMEM.
//   * hmx_acc_store + hmx_unpack_acc (HMXAPI.c:39-44, HMXLayout.c:776-999) on a
//     second thread in batches (HmxVectorExecutor.h:1-27): four epilogue warps
//     drain one TMEM accumulator stage (tcgen05.ld, convert, fused epilogue,
//     store) while the MMA thread fills the other.
//
// One persistent CTA per SM, 192 threads: warp 0 = TMA producer (one lane),
// warp 1 = TMEM owner + MMA issuer (one lane), warps 2-5 = epilogue.
// A is [M,K] row-major (K-major operand); B is [K,N] row-major, consumed as it
// lies through an MN-major shared-memory descriptor.
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.h"
#include "gemm_tc_common.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int BK = 64;                   // 64 fp16 = one 128-byte swizzle row
constexpr int A_STAGE_BYTES = BM * 128;  // 16 KiB
constexpr int B_SLAB_BYTES = BK * 128;   // 64 k-rows x 64 n (128 B) = 8 KiB
constexpr int NUM_THREADS = 192;

template <int BN_MMA, int STAGES, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmB2, const TcParams p) {
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? BN_MMA / 2 : BN_MMA;
  constexpr int N_SLABS = BN_MMA / 64;
  constexpr int B_STAGE_BYTES = N_SLABS * B_SLAB_BYTES;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  constexpr int TMEM_COLS = 2 * BN_MMA <= 32 ? 32 : 2 * BN_MMA;  // power of two by construction
  // int8 form (EPI_I32): both operands K-major (B arrives transposed), 128 int8 per swizzle row,
  // K = 32 per instruction: the same bytes per stage and per step as the fp16 form
  constexpr bool I8 = EPI == EPI_I32;
  constexpr uint32_t IDESC = I8 ? make_idesc(/*D=s32*/ 2, /*A=s8*/ 1, /*B=s8*/ 1, /*A K-major*/ 0, /*B K-major*/ 0,
                                             BM, BN_MMA)
                                : make_idesc(/*D=f32*/ 1, /*A=f16*/ 0, /*B=f16*/ 0, /*A K-major*/ 0,
                                             /*B MN-major*/ 1, BM, BN_MMA);
  constexpr int KSTEP = I8 ? 128 : BK;  // elements of K per stage

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // control block after the stages
  const uint32_t ctrl = smem_base + STAGES * STAGE_BYTES;
  const uint32_t bar_full = ctrl;                     // STAGES x 8
  const uint32_t bar_empty = ctrl + 8 * STAGES;       // STAGES x 8
  const uint32_t bar_tfull = ctrl + 16 * STAGES;      // 2 x 8
  const uint32_t bar_tempty = ctrl + 16 * STAGES + 16;  // 2 x 8
  const uint32_t tmem_slot = ctrl + 16 * STAGES + 32;
  uint8_t *ctrl_gen = smem_raw + (ctrl - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(ctrl_gen + 16 * STAGES + 32);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ctrl_gen + 16 * STAGES + 36);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A programmatic dependent of the previous kernel in the stream: our own successor may start
  // now; we touch what the predecessor wrote only after the producer's griddepcontrol.wait
  // (every other access of the CTA is ordered after it through the mbarriers).
  pdl_trigger();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (EPI == EPI_SWIGLU) tma_prefetch_desc(&tmB2);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, TMEM_COLS);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, p.m_blocks, p.n_blocks, p.group_m, m_blk, n_blk);
        const int m0 = m_blk * BM, n0 = n_blk * BN_OUT;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, 1, tile)) {
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(full, STAGE_BYTES);
          tma_load_2d(sa, &tmA, full, kb * KSTEP, m0);
          if (I8) tma_load_2d(sb, &tmB, full, kb * KSTEP, n0);  // [BN_MMA rows of Bᵀ] x 128 bytes
#pragma unroll
          for (int s = 0; s < (I8 ? 0 : N_SLABS); ++s) {
            if (EPI == EPI_SWIGLU && s >= N_SLABS / 2)
              tma_load_2d(sb + s * B_SLAB_BYTES, &tmB2, full, n0 + (s - N_SLABS / 2) * 64, kb * BK);
            else
              tma_load_2d(sb + s * B_SLAB_BYTES, &tmB, full, n0 + s * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        // Whole-K form: one accumulator per tile.  K-looped form: one per K segment of
        // p.seg_kb k-blocks, started with accumulate off — the read-out warps round each to
        // fp16 and keep the running sum themselves (test_matmul_kloop.py:87-98).
        // (position inside the K segment by counting: a division costs the lone issuing thread ~300 clocks)
        for (int kb = 0, in_seg = 0; kb < p.k_blocks; ++kb) {
          const bool seg_start = EPI == EPI_KLOOP_F16 ? in_seg == 0 : kb == 0;
          if (seg_start) {
            if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, 2, tile)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
          }
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN_MMA);
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, 3, tile)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // A: K-major, 8-row groups 1024 B apart; one K=16 step is 32 bytes inside the swizzle row
            const uint64_t adesc = smem_desc_sw128(sa + k * 32, 16, 1024);
            // B: MN-major, 64-column slabs B_SLAB_BYTES apart, 8-k groups 1024 B apart;
            // one K=16 step is 16 rows of 128 bytes
            if (I8) {
              mma_i8_ss(d_tmem, adesc, smem_desc_sw128(sb + k * 32, 16, 1024), IDESC, (seg_start && k == 0) ? 0u : 1u);
              continue;
            }
            const uint64_t bdesc = smem_desc_sw128(sb + k * 2048, B_SLAB_BYTES, 1024);
            mma_f16_ss(d_tmem, adesc, bdesc, IDESC, (seg_start && k == 0) ? 0u : 1u);
          }
          mma_commit(bar_empty + 8 * stage);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
          if (++in_seg == p.seg_kb) in_seg = 0;
          const bool seg_end = EPI == EPI_KLOOP_F16 ? (in_seg == 0 || kb + 1 == p.k_blocks)
                                                    : kb + 1 == p.k_blocks;
          if (seg_end) {
            mma_commit(bar_tfull + 8 * acc);  // accumulator complete
            if (++acc == 2) {
              acc = 0;
              acc_phase ^= 1u;
            }
          }
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(tile, p.m_blocks, p.n_blocks, p.group_m, m_blk, n_blk);
      const int m0 = m_blk * BM, n0 = n_blk * BN_OUT;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.m;
      if constexpr (EPI == EPI_KLOOP_F16) {
        // running fp32 sums of this row's BN_MMA columns; every segment is rounded to fp16 first
        float sum[BN_MMA];
#pragma unroll
        for (int e = 0; e < BN_MMA; ++e) sum[e] = 0.0f;
        const int segs = (p.k_blocks + p.seg_kb - 1) / p.seg_kb;
        bool ok = true;
        for (int sg = 0; sg < segs; ++sg) {
          ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, 4, tile);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN_MMA);
#pragma unroll
          for (int c = 0; c < BN_MMA / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e += 2)
              add_rounded2(sum[c * 32 + e], sum[c * 32 + e + 1], __uint_as_float(r[e]), __uint_as_float(r[e + 1]));
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1u;
          }
        }
        if (!ok) break;
#pragma unroll
        for (int c = 0; c < BN_MMA / 32; ++c) {
          uint32_t r[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(sum[c * 32 + e]);
          const int col0 = n0 + c * 32;
          if (row_ok && col0 < p.n) epilogue_store_chunk<EPI_F16>(r, r, row, col0, p);
        }
      } else {
        ResChunk rc, rc_next;
        residual_prefetch<EPI>(rc, row, n0, row_ok, p);  // under the tile's main loop
        bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, 4, tile);
        ok = __all_sync(0xffffffffu, ok);  // the loads below need the warp converged
        if (!ok) break;
        tc_fence_after_sync();
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
        if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // A wait ran out: give copies and MMAs still in flight a bounded time to
      // land before the TMEM columns and shared memory are handed back.
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side ------------------------------------------------------------------------

struct Variant {
  TcVariantInfo info;
};

constexpr int ctrl_bytes(int stages) { return 16 * stages + 64; }
constexpr int smem_for(int bn_mma, int stages) {
  return stages * (A_STAGE_BYTES + (bn_mma / 64) * B_SLAB_BYTES) + ctrl_bytes(stages) + 1024;
}

const TcVariantInfo kVariants[] = {
    {"tc128x256x64_s4", 128, 256, 64, 4, 1, smem_for(256, 4), 512, 0.75},
    {"tc128x128x64_s6", 128, 128, 64, 6, 1, smem_for(128, 6), 256, 0.50},
    {"tc128x64x64_s8", 128, 64, 64, 8, 1, smem_for(64, 8), 128, 0.30},
    // a pair of CTAs per 256 x 256 tile (gemm_tcgen05_2cta.cu)
    {"tc256x256x64_2cta_s6", 256, 256, 64, 6, 2, 6 * 32768 + 16 * 6 + 64 + 1024, 512, 0.85},
    {"tc256x256x128_2cta_s3", 256, 256, 128, 3, 2, 6 * 32768 + 16 * 6 + 64 + 1024, 512, 0.10},
    // the same pair tile with the k-blocks of all tiles dealt out evenly (gemm_tcgen05_streamk.cu)
    {"tc256x256x64_2cta_streamk", 256, 256, 64, 6, 2, 6 * 32768 + 16 * 6 + 64 + 1024, 512, 0.85, true},
};
constexpr int kNumVariants = sizeof(kVariants) / sizeof(kVariants[0]);

template <int BN_MMA, int STAGES, int EPI>
int launch_one(const GemmArgs &g, const TcVariantInfo &vi) {
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? BN_MMA / 2 : BN_MMA;
  Context &c = ctx();
  CUtensorMap tmA, tmB, tmB2;
  B200_TRY(make_map_2d(&tmA, g.a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.k, g.m, g.lda, BK, BM));
  B200_TRY(make_map_2d(&tmB, g.b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.n, g.k, g.ldb, 64, BK));
  if (EPI == EPI_SWIGLU)
    B200_TRY(make_map_2d(&tmB2, g.b2, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g.n, g.k, g.ldb, 64, BK));
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
  p.m_blocks = (int)((g.m + BM - 1) / BM);
  p.n_blocks = (int)((g.n + BN_OUT - 1) / BN_OUT);
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.k_blocks = (int)((g.k + BK - 1) / BK);
  p.group_m = ctx().opt.gemm_group_m >= 1 ? (int)ctx().opt.gemm_group_m : GROUP_M;
  p.seg_kb = g.block_k >= BK ? g.block_k / BK : 1;
  set_push_params(p, g);
  p.status = c.d_status;
  auto kern = gemm_tc_kernel<BN_MMA, STAGES, EPI>;
  static bool attr_set = false;  // one per template instantiation
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, vi.smem_bytes));
    attr_set = true;
  }
  int grid = p.num_tiles < c.sm_count ? p.num_tiles : c.sm_count;
  B200_CUDA(launch_maybe_dependent(c.opt.gemm_dependent_launch != 0, kern, dim3((unsigned)grid), dim3(NUM_THREADS),
                                   (size_t)vi.smem_bytes, c.stream, tmA, tmB, tmB2, p));
  return check_launch(vi.name);
}

template <int BN_MMA, int STAGES>
int launch_epi(const GemmArgs &g, const TcVariantInfo &vi) {
  switch (g.epilogue) {
    case EPI_F16: return launch_one<BN_MMA, STAGES, EPI_F16>(g, vi);
    case EPI_F32_RES: return launch_one<BN_MMA, STAGES, EPI_F32_RES>(g, vi);
    case EPI_F16_RES16: return launch_one<BN_MMA, STAGES, EPI_F16_RES16>(g, vi);
    case EPI_PUSH16: return launch_one<BN_MMA, STAGES, EPI_PUSH16>(g, vi);
    case EPI_SWIGLU:
      if constexpr (BN_MMA >= 128) return launch_one<BN_MMA, STAGES, EPI_SWIGLU>(g, vi);
      return set_error(B200MLIR_ERR_UNSUPPORTED, "swiglu epilogue needs a variant with BN >= 128");
    case EPI_KLOOP_F16:
      // the read-out warps hold a row's running sums in registers: 128 columns is what fits
      if constexpr (BN_MMA == 128) return launch_one<BN_MMA, STAGES, EPI_KLOOP_F16>(g, vi);
      return set_error(B200MLIR_ERR_UNSUPPORTED, "k-looped read-out is built for the 128x128 variant only");
    default:
      return set_error(B200MLIR_ERR_UNSUPPORTED, "tensor-core gemm: epilogue %d not built",
                       g.epilogue);
  }
}

bool al16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

}  // namespace

int launch_gemm_i8_tc(const int8_t *a, const int8_t *bt, int32_t *c, int64_t m, int64_t n, int64_t k, int64_t lda,
                      int64_t ldbt, int64_t ldc) {
  B200_TRY(ensure_ready());
  constexpr int BN_MMA = 128, STAGES = 6;
  // enough 256 x 256 tiles for the SM pairs: the two-CTA form (option gemmVariant = 1 keeps this one)
  if (m >= 512 && n >= 512 && (m / 256) * (n / 256) >= 32 && ctx().opt.gemm_variant != 1 && al16(a) && al16(bt) &&
      al16(c) && lda % 16 == 0 && ldbt % 16 == 0 && ldc % 4 == 0 && n % 4 == 0)
    return launch_gemm_i8_tc_pair(a, bt, c, m, n, k, lda, ldbt, ldc);
  if (!al16(a) || !al16(bt) || !al16(c) || lda % 16 || ldbt % 16 || ldc % 4 || n % 4 || m < 1 || n < 1 || k < 1)
    return set_error(B200MLIR_ERR_UNSUPPORTED, "int8 tensor-core gemm: alignment (rows 16-byte aligned, N a multiple of 4)");
  Context &c_ = ctx();
  const TcVariantInfo &vi = kVariants[1];  // 128x128, six stages of 32 KiB: the same ring
  CUtensorMap tmA, tmB;
  B200_TRY(make_map_2d(&tmA, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k, m, lda, 128, BM));
  B200_TRY(make_map_2d(&tmB, bt, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k, n, ldbt, 128, BN_MMA));
  TcParams p;
  p.c = c;
  p.res = nullptr;
  p.ldc = ldc;
  p.ldres = 0;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.m_blocks = (int)((m + BM - 1) / BM);
  p.n_blocks = (int)((n + BN_MMA - 1) / BN_MMA);
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.k_blocks = (int)((k + 127) / 128);
  p.group_m = GROUP_M;
  p.seg_kb = 1;
  GemmArgs none;
  set_push_params(p, none);
  p.status = c_.d_status;
  auto kern = gemm_tc_kernel<BN_MMA, STAGES, EPI_I32>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, vi.smem_bytes));
    attr_set = true;
  }
  const int grid = p.num_tiles < c_.sm_count ? p.num_tiles : c_.sm_count;
  B200_CUDA(launch_maybe_dependent(false, kern, dim3((unsigned)grid), dim3(NUM_THREADS), (size_t)vi.smem_bytes, c_.stream,
                                   tmA, tmB, tmB, p));
  return check_launch("gemm_tc_i8_128x128");
}

int tc_variant_count() { return kNumVariants; }
const TcVariantInfo &tc_variant_info(int v) { return kVariants[v]; }

// Legality of one variant for one problem.  The vocabulary follows the
// reference's refusal reasons (hmx_search.py:196-205): "min-rows" and
// "tile-alignment" mean the same thing; the VTCM budget becomes the
// shared-memory / TMEM budget of the variant.
const char *tc_variant_verdict(int v, const GemmArgs &g) {
  if (v < 0 || v >= kNumVariants) return "no-such-variant";
  const TcVariantInfo &vi = kVariants[v];
  if (g.m <= 4) return "min-rows";  // HmxTarget.h:100,201 — decode rows go to the vector path
  if (g.k < 8 || g.n < 8) return "tile-alignment";
  if (g.k % 8 || g.n % 8 || g.lda % 8 || (!g.b_kblocked && g.ldb % 8)) return "tile-alignment";
  // the K-blocked B image: the pair kernels' plain fp16 read-out only
  if (g.b_kblocked && (vi.cta_group != 2 || vi.bk != 64 || g.epilogue != EPI_F16)) return "epilogue-unsupported";
  if (g.epilogue == EPI_PUSH16) {
    if (!g.push || g.push->world < 1 || g.push->world > kMaxPushRanks || g.push->rows_per_rank < 1 ||
        g.push->rows_per_rank * g.push->world != g.m)
      return "epilogue-unsupported";
    for (int i = 0; i < g.push->world; ++i)
      if (!g.push->recv[i] || !al16(g.push->recv[i])) return "tile-alignment";
    if (!al16(g.a) || !al16(g.b)) return "tile-alignment";
  } else if (!al16(g.a) || !al16(g.b) || !al16(g.c)) {
    return "tile-alignment";
  }
  if (g.epilogue == EPI_F32_RES) {
    if (g.ldc % 4 || (g.res && (g.ldres % 4 || !al16(g.res)))) return "tile-alignment";
  } else {
    if (g.ldc % 8) return "tile-alignment";
    if (g.epilogue == EPI_F16_RES16 && (g.ldres % 8 || !al16(g.res))) return "tile-alignment";
  }
  if (g.epilogue == EPI_SWIGLU && (!g.b2 || !al16(g.b2))) return "tile-alignment";
  if (g.epilogue == EPI_SWIGLU && vi.bn < 128) return "epilogue-unsupported";
  // K-looped accumulation: segments of whole k-blocks, on the variant whose read-out warps
  // can hold a row of running sums (anything else stays on the CUDA-core path)
  // (the one-CTA 128x128 variant, and the two-CTA variant with 64-deep stages, whose eight read-out warps take 128 columns each)
  if (g.epilogue == EPI_KLOOP_F16 &&
      (!((vi.cta_group == 1 && vi.bn == 128) ||
         (vi.cta_group == 2 && vi.bk == 64 && !vi.stream_k && ctx().opt.kloop_pairs != 0)) ||
       g.block_k < BK || g.block_k % BK))
    return "epilogue-unsupported";
  if (vi.stream_k) {
    if (g.epilogue == EPI_KLOOP_F16 || g.epilogue == EPI_I32) return "epilogue-unsupported";
    if (!streamk_shape_ok(g)) return "extent-range";
  }
  if (g.m > 0x7fffffff || g.n > 0x7fffffff || g.k > 0x7fffffff) return "extent-range";
  if (((g.m + BM - 1) / BM) * ((g.n + 31) / 32) > 0x3fffffff) return "extent-range";
  if (vi.smem_bytes > 227 * 1024) return "smem-budget";
  if (vi.tmem_cols > 512) return "tmem-budget";
  return "ok";
}

int launch_gemm_tc(int v, const GemmArgs &g) {
  B200_TRY(ensure_ready());
  const char *verdict = tc_variant_verdict(v, g);
  if (strcmp(verdict, "ok") != 0)
    return set_error(B200MLIR_ERR_UNSUPPORTED, "gemm variant %d refused: %s", v, verdict);
  const TcVariantInfo &vi = kVariants[v];
  switch (v) {
    case 0: return launch_epi<256, 4>(g, vi);
    case 1: return launch_epi<128, 6>(g, vi);
    case 2: return launch_epi<64, 8>(g, vi);
    case 3: return launch_gemm_tc_pair(g, false);
    case 4: return launch_gemm_tc_pair(g, true);
    case 5: return launch_gemm_tc_streamk(g);
  }
  return set_error(B200MLIR_ERR_BAD_ARG, "no such gemm variant %d", v);
}

}  // namespace b200
