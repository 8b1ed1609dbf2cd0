// w8a16 GEMM, C[M,N] = A[M,K] · (q[K,N] · s[N]), as a weight-streaming kernel whose
// dequantised operand never touches shared memory.
//
// The op reads 45 MB of int8 for the 4096 x 11008 config and little else, so everything is
// arranged around moving that stream at HBM speed and keeping the per-byte work small:
//   * every CTA (one per SM) owns a contiguous range of output channels (74-75 of 11008) for
//     the WHOLE of K: no split-K, no partial sums in memory, no atomics, no scratch, nothing
//     to wait for at the end, and the result is bit-reproducible;
//   * two threads feed the SM (one issues a copy per ~650 clocks): per K=128 step one `cp.async.bulk` of the CTA's channels
//     (9.5 KB, contiguous in the image) into a twelve-slot ring (~110 KB in flight; a read-only
//     bulk stream measured 6.2-6.6 TB/s chip-wide at 64-128 KB in flight per SM); the first
//     twelve copies are issued before the rest of the CTA's set-up;
//   * sixteen converter warps (four groups, four steps in flight) turn a slot into fp16 in registers (`prmt` + `sub.f16x2`,
//     exact) and write it with `tcgen05.st` straight into TMEM, where the MMA takes its A
//     operand from (channels on the 128 lanes, two k per 32-bit column).  Shared memory
//     carries the int8 bytes in and out once, nothing else (tcgen05.st sustains ~170 B/clk);
//   * a thread can issue one small MMA per ~50 clocks whatever its M and N, but threads of
//     different warps issue in parallel (four issuers: 13.6 clocks per 128x16x16 MMA in
//     aggregate), so steps rotate over up to 4 issuer warps, each with its own accumulator,
//     summed at read-out;
//   * operands are swapped: weights are the MMA's A (128 rows, 74 live), the activations its
//     B (N_mma = M rows padded to 16, 64 or 128), fetched per step by TMA (L2 hits).
//
// Resident image, built once per weight (the analogue of the reference's pre-packed weight:
// backend/hmx_weight_prepack.py:124-212, lib/Dialect/Hmx/Transforms/WeightResidentPass.cpp:9-93):
//   [step = k/128][channel n][8 pieces of 16 bytes]
// where piece j of channel n (stored at position j ^ (n & 7), so that 8 neighbouring channels'
// piece j fall in 8 different bank groups) holds q[128*step + 16*j + 0..15][n] + 128;
// positions with k >= K hold 128 (zero weight).  Any channel range of one step is contiguous.
#include "common.h"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

using namespace ptx;

constexpr int CH_PASS = 128;             // channels per pass = MMA rows
constexpr int STEP_K = 128;              // k per step
constexpr int CH_BYTES = STEP_K;         // bytes of one channel in one step
constexpr int SLOT_BYTES = 10 * 1024;    // ring slot (80 channels); wider ranges use 2 slots' worth
constexpr int CONV_W = 16;               // converter warps: quadrant = warp % 4, group = warp / 4
constexpr int CONV_G = CONV_W / 4;       // converter groups; a step is converted by one group
constexpr int EPI_W = 4;                 // issue / read-out warps: lane 0 of the first ISS issues MMAs,
                                         // then each warp reads out its TMEM lane quadrant (warp % 4)
constexpr int W_MMA0 = CONV_W;           // first of them (also allocates TMEM)
constexpr int W_WPROD = CONV_W + EPI_W;  // first of the WPRODS weight producer warps
constexpr int WPRODS = 2;                // a thread issues a copy per ~650 clocks; two keep ahead of HBM
constexpr int W_APROD = W_WPROD + WPRODS;  // activation producer warp
constexpr int THREADS = (W_APROD + 1) * 32;  // 736
constexpr int TMEM_COLS = 512;

__device__ __forceinline__ uint32_t dq2(uint32_t word, uint32_t selector) {
  // two biased bytes -> two fp16 values: 0x64xx is 1024 + xx; minus 1152 gives xx - 128
  uint32_t h, out;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(h) : "r"(word), "r"(0x64646464u), "r"(selector));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(out) : "r"(h), "r"(0x64806480u));
  return out;
}
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_st_32x32_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32_x32(uint32_t taddr, const uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_32x32_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// D[tmem] (+)= A[tmem] · B[smem descriptor]
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Region stamps for timeline debugging (the analogue of the reference's light-weight profiling
// regions, lib/Transforms/HexagonLWPInstrumentation.cpp): compiled in only with
// -DB200MLIR_W8_TRACE; CTA 3 records clock64() per role and step.
#ifdef B200MLIR_W8_TRACE
__device__ long long g_trace3_buf[8 * 64];
#define TR(role, u) do { if (blockIdx.x == 3 && (u) < 64) trace_s[(role) * 64 + (u)] = clock64(); } while (0)
#else
#define TR(role, u) do { } while (0)
#endif

struct StreamParams {
  const uint8_t *image;  // [ksteps][n][128]
  const __half *scales;
  __half *c;
  int64_t ldc;
  int m, n, ksteps;
  int chan_q, chan_r;  // n = grid * chan_q + chan_r: CTA b owns chan_q channels, one more if b < chan_r
  int rot_mul;         // (ksteps << 16) / grid: CTA b starts at k step (b * rot_mul) >> 16
  int *status;
};

// NM: activation rows padded to the MMA's N.  ISS: MMA issuer warps.  TB: TMEM A buffers.
// DA: activation slots (their TMA round trip is ~2000 clocks even from L2, so the ring runs
// well ahead of the TMEM buffers).  DEPTH: int8 ring slots of SLOT bytes (SLOT >= channels
// per pass * 128).  TMEM columns: accumulators [0, ISS*NM), A buffers from ISS*NM, 64 each.
template <int NM, int ISS, int TB, int DA, int DEPTH, int SLOT>
__global__ void __launch_bounds__(THREADS, 1)
w8a16_tmem_kernel(const __grid_constant__ CUtensorMap tmA, const StreamParams p) {
  constexpr int A_BYTES = 2 * NM * 128;  // two [NM][64] activation sub-tiles per step
  constexpr int A_COL0 = ISS * NM;
  static_assert(A_COL0 + TB * 64 <= TMEM_COLS, "TMEM budget");
  // A parity wait tells "phase q of this barrier is complete" from "not yet" only for a
  // waiter that has seen phase q-1 complete; one that skips a phase can be let through a
  // whole ring turn early.  So every ring slot belongs to ONE waiter on each side: int8 slot
  // i % DEPTH and TMEM buffer i % TB to converter group i % CONV_G, TMEM buffer and
  // activation slot i % DA to issuer i % ISS; the producers walk all steps in order.
  static_assert(DEPTH % CONV_G == 0 && DEPTH % WPRODS == 0 && TB % CONV_G == 0 && TB % ISS == 0 && DA % ISS == 0,
                "slot ownership");
  constexpr uint32_t IDESC = make_idesc(/*D f32*/ 1, /*A f16*/ 0, /*B f16*/ 0, /*A K-major*/ 0,
                                        /*B K-major*/ 0, 128, NM);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t act0 = base;                         // DA activation slots (1 KiB aligned)
  const uint32_t wq0 = act0 + DA * A_BYTES;           // DEPTH int8 slots
  const uint32_t ctrl = wq0 + DEPTH * SLOT;
  const uint32_t bar_wfull = ctrl;                    // DEPTH: weights landed (bulk copy bytes)
  const uint32_t bar_wfree = ctrl + 128;              // DEPTH: int8 slot read by the step's converter warps
  const uint32_t bar_afull = ctrl + 256;              // DA: activations landed (TMA bytes)
  const uint32_t bar_afree = ctrl + 384;              // DA: MMAs that read the slot complete (commit)
  const uint32_t bar_tfull = ctrl + 512;              // TB: TMEM A buffer written by the step's converter warps
  const uint32_t bar_done = ctrl + 576;               // TB: MMAs that read the buffer complete (commit)
  const uint32_t bar_accfull = ctrl + 640;            // pass's accumulators complete (ISS arrivals)
  const uint32_t bar_accfree = ctrl + 648;            // accumulators read out (EPI_W arrivals)
  const uint32_t tmem_slot = ctrl + 656;
  uint8_t *ctrl_gen = smem_raw + (ctrl - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(ctrl_gen + 656);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ctrl_gen + 660);
  static_assert(DEPTH <= 16 && DA <= 16 && TB <= 8, "barrier table");

#ifdef B200MLIR_W8_TRACE
  __shared__ long long trace_s[8 * 64];
#endif
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) TR(7, 0);
  // Launched as a programmatic dependent of the previous kernel in the stream (option
  // w8a16DependentLaunch): let OUR successor start as early, and wait for our predecessor only
  // where its data is touched — the activations and C.  The weight stream does not wait.
  pdl_trigger();
  // this CTA's channels, walked in passes of at most SLOT / 128
  constexpr int CH_MAX = SLOT / CH_BYTES;
  // (no division here: the first weight copies wait for these, and a 64-bit division is a
  // subroutine of several hundred clocks)
  const int c_begin = (int)blockIdx.x * p.chan_q + min((int)blockIdx.x, p.chan_r);
  const int c_end = c_begin + p.chan_q + ((int)blockIdx.x < p.chan_r ? 1 : 0);
  const int passes = (c_end - c_begin + CH_MAX - 1) / CH_MAX;
  const int ksteps = p.ksteps;
  const int nsteps = passes * ksteps;  // local steps: pass-major, then k
  // Owning all of K, a CTA is free to walk it in any order: each starts at its own k step, so
  // that at any moment the 148 CTAs read 148 different places of the image (all of them
  // asking for the same 1.4 MB row at once leaves most DRAM channels idle).
  const int rot = (int)(((unsigned)blockIdx.x * (unsigned)p.rot_mul) >> 16);
  // Position of a local step without divisions (a lone thread pays ~300 clocks for one): the
  // pass, the step inside the pass, and what they select.
  struct Cursor {
    int pass, kin;
    __device__ void advance(int n, int ksteps) {
      kin += n;
      while (kin >= ksteps) {
        kin -= ksteps;
        ++pass;
      }
    }
  };
  auto k_of = [&](const Cursor &c) { const int ks = c.kin + rot; return ks >= ksteps ? ks - ksteps : ks; };
  auto ch0_of = [&](const Cursor &c) { return c_begin + c.pass * CH_MAX; };
  auto ch_of = [&](const Cursor &c) { return min(CH_MAX, c_end - ch0_of(c)); };
  auto src_of = [&](const Cursor &c) { return p.image + ((size_t)k_of(c) * p.n + ch0_of(c)) * CH_BYTES; };

  // The two producer warps set up their own barriers, tell the others (barrier 1, without
  // waiting) and start the first copies while the rest of the CTA is still setting up.
  if (warp >= W_WPROD && warp < W_APROD) {
    const int r = warp - W_WPROD;  // this producer's steps: r, r + WPRODS, ...
    if (lane < DEPTH && lane % WPRODS == r) mbar_init(bar_wfull + 8 * lane, 1);
    fence_barrier_init();
    __syncwarp();
    asm volatile("bar.arrive 1, %0;" ::"n"(THREADS) : "memory");
    if (lane == 0) {
      Cursor c{0, 0};
      c.advance(r, ksteps);
      for (int i = r; i < DEPTH && i < nsteps; i += WPRODS, c.advance(WPRODS, ksteps)) {
        const uint32_t bytes = (uint32_t)(ch_of(c) * CH_BYTES);
        mbar_expect_tx(bar_wfull + 8 * i, bytes);
        bulk_load(wq0 + i * SLOT, src_of(c), bytes, bar_wfull + 8 * i);
      }
    }
  }
  if (warp == W_APROD) {
    if (lane < DA) mbar_init(bar_afull + 8 * lane, 1);
    fence_barrier_init();
    __syncwarp();
    asm volatile("bar.arrive 1, %0;" ::"n"(THREADS) : "memory");
    if (lane == 0) {
      pdl_wait();  // the activations may be the previous kernel's output
      Cursor c{0, 0};
      for (int i = 0; i < DA && i < nsteps; ++i, c.advance(1, ksteps)) {
        const uint32_t full = bar_afull + 8 * i, dst = act0 + i * A_BYTES;
        const int ks = k_of(c);
        mbar_expect_tx(full, A_BYTES);
        tma_load_2d(dst, &tmA, full, ks * STEP_K, 0);                  // zero fill past K and past M
        tma_load_2d(dst + NM * 128, &tmA, full, ks * STEP_K + 64, 0);
      }
    }
  }
  if (warp == 0) {
    // the remaining ~40 barriers, one lane each (a lone thread needs ~1000 clocks for them)
    if (lane < DEPTH) mbar_init(bar_wfree + 8 * lane, 4);
    if (lane < DA) mbar_init(bar_afree + 8 * lane, 1);
    if (lane < TB) {
      mbar_init(bar_tfull + 8 * lane, 4);
      mbar_init(bar_done + 8 * lane, 1);
    }
    if (lane == 0) {
      mbar_init(bar_accfull, ISS);
      mbar_init(bar_accfree, EPI_W);
      *abort_flag = 0;
    }
    fence_barrier_init();
  }
  if (warp == W_MMA0) {
    __syncwarp();
    tmem_alloc(tmem_slot, TMEM_COLS);
  }
  // Everyone else meets at barrier 1 (the producers only arrived there); the producers wait at
  // barrier 2 for the barriers the others set up, which the others only arrive at.
  uint32_t tmem_base = 0;
  if (warp < W_WPROD) {
    tc_fence_before_sync();
    asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
    tc_fence_after_sync();
    tmem_base = *tmem_slot_gen;
    asm volatile("bar.arrive 2, %0;" ::"n"(THREADS) : "memory");
  } else {
    __syncwarp();
    asm volatile("bar.sync 2, %0;" ::"n"(THREADS) : "memory");
  }
  if (threadIdx.x == 0) TR(7, 1);

  if (warp >= W_WPROD && warp < W_APROD) {
    // ---------------- weight producers: one bulk copy per step, steps dealt round-robin ----------------
    if (lane == 0) {
      const int r = warp - W_WPROD;
      Cursor c{0, 0};
      c.advance(DEPTH + r, ksteps);
      int slot = r;
      uint32_t par = 0;  // parity of the phase that frees the slot: the turn before this one
      for (int i = DEPTH + r; i < nsteps; i += WPRODS, c.advance(WPRODS, ksteps)) {
        if (!mbar_wait(bar_wfree + 8 * slot, par, abort_flag, p.status, 31, i + 1000 * (int)blockIdx.x)) goto done;
        TR(0, i);
        const uint32_t bytes = (uint32_t)(ch_of(c) * CH_BYTES);
        mbar_expect_tx(bar_wfull + 8 * slot, bytes);
        bulk_load(wq0 + slot * SLOT, src_of(c), bytes, bar_wfull + 8 * slot);
        if ((slot += WPRODS) >= DEPTH) {
          slot -= DEPTH;
          par ^= 1u;
        }
      }
    }
  } else if (warp == W_APROD) {
    // ---------------- activation producer: two TMA boxes per step (L2 hits) ----------------
    if (lane == 0) {
      Cursor c{0, 0};
      c.advance(DA, ksteps);
      int b = 0;
      uint32_t par = 0;
      for (int i = DA; i < nsteps; ++i, c.advance(1, ksteps)) {
        if (!mbar_wait(bar_afree + 8 * b, par, abort_flag, p.status, 32, i + 1000 * (int)blockIdx.x)) goto done;
        const uint32_t full = bar_afull + 8 * b;
        const uint32_t dst = act0 + b * A_BYTES;
        const int ks = k_of(c);
        mbar_expect_tx(full, A_BYTES);
        tma_load_2d(dst, &tmA, full, ks * STEP_K, 0);
        tma_load_2d(dst + NM * 128, &tmA, full, ks * STEP_K + 64, 0);
        if (++b == DA) {
          b = 0;
          par ^= 1u;
        }
      }
    }
  } else if (warp < CONV_W) {
    // ---------------- converters: int8 slot -> fp16 in TMEM ----------------
    // Four groups of four warps (one per TMEM lane quadrant); group g takes steps g, g+4, ...
    // so that four steps are in flight and one group's waits hide behind the others' work.
    // A thread converts its channel's whole 128 bytes of the step, in two halves.
    const int q = warp & 3, grp = warp >> 2;
    const int cl = q * 32 + lane;                 // local channel = TMEM lane
    const uint32_t t_dst = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)A_COL0;
    Cursor c{0, 0};
    c.advance(grp, ksteps);
    int slot = grp, b = grp % TB;      // ring positions of step i, kept without divisions
    uint32_t wpar = 0, tpar = 1;       // parities: weights of this turn landed; buffer's previous turn drained
    for (int i = grp; i < nsteps; i += CONV_G, c.advance(CONV_G, ksteps)) {
      const int ch0 = ch0_of(c);
      const int ch = ch_of(c);
      const bool live = cl < ch;
      if ((threadIdx.x & 127) == 0) TR(1, i);
      bool ok = mbar_wait(bar_wfull + 8 * slot, wpar, abort_flag, p.status, 36, i + 1000 * (int)blockIdx.x);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) goto done;
      if ((threadIdx.x & 127) == 0) TR(6, i);
      const uint32_t sw = (uint32_t)((ch0 + cl) & 7);
      const uint32_t s = wq0 + slot * SLOT + (uint32_t)(cl * CH_BYTES);
      uint4 v[8];
      if (live) {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) v[jj] = lds128(s + ((((uint32_t)jj) ^ sw) << 4));
      } else {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) v[jj] = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t r[32];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const uint4 w = v[4 * h + jj];
          r[8 * jj + 0] = dq2(w.x, 0x5140u); r[8 * jj + 1] = dq2(w.x, 0x5342u);
          r[8 * jj + 2] = dq2(w.y, 0x5140u); r[8 * jj + 3] = dq2(w.y, 0x5342u);
          r[8 * jj + 4] = dq2(w.z, 0x5140u); r[8 * jj + 5] = dq2(w.z, 0x5342u);
          r[8 * jj + 6] = dq2(w.w, 0x5140u); r[8 * jj + 7] = dq2(w.w, 0x5342u);
        }
        if (h == 0) {
          if ((threadIdx.x & 127) == 0) TR(2, i);
          ok = mbar_wait(bar_done + 8 * b, tpar, abort_flag, p.status, 37, i + 1000 * (int)blockIdx.x);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) goto done;
        } else {
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_wfree + 8 * slot);  // every byte of the slot has been used: it may be refilled
        }
        tmem_st_32x32_x32(t_dst + (uint32_t)(b * 64 + h * 32), r);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tfull + 8 * b);
      if ((threadIdx.x & 127) == 0) TR(3, i);
      if ((slot += CONV_G) >= DEPTH) {
        slot -= DEPTH;
        wpar ^= 1u;
      }
      if ((b += CONV_G) >= TB) {
        b -= TB;
        tpar ^= 1u;
      }
    }
  } else {
    // ---------------- issue / read-out warps ----------------
    // Per pass: lane 0 of issuer warp j issues the MMAs of steps i = j, j + ISS, ... of the pass,
    // then the whole warp waits for every issuer's MMAs and reads out its lane quadrant.
    const int j = warp - W_MMA0;
    const int q = warp & 3;
    const int cl = q * 32 + lane;
    const uint32_t d_tmem = tmem_base + (uint32_t)(j * NM);
    int i_next = j, b = j % TB, ia = j % DA;  // (lane 0 of an issuer warp only)
    uint32_t tpar = 0, apar = 0;
    for (int pass = 0; pass < passes; ++pass) {
      if (j < ISS && lane == 0) {
        // (a failed wait has raised the CTA's abort flag; the whole warp leaves together below)
        bool ok = pass == 0 || mbar_wait(bar_accfree, (uint32_t)((pass & 1) ^ 1), abort_flag, p.status, 33, pass + 1000 * (int)blockIdx.x);
        const int i_end = (pass + 1) * ksteps;
        bool issued = false;
        // `i_next` is this issuer's next step; its ring positions travel with it
        for (; ok && i_next < i_end; i_next += ISS) {
          const int i = i_next;
          TR(4, i);
          ok = mbar_wait(bar_tfull + 8 * b, tpar, abort_flag, p.status, 34, i + 1000 * (int)blockIdx.x) &&
               mbar_wait(bar_afull + 8 * ia, apar, abort_flag, p.status, 35, i + 1000 * (int)blockIdx.x);
          if (!ok) break;
          tc_fence_after_sync();
          TR(5, i);
          const uint32_t a_tmem = tmem_base + (uint32_t)(A_COL0 + b * 64);
          const uint64_t bdesc0 = smem_desc_sw128(act0 + ia * A_BYTES, 16, 1024);
          const uint64_t bdesc1 = smem_desc_sw128(act0 + ia * A_BYTES + NM * 128, 16, 1024);
          mma_f16_ts(d_tmem, a_tmem, bdesc0, IDESC, issued ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < 8; ++k)
            mma_f16_ts(d_tmem, a_tmem + (uint32_t)(k * 8), (k < 4 ? bdesc0 : bdesc1) + (uint64_t)((k & 3) * 2), IDESC, 1u);
          issued = true;
          mma_commit(bar_done + 8 * b);    // the TMEM A buffer may be rewritten
          mma_commit(bar_afree + 8 * ia);  // and the activation slot
          if ((b += ISS) >= TB) {
            b -= TB;
            tpar ^= 1u;
          }
          if ((ia += ISS) >= DA) {
            ia -= DA;
            apar ^= 1u;
          }
        }
        if (issued) mma_commit(bar_accfull);
        else mbar_arrive(bar_accfull);
      }
      __syncwarp();
      if (*abort_flag) goto done;
      // read-out: sum the issuers' accumulators, scale, round, store
      const int ch0 = c_begin + pass * CH_MAX;
      const int ch = min(CH_MAX, c_end - ch0);
      bool ok = mbar_wait(bar_accfull, (uint32_t)(pass & 1), abort_flag, p.status, 38, pass + 1000 * (int)blockIdx.x);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) goto done;
      tc_fence_after_sync();
      if (warp == W_MMA0 && lane == 0) TR(7, 2 + 2 * pass);
      const bool live = cl < ch;
      const float sc = live ? __half2float(p.scales[ch0 + cl]) : 0.0f;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
      const int pass_first = pass * ksteps;
      pdl_wait();  // C may be something the previous kernel still reads
#pragma unroll 1
      for (int m0 = 0; m0 < NM; m0 += 16) {
        if (m0 >= p.m) break;  // uniform across the warp
        float acc[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] = 0.0f;
#pragma unroll
        for (int jj = 0; jj < ISS; ++jj) {
          // issuer jj's first step in the pass is local step (jj - pass*ksteps) mod ISS
          const int first = ((jj - pass_first % ISS) + ISS) % ISS;
          if (first < ksteps) {
            uint32_t rr[16];
            tmem_ld_32x32_x16(t_row + (uint32_t)(jj * NM + m0), rr);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[e] += __uint_as_float(rr[e]);
          }
        }
        if (live) {
#pragma unroll
          for (int e = 0; e < 16; ++e)
            if (m0 + e < p.m) p.c[(int64_t)(m0 + e) * p.ldc + ch0 + cl] = __float2half_rn(acc[e] * sc);
        }
      }
      if (warp == W_MMA0 && lane == 0) TR(7, 3 + 2 * pass);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_accfree);
    }
  }
done:
  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
#ifdef B200MLIR_W8_TRACE
  if (blockIdx.x == 3) for (int i = threadIdx.x; i < 8 * 64; i += blockDim.x) g_trace3_buf[i] = trace_s[i];
#endif
  if (warp == W_MMA0) {
    if (*abort_flag)
      for (int i = 0; i < 64; ++i) __nanosleep(1000);  // bounded grace for copies / MMAs in flight
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// row-major int8 [K,N] -> [step][channel][8 swizzled pieces of 16 B]; one piece per thread
__global__ void __launch_bounds__(256)
w8a16_tmem_image_kernel(const int8_t *__restrict__ wq, uint4 *__restrict__ image, int K, int N, int ksteps) {
  const int64_t total = (int64_t)ksteps * N * 8;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    // consecutive threads take consecutive channels so that the reads of wq coalesce
    const int n = (int)(i % N);
    const int64_t r = i / N;
    const int j = (int)(r & 7);
    const int ks = (int)(r >> 3);
    uint32_t words[4];
#pragma unroll
    for (int wv = 0; wv < 4; ++wv) {
      uint32_t w = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int k = ks * STEP_K + j * 16 + wv * 4 + e;
        const int qv = k < K ? (int)wq[(int64_t)k * N + n] : 0;
        w |= (uint32_t)((qv + 128) & 0xff) << (8 * e);
      }
      words[wv] = w;
    }
    image[((int64_t)ks * N + n) * 8 + (j ^ (n & 7))] = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

// resident image -> row-major fp16 [K,N], w16[k][n] = f16(f32(q) * f32(s[n])) (the oracle's dequantised
// weight); one 16-byte piece (16 k of one channel) per thread, consecutive threads consecutive channels
__global__ void __launch_bounds__(256)
w8a16_expand_kernel(const uint4 *__restrict__ image, const __half *__restrict__ scales, __half *__restrict__ w16, int K,
                    int N, int ksteps) {
  const int64_t total = (int64_t)ksteps * N * 8;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int n = (int)(i % N);
    const int64_t r = i / N;
    const int j = (int)(r & 7);
    const int ks = (int)(r >> 3);
    const uint4 v = image[((int64_t)ks * N + n) * 8 + (j ^ (n & 7))];
    const float sc = __half2float(scales[n]);
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
    // 16 consecutive k of one channel: 32 contiguous bytes of the K-blocked image
    // [k/64][n][64] (GemmArgs::b_kblocked); k at or past K reads as zero
    const int k0 = ks * STEP_K + j * 16;
    uint32_t outw[8];
#pragma unroll
    for (int e = 0; e < 16; e += 2) {
      const int q0 = (int)((words[e >> 2] >> (8 * (e & 3))) & 0xffu) - 128;
      const int q1 = (int)((words[(e + 1) >> 2] >> (8 * ((e + 1) & 3))) & 0xffu) - 128;
      const __half h0 = k0 + e < K ? __float2half_rn((float)q0 * sc) : __float2half_rn(0.0f);
      const __half h1 = k0 + e + 1 < K ? __float2half_rn((float)q1 * sc) : __float2half_rn(0.0f);
      outw[e >> 1] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
    }
    uint4 *dst = reinterpret_cast<uint4 *>(w16 + ((int64_t)(k0 >> 6) * N + n) * 64 + (k0 & 63));
    dst[0] = make_uint4(outw[0], outw[1], outw[2], outw[3]);
    dst[1] = make_uint4(outw[4], outw[5], outw[6], outw[7]);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

int make_act_map(CUtensorMap *map, const void *a, int64_t m, int64_t k, int64_t lda, int box_rows) {
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

template <int NM, int ISS, int TB, int DA, int DEPTH, int SLOT>
int launch_tmem(const CUtensorMap &tmA, const StreamParams &p, int grid) {
  constexpr int smem = DA * 2 * NM * 128 + DEPTH * SLOT + 1024 + 1024;
  static_assert(smem <= 227 * 1024, "w8a16 kernel exceeds shared memory");
  auto kern = w8a16_tmem_kernel<NM, ISS, TB, DA, DEPTH, SLOT>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set = true;
  }
  if (ctx().opt.w8a16_dependent_launch != 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx().stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    B200_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, p));
  } else {
    kern<<<grid, THREADS, smem, ctx().stream>>>(tmA, p);
  }
  return check_launch("w8a16_tmem");
}

}  // namespace

#ifdef B200MLIR_W8_TRACE
extern "C" __attribute__((visibility("default"))) int b200mlir_debug_get_trace3(long long *host) {
  return (int)cudaMemcpyFromSymbol(host, g_trace3_buf, sizeof(long long) * 8 * 64);
}
#endif

int w8a16_expand_f16(const void *image, const __half *scales_dev, int64_t k, int64_t n, void **w16) {
  B200_TRY(ensure_ready());
  const int ksteps = (int)((k + STEP_K - 1) / STEP_K);
  void *out = nullptr;
  B200_CUDA(cudaMalloc(&out, (size_t)ksteps * STEP_K * n * 2));  // K padded to whole 128-deep steps (two 64-deep blocks each)
  int64_t blocks = ((int64_t)ksteps * n * 8 + 255) / 256;
  const int64_t cap = (int64_t)ctx().sm_count * 32;
  if (blocks > cap) blocks = cap;
  w8a16_expand_kernel<<<(unsigned)blocks, 256, 0, ctx().stream>>>((const uint4 *)image, scales_dev, (__half *)out, (int)k,
                                                                (int)n, ksteps);
  int rc = check_launch("w8a16_expand");
  if (rc) {
    cudaFree(out);
    return rc;
  }
  *w16 = out;
  return 0;
}

int w8a16_build_tmem_image(const int8_t *wq_dev, int64_t k, int64_t n, void **image, size_t *bytes) {
  B200_TRY(ensure_ready());
  const int ksteps = (int)((k + STEP_K - 1) / STEP_K);
  const size_t sz = (size_t)ksteps * n * CH_BYTES;
  void *img = nullptr;
  B200_CUDA(cudaMalloc(&img, sz));
  int64_t blocks = ((int64_t)(sz / 16) + 255) / 256;
  const int64_t cap = (int64_t)ctx().sm_count * 32;
  if (blocks > cap) blocks = cap;
  w8a16_tmem_image_kernel<<<(unsigned)blocks, 256, 0, ctx().stream>>>(wq_dev, (uint4 *)img, (int)k, (int)n, ksteps);
  int rc = check_launch("w8a16_tmem_image");
  if (rc) {
    cudaFree(img);
    return rc;
  }
  *image = img;
  *bytes = sz;
  return 0;
}

// Up to 128 rows per call (the caller loops over row passes).
int launch_w8a16_tmem(const __half *a, const void *image, const __half *scales_dev, int64_t k, int64_t n,
                      __half *c, int64_t m, int64_t lda, int64_t ldc) {
  if (m <= 0 || n <= 0) return 0;
  if (m > 128) return set_error(B200MLIR_ERR_BAD_ARG, "w8a16 kernel takes at most 128 rows per pass");
  const int nm = m <= 16 ? 16 : m <= 64 ? 64 : 128;
  StreamParams p;
  p.image = (const uint8_t *)image;
  p.scales = scales_dev;
  p.c = c;
  p.ldc = ldc;
  p.m = (int)m;
  p.n = (int)n;
  p.ksteps = (int)((k + STEP_K - 1) / STEP_K);
  p.status = ctx().d_status;
  int grid = ctx().sm_count;
  if (grid > n) grid = (int)n;
  p.chan_q = (int)(n / grid);
  p.chan_r = (int)(n % grid);
  p.rot_mul = (p.ksteps << 16) / grid;
  CUtensorMap tmA;
  B200_TRY(make_act_map(&tmA, a, m, k, lda, nm));
  // up to 80 channels per CTA take the deep ring of 10 KiB slots; wider ranges 16 KiB slots
  const bool narrow = (n + grid - 1) / grid <= SLOT_BYTES / CH_BYTES;
  if (nm == 16) return narrow ? launch_tmem<16, 4, 4, 16, 12, SLOT_BYTES>(tmA, p, grid) : launch_tmem<16, 4, 4, 16, 8, 16384>(tmA, p, grid);
  if (nm == 64) return narrow ? launch_tmem<64, 2, 4, 8, 8, SLOT_BYTES>(tmA, p, grid) : launch_tmem<64, 2, 4, 8, 4, 16384>(tmA, p, grid);
  return narrow ? launch_tmem<128, 1, 4, 4, 8, SLOT_BYTES>(tmA, p, grid) : launch_tmem<128, 1, 4, 4, 4, 16384>(tmA, p, grid);
}

}  // namespace b200
