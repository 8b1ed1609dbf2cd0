// Shared host-side declarations of libb200mlir: context, error recording,
// launch accounting and the internal launch functions of every kernel file.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <string>

#include "b200mlir_capi.h"

namespace b200 {

// ---- error recording (thread-local, like cudaGetLastError) ------------------
int set_error(int code, const char *fmt, ...);
void clear_error();

#define B200_CUDA(expr)                                                          \
  do {                                                                           \
    cudaError_t _e = (expr);                                                     \
    if (_e != cudaSuccess)                                                       \
      return b200::set_error(B200MLIR_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,  \
                             cudaGetErrorString(_e), __FILE__, __LINE__);        \
  } while (0)

#define B200_TRY(expr)          \
  do {                          \
    int _rc = (expr);           \
    if (_rc != 0) return _rc;   \
  } while (0)

// ---- process-wide context ------------------------------------------------------
struct Options {
  double rms_eps = 1e-5;           // test_rms_norm.py:17
  double iterations = 10;          // hexagon_options.py:51
  double enable_weight_resident = 1;
  double gemm_variant = -1;        // -1: dispatcher chooses
  double kloop_block_k = 64;
  double kloop_pairs = 1;          // K-looped matmul on the two-CTA kernel (eight read-out warps per CTA); 0 keeps it on the one-CTA kernel
  double w8a16_variant = -1;
  double gemm_group_m = 0;         // 0: the kernels' default band height
  double gemm_dependent_launch = 1;   // programmatic dependent launch of the tcgen05 GEMM kernels
  double w8a16_dependent_launch = 1;  // programmatic dependent launch of the w8a16 kernel (measured: -7 % per call in a chain)
  double w8a16_expand_rows = 64;   // above this many activation rows a w8a16 product takes the expanded fp16 weight
  double attention_stage = 1;      // STAGE of the reference kernel's signature: 1 all keys, 3 causal
  double attention_splits = 0;     // key splits of the attention kernel: 0 chooses by size
  double mlp_residual_mod = 1;     // mlp_block with the residual: add x only in 256-row blocks b with b % mod == rem
  double mlp_residual_rem = 0;     //   (tensor-parallel ranks that sum their partials take turns)
  double attention_tiles = 0;      // query tiles per CTA of the attention kernel: 0 chooses by size, 1 or 2
  double enable_pdl = 0;           // programmatic dependent launch of the row kernels (measured: no gain)
  double replicated_operand_a = 0;  // host-buffer GEMM in a tensor-parallel group: every rank passes the same A; each uploads a row slab and the slabs are exchanged GPU to GPU
  double mlp_phase_timing = 0;      // the MLP block records an event after each of its phases (b200mlir_mlp_phase_times reads them; the read synchronises)
  double row_kernel_walk = -1;     // softmax / RMSNorm grid: 0 one group per row, k resident blocks per SM walking the rows, -1 by size
};

// The stream kernels are enqueued on is a property of the calling thread: b200mlir_set_stream
// binds one to the thread that calls it, a thread that never did uses the legacy default
// stream.  (Seam 1 lets several host threads call the same kernel symbol at once; a single
// process-wide stream would make them race on it.)
struct StreamSlot {
  operator cudaStream_t() const;
  StreamSlot &operator=(cudaStream_t s);
};

struct Context {
  bool ready = false;
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t l2_bytes = 0;
  size_t persisting_l2_max = 0;
  std::string gpu_name;
  StreamSlot stream;
  int *d_status = nullptr;  // device status word: 0 clean, else first failure
  Options opt;
};

Context &ctx();
int ensure_ready();  // lazy init on device 0 if b200mlir_init was not called
extern std::atomic<int64_t> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int check_launch(const char *what);

// Persistent per-process workspace (grown on demand, never inside a capture).
int workspace(size_t bytes, void **out);
// Second, independent workspace for callers that hold the first.
int workspace2(size_t bytes, void **out);
// Device image of host tensors for the pipelined host-buffer GEMM, and its two copy streams.
int staging_workspace(size_t bytes, void **out);
int copy_streams(cudaStream_t *in, cudaStream_t *out);
// Workspace of the split-K GEMM variant (tile counters, then fp32 partial tiles); zero-filled when (re)allocated.
int splitk_workspace(size_t bytes, void **out);
// L2 persistence window over a resident weight image: set (raises the device's set-aside size,
// never lowers it), clear when that image goes away, and apply to the calling thread's stream.
int l2_window_set(const void *base, size_t bytes);
void l2_window_clear(const void *base);
void l2_window_apply();

// ---- programmatic dependent launch ---------------------------------------------------
// A kernel launched this way may start while its predecessor in the stream drains: its
// CTAs become resident and run up to their `pdl_wait()`, which returns once the
// predecessor has completed and its writes are visible.  Kernels call `pdl_trigger()` first
// so that their own successor can do the same.  Both are no-ops for a plain launch.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = ctx().opt.enable_pdl != 0 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
// The same for any kernel, switched by `dependent` (the GEMM kernels use option gemmDependentLaunch).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_maybe_dependent(bool dependent, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                          cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

// ---- manifest of planned matmuls (report.cu) ---------------------------------------
struct GemmArgs;
void manifest_record(const GemmArgs &g, int variant, const std::string &why);

// ---- pointer classification / host staging -------------------------------------
bool is_device_ptr(const void *p);

// ---- kernels (each returns 0 or an error code; all enqueue on ctx().stream) -------
// row_kernels.cu
int launch_softmax_f16(const __half *x, __half *y, int64_t rows, int64_t cols, int64_t ldx,
                       int64_t ldy);
int launch_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols, int64_t ldx,
                       int64_t ldy);
int launch_rmsnorm_f16(const __half *x, const __half *w, __half *y, int64_t rows, int64_t cols,
                       int64_t ldx, int64_t ldy, float eps);
int launch_rmsnorm_f32(const float *x, const float *w, float *y, int64_t rows, int64_t cols,
                       int64_t ldx, int64_t ldy, float eps);
int launch_silu_f16(const __half *x, __half *y, int64_t n);
int launch_silu_f32(const float *x, float *y, int64_t n);
int launch_swiglu_f16(const __half *g, const __half *u, __half *y, int64_t n);
int launch_add_f16(const __half *a, const __half *b, __half *y, int64_t n);
// out rows of this rank = f16(sum_w f32(recv[w]) + f32(residual)), stored to every rank's out
int launch_reduce_rows_push(const __half *recv, const __half *residual, int64_t ldres, void *const *peer_out,
                            int world, int rank, int64_t rows_per_rank, int64_t cols);

// sum over the ranks' copies of elements [offset, offset + count) of a multicast-mapped fp16 buffer, written back to every copy
int launch_allreduce_multimem(const void *mc_in, void *mc_out, int64_t elem_offset, int64_t count);
// a barrier of the ranks as its own one-warp launch (flag words in the symmetric buffer, two slots)
int launch_rank_barrier(void *const *peer_bufs, int64_t flags_elem_offset, int slot, int rank, int world, void *state);
// the same with both rendezvous of the ranks inside the launch (flag words in the buffer itself)
int launch_allreduce_multimem_sync(void *mc_buf, void *const *peer_bufs, int64_t elem_offset, int64_t count,
                                   int64_t flags_elem_offset, int rank, int world, void *state,
                                   cudaStream_t stream = nullptr,  // null: the calling thread's stream
                                   int exit_rendezvous = 1);       // 0: the caller puts a barrier after the launch

// layout.cu
int launch_transpose_i8(const int8_t *src, int8_t *dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst);
int launch_pack_weight_f16(const uint16_t *src, uint16_t *dst, int64_t k, int64_t n, int64_t ld);
int launch_pack_act_f16(const uint16_t *src, uint16_t *dst, int64_t rows, int64_t cols,
                        int64_t ld);
int launch_unpack_acc_f16(const uint16_t *tiles, uint16_t *dst, int64_t rows, int64_t cols,
                          int64_t ld);

// GEMM epilogue selector shared by every GEMM variant.
enum Epilogue : int {
  EPI_F16 = 0,        // C16 = f16(acc)
  EPI_F32_RES = 1,    // C32 = f32(f16(acc)) [+ R32]
  EPI_KLOOP_F16 = 2,  // C16 = f16(sum_seg f32(f16(acc_seg)))
  EPI_F16_RES16 = 3,  // C16 = f16(f32(f16(acc)) + f32(R16))
  EPI_SWIGLU = 4,     // B holds [Wg | Wu] interleaved per tile; C16 = swiglu
  EPI_PUSH16 = 5,     // f16(acc) stored into the row owner's receive slot on another GPU (PushTargets)
  EPI_I32 = 6         // int8 operands (B given transposed, [N,K]), C32 = the exact int32 sums
};

// Where EPI_PUSH16 stores: row r of the partial product belongs to rank r / rows_per_rank, whose
// receive buffer is [world][rows_per_rank][N] fp16; this rank writes slot `rank` of it.  The
// pointers are peer-mapped device addresses (one per rank, this rank's own included).
constexpr int kMaxPushRanks = 8;
struct PushTargets {
  void *recv[kMaxPushRanks] = {};
  int world = 0, rank = 0;
  int64_t rows_per_rank = 0;
};

struct GemmArgs {
  const void *a = nullptr;  // [M,K] row-major fp16 (int8 for the i8 path)
  const void *b = nullptr;  // [K,N] row-major
  void *c = nullptr;        // [M,N]
  const void *res = nullptr;
  const void *b2 = nullptr;  // second B operand (EPI_SWIGLU: Wu), same shape/stride as b
  int64_t m = 0, n = 0, k = 0;
  int64_t lda = 0, ldb = 0, ldc = 0, ldres = 0;
  int epilogue = EPI_F16;
  int block_k = 0;  // EPI_KLOOP_F16 only
  // EPI_F16_RES16: the residual is added only in the 256-row blocks b with b % res_mod == res_rem
  // (tensor-parallel ranks share the residual read-out: each adds it to its blocks of the partial)
  int res_mod = 1, res_rem = 0;
  // B is not row-major [K,N] but the K-blocked image [ceil(K/64)][N][64] fp16: per 64-deep k-block
  // every column's 64 values are one contiguous 128-byte row, so a CTA's operand tile of a k-block
  // is ONE contiguous piece of HBM (a row-major B hands the memory system 128-byte pieces a whole
  // row of B apart, which held DRAM at ~2.9 TB/s when every tile reads its own columns).  Built by
  // the w8a16 registry for its many-row route; `ldb` is ignored.
  bool b_kblocked = false;
  const PushTargets *push = nullptr;  // EPI_PUSH16 only
};

// gemm_simt.cu — any-shape fallback ("hmx-tail"/"hvx" plans of the reference)
int launch_gemm_simt(const GemmArgs &g);
int launch_gemm_i8_simt(const int8_t *a, const int8_t *b, int32_t *c, int64_t m, int64_t n,
                        int64_t k, int64_t lda, int64_t ldb, int64_t ldc);

// gemm_tcgen05.cu — tensor-core variants
int tc_variant_count();
struct TcVariantInfo {
  const char *name;
  int bm, bn, bk, stages, cta_group;
  int smem_bytes, tmem_cols;
  double model_eff;  // fraction of the tensor pipe this tiling sustained when measured
  bool stream_k = false;  // work is dealt out in k-blocks, not whole tiles (gemm_tcgen05_streamk.cu)
};
const TcVariantInfo &tc_variant_info(int v);
// "ok" or a refusal reason for variant v on (m,n,k) with the given epilogue.
const char *tc_variant_verdict(int v, const GemmArgs &g);
int launch_gemm_tc(int v, const GemmArgs &g);
// int8 x int8 -> int32 on the tensor cores (kind::i8); bt is B transposed, [N,K] row-major
int launch_gemm_i8_tc(const int8_t *a, const int8_t *bt, int32_t *c, int64_t m, int64_t n, int64_t k, int64_t lda,
                      int64_t ldbt, int64_t ldc);
// gemm_tcgen05_2cta.cu
int launch_gemm_i8_tc_pair(const int8_t *a, const int8_t *bt, int32_t *c, int64_t m, int64_t n, int64_t k, int64_t lda,
                           int64_t ldbt, int64_t ldc);
int launch_gemm_tc_pair(const GemmArgs &g, bool deep_k);
int pair_variant_smem_bytes();
// gemm_tcgen05_streamk.cu — the pair kernel with the k-blocks of its tiles dealt out evenly over the pairs
int launch_gemm_tc_streamk(const GemmArgs &g);
bool streamk_shape_ok(const GemmArgs &g);

// w8a16.cu
struct W8A16Weight {
  const void *src = nullptr;     // caller's row-major int8 [K,N] (identity key)
  const void *scales = nullptr;  // fp16 [N]
  void *image = nullptr;         // resident device image: [k/128][channel][128 B, pieces swizzled]
  void *scales_dev = nullptr;
  void *w16 = nullptr;           // row-major fp16 f16(q*s), built on the first many-row call (option w8a16ExpandRows)
  int64_t k = 0, n = 0;
  size_t image_bytes = 0;
  bool l2_persist = false;
};
int launch_w8a16(const __half *a, const W8A16Weight &w, __half *c, int64_t m, int64_t lda,
                 int64_t ldc);
// Above option w8a16ExpandRows activation rows (default 64) every CTA of the streaming kernel
// re-reads so many activations from L2 that it falls behind the fp16 GEMM (measured on
// 4096x11008: 96 rows 26.8 against 24.5 us, 128 rows 28.3 against 25.1; 64 rows 18.2 against
// 24.2): the weight is expanded once to fp16 (2 bytes per weight, kept with the registry entry)
// and the product goes through the fp16 GEMM.
// w8a16_tmem.cu
int w8a16_expand_f16(const void *image, const __half *scales_dev, int64_t k, int64_t n, void **w16);  // K-blocked image (GemmArgs::b_kblocked)
int w8a16_build_tmem_image(const int8_t *wq_dev, int64_t k, int64_t n, void **image, size_t *bytes);
int launch_w8a16_tmem(const __half *a, const void *image, const __half *scales_dev, int64_t k, int64_t n,
                      __half *c, int64_t m, int64_t lda, int64_t ldc);

// attention_tmem.cu — softmax(Q·Kᵀ·sm_scale)·V per (batch, head); q, k, v share one stride set
// (elements; the head dimension is contiguous), out has its own; f32 = fp32 tensors (operands are
// rounded to fp16 first), else fp16
int launch_attention(const void *q, const void *k, const void *v, void *out, bool f32, int64_t z, int64_t h,
                     int64_t n, int64_t d, int64_t sz, int64_t sh, int64_t sn, int64_t soz, int64_t soh,
                     int64_t son, double sm_scale, bool causal);

// tp_nccl.cu — the process's tensor-parallel group (NCCL bound at run time)
int tp_rank();
int tp_world();  // 1 when no group is initialised
int tp_all_gather_bytes(const void *src, void *dst, size_t bytes_per_rank, cudaStream_t s);
int tp_all_reduce_f16(void *buf, size_t count, cudaStream_t s);
int tp_comm_stream(cudaStream_t *s);
// Exchange of row slabs between the ranks by copy engines, without a kernel: every rank keeps a
// window (an A buffer and a flag word per panel and rank) that the others map through CUDA IPC; a
// rank copies its slab into every peer's buffer and then the call's sequence number into the
// peer's flag, on one stream, so the flag lands after the data.
struct SlabExchange {
  char *a = nullptr;                        // this rank's A buffer
  char *peer_a[kMaxPushRanks] = {};         // the same buffer of every rank, as this process maps it
  uint32_t *flags = nullptr;                // [panel][kMaxPushRanks], this rank's
  uint32_t *peer_flags[kMaxPushRanks] = {};
  const uint32_t *d_seq = nullptr;          // device word holding `seq` (source of the flag copies on `push`)
  uint32_t seq = 0;
  cudaStream_t push = nullptr;
};
constexpr int kExchangePanels = 16;
// Collective, called by every rank with the same `a_bytes`: waits (on the host) until every rank
// is in the call, (re)creates the windows when they are too small, and hands out this call's
// sequence number.  *x.a stays null when the machine gives no IPC mapping (the caller then
// exchanges through ncclAllGather).
int tp_slab_exchange_begin(size_t a_bytes, SlabExchange *x);
// on stream s: wait (bounded) until every other rank's flag of `panel` has reached x.seq
int tp_slab_exchange_wait(const SlabExchange &x, int panel, cudaStream_t s);

// dispatch.cpp
int gemm_dispatch(const GemmArgs &g);  // picks a variant (option / cache / heuristic) and launches
int choose_gemm_variant(const GemmArgs &g, std::string *why);  // -1 => simt fallback

}  // namespace b200
