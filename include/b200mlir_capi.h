/* b200mlir_capi.h — the C ABI of libb200mlir.so.
 *
 * A B200 (sm_100a) implementation of the operator hot path that the
 * hexagon-mlir backend lowers linalg/Triton kernels into.  Two seams of the
 * reference are answered here, with the same names, argument order and
 * argument meaning, so that a host that binds the reference's symbols can bind
 * these instead:
 *
 *   seam 1  the compiled-kernel entry points the generated wrapper calls
 *           (one (rank, descriptor*) pair per tensor, scalars by value, then
 *            num_programs x/y/z and program_id x/y/z);
 *   seam 2  the runtime the kernels call (hexagon_runtime_*).
 *
 * Plain C: pointers, sizes and integers only.  Every tensor pointer may be a
 * CUDA device pointer or an ordinary host pointer; host tensors are staged
 * through device memory inside the call (copy in, compute, copy out, wait).
 * Device tensors are processed asynchronously on the stream set with
 * b200mlir_set_stream (default: the legacy default stream).
 *
 * Errors: the reference's entry points return void and abort on failure.
 * These never abort; a failed call leaves its outputs untouched, and
 * b200mlir_last_error() returns the code and message of the most recent
 * failure on the calling thread.  There is no CPU fallback: without a usable
 * CUDA device every compute entry fails with B200MLIR_ERR_NO_DEVICE.
 *
 * Citations are file:line inside the reference project (hexagon-mlir).
 */
#ifndef B200MLIR_CAPI_H
#define B200MLIR_CAPI_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

/* ---- descriptors ---------------------------------------------------------
 * MLIR memref descriptor, every index field int64
 * (test/utils/dsp/include/common.h:15-27). */
typedef struct {
  void *allocated;
  void *aligned;
  int64_t offset;
  int64_t sizes[1];
  int64_t strides[1];
} B200MemRef1D;

typedef struct {
  void *allocated;
  void *aligned;
  int64_t offset;
  int64_t sizes[2];
  int64_t strides[2];
} B200MemRef2D;

typedef struct {
  void *allocated;
  void *aligned;
  int64_t offset;
  int64_t sizes[4];
  int64_t strides[4];
} B200MemRef4D;

enum {
  B200MLIR_OK = 0,
  B200MLIR_ERR_NO_DEVICE = 1,   /* no CUDA device / driver, or not sm_100 */
  B200MLIR_ERR_BAD_ARG = 2,     /* rank, shape, stride or pointer contract broken */
  B200MLIR_ERR_CUDA = 3,        /* a CUDA call failed; message carries the text */
  B200MLIR_ERR_SCOPE = 4,       /* resident request outside / against the scope */
  B200MLIR_ERR_DEVICE_WAIT = 5, /* a bounded device-side wait ran out */
  B200MLIR_ERR_UNSUPPORTED = 6, /* no kernel variant is legal for this request */
  B200MLIR_ERR_VERIFY = 7       /* autotune candidate produced a wrong result */
};

/* ---- library management (no counterpart in the reference: its runtime is a
 * process-wide singleton created on first use,
 * qcom_hexagon_backend/bin/runtime/include/HexagonAPI.h:47-115) ------------- */
B200_API int b200mlir_init(int device);
B200_API int b200mlir_set_stream(void *cuda_stream);
B200_API int b200mlir_synchronize(void);
B200_API int b200mlir_last_error(char *buf, int cap);
B200_API const char *b200mlir_version(void);
/* Kernels of this library launched by this process since the last reset. */
B200_API int64_t b200mlir_launch_count(void);
B200_API void b200mlir_reset_launch_count(void);
/* Status word the device kernels write when a bounded wait expires; 0 = clean.
 * Reading it synchronises the stream. */
B200_API int b200mlir_device_status(void);

/* Options, the subset of the reference's option dataclass that reaches this
 * path (qcom_hexagon_backend/backend/hexagon_options.py:16-278).  Names are
 * the reference's: "enableWeightResident", "iterations", plus
 * "rmsNormEpsilon" (a tl.constexpr in the reference kernel,
 * test/python/triton/test_rms_norm.py:17,39), "gemmVariant" (-1 = dispatcher's
 * choice), "kloopBlockK", "attentionTiles" (query tiles per CTA of the
 * attention kernel: 0 = by size, 1 or 2), "attentionSplits" (CTAs that share the keys of one
 * query tile, merged by a second kernel: 0 = by size), "attentionStage" (1 or 3, see the
 * attention entry), "w8a16ExpandRows" and "kloopPairs" (1: the K-looped matmul may take the
 * two-CTA kernel, the default; 0: one-CTA kernel only).  Returns 0, or B200MLIR_ERR_BAD_ARG for
 * an unknown name. */
B200_API int b200mlir_set_option(const char *name, double value);
B200_API int b200mlir_get_option(const char *name, double *value);

/* ---- seam 1: kernel entry points ------------------------------------------
 * Signature rule: backend/hexagon_launcher_base.py:58-60,72-74 and
 * backend/triton_hexagon_launcher.py:241-252 — tensors as (rank, descriptor*),
 * tl.constexpr parameters not passed (backend/driver.py:207-212), six trailing
 * ints.  One call computes the WHOLE problem: the instance with program id
 * (0,0,0) enqueues it and every other instance of a grid>1 launch returns at
 * once, which keeps the reference's "each program owns a row slice" contract
 * observable from outside (same bytes written once).
 */
#define B200_GRID_ARGS int num_programs_x, int num_programs_y, int num_programs_z, \
                       int pid_x, int pid_y, int pid_z

/* C[M,N] = A[M,K]·B[K,N]; fp16 in, fp32 accumulate, fp16 out; C overwritten.
 * Kernel: test/python/triton/test_matmul.py:32-72.  Engine leaves replaced:
 * qcom_hexagon_backend/bin/runtime/hmx/src/HMXAPI.c:22-55 (bias_init, acc_clear,
 * mma, acc_store) and the pack/unpack leaves of hmx/src/HMXLayout.c. */
B200_API void matmul(int64_t rank_a, B200MemRef2D *a, int64_t rank_b, B200MemRef2D *b,
                     int64_t rank_c, B200MemRef2D *c, B200_GRID_ARGS);
/* The multi-span form: the kernel tiles M and N itself (BLOCK_M x BLOCK_N spans, whole K),
 * each span stored to its own window of C with C's row stride
 * (test/python/triton/test_matmul_multispan.py:82-107).  The span sizes are tl.constexpr
 * and do not reach the ABI; one rounding per element, like `matmul`. */
B200_API void multispan_matmul(int64_t rank_a, B200MemRef2D *a, int64_t rank_b, B200MemRef2D *b,
                               int64_t rank_c, B200MemRef2D *c, B200_GRID_ARGS);
/* Same contraction with the K-segmented accumulation of a K-looped tl.dot:
 * each BLOCK_K segment is read out as fp16, widened and added in fp32
 * (test/python/triton/test_matmul_kloop.py:27-34,87-98).  BLOCK_K = option
 * "kloopBlockK" (default 64).  Multiples of 64 run on the tensor cores (one
 * accumulator per segment), other values on the CUDA-core path; same arithmetic. */
B200_API void klooped_matmul(int64_t rank_a, B200MemRef2D *a, int64_t rank_b, B200MemRef2D *b,
                             int64_t rank_c, B200MemRef2D *c, B200_GRID_ARGS);
/* fp32 read-out with optional fp32 residual: C32 = f32(f16(A·B)) [+ R]
 * (hmx_unpack_acc_f32_bulk, hmx/src/HMXLayout.c:868-999; `res` may be NULL /
 * rank 0). */
B200_API void matmul_f32out(int64_t rank_a, B200MemRef2D *a, int64_t rank_b, B200MemRef2D *b,
                            int64_t rank_c, B200MemRef2D *c32, int64_t rank_r,
                            B200MemRef2D *res32, B200_GRID_ARGS);
/* int8 x int8 -> int32, exact (the reference routes integer matmuls to exact
 * vector loops: include/hexagon/Dialect/Hmx/Transforms/HmxTarget.h:198-200).  Runs on the tensor
 * cores (tcgen05 kind::i8, over SM pairs for large problems; B transposed once into the workspace) when M, N, K >= 64, N is a
 * multiple of 4 and the rows of A and C are 16-byte multiples; otherwise on CUDA cores.  Both are
 * bit-exact. */
B200_API void matmul_i8(int64_t rank_a, B200MemRef2D *a, int64_t rank_b, B200MemRef2D *b,
                        int64_t rank_c, B200MemRef2D *c, B200_GRID_ARGS);

/* Row softmax (test/python/triton/test_softmax.py:39-70; lowered form
 * docs/tutorials/triton/softmax.md:150-226). */
B200_API void softmax_kernel_float16(int64_t rank_x, B200MemRef2D *x, int64_t rank_y,
                                     B200MemRef2D *y, B200_GRID_ARGS);
B200_API void softmax_kernel_float32(int64_t rank_x, B200MemRef2D *x, int64_t rank_y,
                                     B200MemRef2D *y, B200_GRID_ARGS);
/* RMSNorm y = x * rsqrt(mean(x^2) + eps) * w
 * (test/python/triton/test_rms_norm.py:32-60); eps = option "rmsNormEpsilon". */
B200_API void rms_norm_fwd_kernel_float16(int64_t rank_x, B200MemRef2D *x, int64_t rank_y,
                                          B200MemRef2D *y, int64_t rank_w, B200MemRef1D *w,
                                          B200_GRID_ARGS);
B200_API void rms_norm_fwd_kernel_float32(int64_t rank_x, B200MemRef2D *x, int64_t rank_y,
                                          B200MemRef2D *y, int64_t rank_w, B200MemRef1D *w,
                                          B200_GRID_ARGS);
/* SiLU x / (1 + exp(-x)) (test/python/triton/test_silu.py:38-49). */
B200_API void silu_kernel_float16(int64_t rank_x, B200MemRef1D *x, int64_t rank_y,
                                  B200MemRef1D *y, B200_GRID_ARGS);
B200_API void silu_kernel_float32(int64_t rank_x, B200MemRef1D *x, int64_t rank_y,
                                  B200MemRef1D *y, B200_GRID_ARGS);
/* Vector add (test/python/triton/test_vec_add.py), the residual-add generic. */
B200_API void add_kernel_float16(int64_t rank_x, B200MemRef1D *x, int64_t rank_y,
                                 B200MemRef1D *y, int64_t rank_o, B200MemRef1D *out,
                                 B200_GRID_ARGS);

/* Ops the reference has no kernel for; they follow the same convention and
 * are defined as the composition its lowering would produce. */
/* out = silu(gate) * up, the fused two-input elementwise generic
 * (qcom_hexagon_backend/lib/Conversion/LinalgToLLVM/FusionPass.cpp). */
B200_API void swiglu_kernel_float16(int64_t rank_g, B200MemRef1D *gate, int64_t rank_u,
                                    B200MemRef1D *up, int64_t rank_o, B200MemRef1D *out,
                                    B200_GRID_ARGS);
/* C[M,N] = A[M,K] · dequant(Wq[K,N], s[N]); Wq int8 row-major, s fp16 per
 * output channel, fp32 accumulate, fp16 out.  No reference function (HMX admits
 * f16/f32 only: include/hexagon/Dialect/Hmx/IR/HmxDType.h:59,69).  Up to 64 rows
 * (option "w8a16ExpandRows") stream the resident int8 image; a call with more rows expands the
 * weight once to fp16 (2 bytes per weight, kept until the weight is unregistered) and runs the
 * fp16 GEMM. */
B200_API void w8a16_matmul(int64_t rank_a, B200MemRef2D *a, int64_t rank_w, B200MemRef2D *wq,
                           int64_t rank_s, B200MemRef1D *scales, int64_t rank_c,
                           B200MemRef2D *c, B200_GRID_ARGS);
/* Llama-style MLP block over this rank's shard of the hidden dimension:
 *   h = rmsnorm(x, gain, eps); a = swiglu(h·Wg, h·Wu); out = a·Wd (+ x if add_residual)
 * Wg, Wu: [D, F_local]; Wd: [F_local, D].  With tensor parallelism each rank
 * passes its column block of Wg/Wu and row block of Wd, add_residual = 0, sums
 * `out` over ranks and adds x afterwards (add_kernel_float16). */
B200_API void mlp_block_float16(int64_t rank_x, B200MemRef2D *x, int64_t rank_gain,
                                B200MemRef1D *gain, int64_t rank_wg, B200MemRef2D *wg,
                                int64_t rank_wu, B200MemRef2D *wu, int64_t rank_wd,
                                B200MemRef2D *wd, int64_t rank_o, B200MemRef2D *out,
                                float eps, int add_residual, B200_GRID_ARGS);
/* The same block with the reduction over ranks fused in, for `world` GPUs of one node whose
 * buffers are mapped into each other's address space (peer access / symmetric memory).  The
 * down projection's read-out stores this rank's fp16 partial rows straight into the receive
 * buffer of the rank that owns them: row r belongs to rank r / (T/world), whose buffer is
 * [world][T/world][D] fp16 and is filled at slot `rank`; peer_recv[i] is rank i's buffer as
 * mapped here.  After every rank's call has completed (a barrier the caller provides),
 * b200mlir_tp_reduce_rows_float16 sums the owner's `world` slots, adds the residual rows and
 * stores the finished rows into every rank's [T][D] output (peer_out[i]); after a second
 * barrier all ranks hold the block output.  No reference counterpart (the reference is a
 * single device); it replaces the all-reduce of the tensor-parallel form above.  Needs T
 * divisible by world, world <= 8, D a multiple of 8. */
B200_API void mlp_block_push_float16(int64_t rank_x, B200MemRef2D *x, int64_t rank_gain, B200MemRef1D *gain,
                                     int64_t rank_wg, B200MemRef2D *wg, int64_t rank_wu, B200MemRef2D *wu,
                                     int64_t rank_wd, B200MemRef2D *wd, void *const *peer_recv, int world,
                                     int rank, float eps, B200_GRID_ARGS);
B200_API int b200mlir_tp_reduce_rows_float16(const void *recv, const void *residual_rows, int64_t ld_residual,
                                             void *const *peer_out, int world, int rank, int64_t rows_per_rank,
                                             int64_t cols);

/* Tensor-parallel group of this process (one process per GPU; NCCL over NVLink, bound at run
 * time: on a machine without libnccl.so.2 these fail with B200MLIR_ERR_UNSUPPORTED and everything
 * else works).  Rank 0 obtains 128 bytes with b200mlir_tp_unique_id and hands them to the other
 * ranks by any means (a file, a pipe, a socket, MPI); every rank then calls
 * b200mlir_tp_init(id, rank, world) once, after b200mlir_init.  b200mlir_tp_info returns 1 and the
 * rank / world when a group exists, 0 (rank 0 of 1) otherwise.  No counterpart in the reference,
 * which drives one device. */
B200_API int b200mlir_tp_unique_id(void *id128);
B200_API int b200mlir_tp_init(const void *id128, int rank, int world);
B200_API int b200mlir_tp_info(int *rank, int *world);
B200_API int b200mlir_tp_shutdown(void);
/* How the last host-buffer GEMM under option replicatedOperandA exchanged the row slabs of A
 * between the ranks: 0 none yet, 1 copy engines writing into windows the ranks map from one
 * another through CUDA IPC (a flag word per panel and rank follows each slab), 2 ncclAllGather
 * (where the machine gives no such mapping, or B200MLIR_SLAB_EXCHANGE=nccl is set). */
B200_API int b200mlir_tp_slab_exchange_mode(void);
/* In-place sum over the group of `count` fp16 elements at the device address `buf`
 * (ncclAllReduce on the calling thread's stream). */
B200_API int b200mlir_tp_all_reduce_float16(void *buf, int64_t count);
/* The MLP block, tensor-parallel, reduction included: each rank passes its column block of Wg / Wu
 * and its row block of Wd (as for mlp_block_float16) and the same x; on return (in stream order)
 * every rank's `out` holds x + down(swiglu(gate(h), up(h))).  Every rank's partial carries the
 * residual of its share of the 256-row blocks (block b: rank b mod world), the partials are summed
 * in place with one ncclAllReduce per token chunk; `chunks` > 1 cuts the down projection into token chunks (whole 256-row tiles) and runs the all-reduce of a
 * chunk on a second stream while the next chunk's GEMM is computed.  x and out
 * are device tensors, out dense.  Without a group it is mlp_block_float16 with the residual.  A
 * collective call: every rank of the group must make it, with the same T, D and chunks. */
B200_API void mlp_block_tp_float16(int64_t rank_x, B200MemRef2D *x, int64_t rank_gain, B200MemRef1D *gain,
                                   int64_t rank_wg, B200MemRef2D *wg, int64_t rank_wu, B200MemRef2D *wu,
                                   int64_t rank_wd, B200MemRef2D *wd, int64_t rank_o, B200MemRef2D *out,
                                   float eps, int chunks, B200_GRID_ARGS);
/* The same block with the sum over ranks done by this library's own kernel through the NVSwitch's
 * multicast addresses and overlapped with the math, one fused call: `out` is this rank's dense
 * [T, D] view at the START of a symmetric fp16 buffer, `mc_buf` that buffer's multicast address,
 * `peer_bufs[r]` the address of rank r's copy (peer_bufs[rank] == out's data), `flags_elem_offset` (>= T*D) the element at which the buffer holds 16 zero-initialised flag
 * words, `state` FOUR zero-initialised 32-bit words of this rank's device memory (as for
 * b200mlir_tp_allreduce_multimem_sync_float16 and b200mlir_tp_barrier).  With one chunk the block
 * ends with b200mlir_tp_barrier, the plain multicast all-reduce and a second barrier.  The down projection is cut into `chunks` token
 * chunks (whole 256-row tiles whose rows divide over the ranks, else one chunk); a chunk's
 * all-reduce is launched on a second stream as soon as its GEMM has been issued and runs beside
 * the next chunk's GEMM on the same SMs.  Tokens divisible by the world size.  A collective call:
 * every rank makes it with the same T, D and chunks.  No reference counterpart (single device). */
B200_API void mlp_block_tp_multicast_float16(int64_t rank_x, B200MemRef2D *x, int64_t rank_gain, B200MemRef1D *gain,
                                             int64_t rank_wg, B200MemRef2D *wg, int64_t rank_wu, B200MemRef2D *wu,
                                             int64_t rank_wd, B200MemRef2D *wd, int64_t rank_o, B200MemRef2D *out,
                                             void *mc_buf, void *const *peer_bufs, int64_t flags_elem_offset,
                                             void *state, int rank, int world, float eps, int chunks,
                                             B200_GRID_ARGS);

/* This rank's share of an all-reduce through NVSwitch multicast (NVLS): `mc_in` / `mc_out` are
 * MULTICAST addresses of fp16 buffers that every rank of the group holds (the symmetric-memory
 * mapping the host obtained for them; they may be the same buffer).  Elements
 * [elem_offset, elem_offset + count) are summed over all ranks' copies inside the switch (fp32
 * accumulation, one rounding) and the sums are written to every rank's copy.  Each rank calls it
 * for its own disjoint slice after a barrier that follows the producers of the data, and a second
 * barrier makes the result visible everywhere; the barriers are the caller's.  Offsets and counts
 * in elements, multiples of 8.  No reference counterpart (single device). */
B200_API int b200mlir_tp_allreduce_multimem_float16(const void *mc_in, void *mc_out, int64_t elem_offset,
                                                    int64_t count);
/* A barrier of the ranks as a one-warp launch on the calling thread's stream: rank r's flag word
 * [slot * 8 + rank] in every peer's copy of a symmetric buffer (16 flag words at element
 * `flags_elem_offset`, zero before the first call; `peer_bufs[r]` = rank r's copy as this process
 * maps it) is set with a release store over NVLink, the local words are polled (bounded: device
 * status site 49 with the late rank).  `slot` is 0 or 1 (the barrier before and the one after an
 * all-reduce use different words); `state` is FOUR zero-initialised 32-bit words of this rank's
 * device memory shared with b200mlir_tp_allreduce_multimem_sync_float16 (words 2 and 3 are the
 * barriers' launch numbers), so the call can be replayed from a captured graph.  Every rank issues
 * the same sequence of barriers.  No reference counterpart (single device). */
B200_API int b200mlir_tp_barrier(void *const *peer_bufs, int64_t flags_elem_offset, int slot, int rank, int world,
                                 void *state);
/* The same, in place, with both rendezvous inside the launch: `mc_buf` is the multicast address
 * of ONE symmetric fp16 buffer and `peer_bufs[r]` the address of rank r's copy as this process
 * maps it (peer_bufs[rank] is this rank's own); the buffer also holds 16 flag words (64 bytes, zero
 * before the first call) at element `flags_elem_offset`; `state` is two zero-initialised 32-bit
 * words of this rank's device memory that the calls keep between them.  Every rank of the group
 * issues the call once per all-reduce, in the same order, after the producer of its copy on the
 * same stream.  The launch tells every peer (a release store into its flag words over NVLink) that
 * this rank's copy is complete, waits (each wait bounded to about a second, then device status
 * B200MLIR_ERR_DEVICE_WAIT site 48 with the late rank) until every rank's is, sums this rank's
 * slice, and ends only when every rank's sums are in this rank's copy and no rank still reads
 * it.  With `exit_rendezvous` = 0 the launch ends after this rank's sums are issued and the
 * caller puts a barrier of its own after it (the rendezvous at the end costs a system-scope fence
 * per CTA; a barrier kernel in a graph measured cheaper).  The flag epoch lives on the device, so
 * the call can be replayed from a captured graph.  No reference counterpart (single device). */
B200_API int b200mlir_tp_allreduce_multimem_sync_float16(void *mc_buf, void *const *peer_bufs, int64_t elem_offset,
                                                         int64_t count, int64_t flags_elem_offset, int rank,
                                                         int world, void *state, int exit_rendezvous);

/* Phase times of the most recent MLP block issued by the calling thread while option
 * "mlpPhaseTiming" was non-zero: microseconds of RMSNorm, gate/up GEMM (SwiGLU read-out), down
 * GEMM and — tensor-parallel entry with one chunk — the all-reduce, from CUDA events recorded
 * between the phases.  Returns how many were written (0 when none were recorded, -1 on error); synchronises
 * with the last phase.  The analogue of the reference's per-region cycle counts
 * (qcom_hexagon_backend/lib/Transforms/HexagonLWPInstrumentation.cpp). */
B200_API int b200mlir_mlp_phase_times(double *us, int cap);

/* The two-phase ("online") softmax of test/python/triton/test_online_softmax.py:27-77, fp32 rows:
 * running maximum and running sum over column blocks, then exp(x - m) / l.  The block sizes are
 * tl.constexpr there and do not change the result beyond fp32 round-off (the test's tolerance is
 * 1e-5 against a plain softmax), so this entry runs the row-softmax kernel: one pass, row in
 * registers.  The symbol has no dtype suffix because the reference kernel has none. */
B200_API void online_softmax(int64_t rank_x, B200MemRef2D *x, int64_t rank_y, B200MemRef2D *y, B200_GRID_ARGS);

/* Attention block, softmax(Q·K^T·sm_scale)·V per (batch, head): the reference's flash-attention
 * kernel (test/python/triton/test_flash_attention.py:116-195, loop over key blocks :43-113;
 * launched at :198-236).  Q, K, V, Out are [Z, H, N_CTX, D_HEAD] with the head dimension
 * contiguous; Q, K and V share one stride set as in the reference (:31-34), Out may have its own.
 * sm_scale is a tl.constexpr in the reference kernel and an argument here; it must be positive.
 * Both products take fp16 operands with fp32 accumulation (the float32 entry rounds Q, K, V to
 * fp16 first, as the engine's pack leaf does, :239-246); the running maximum, the row sums and
 * the output accumulator are fp32.  D_HEAD is 64 or 128, strides multiples of 8 elements, any
 * N_CTX (a short last key block is masked).  Option "attentionStage" is the kernel's STAGE
 * constexpr (:183-185): 1, the default and the only form the reference's loop implements, lets
 * every query see every key; 3 is causal (query i sees keys 0..i; key blocks past the diagonal
 * are skipped).  The causal form is UNPINNED: the reference declares STAGE = 3 but has no
 * implementation of it, so there is no reference output to compare with; it is checked against a
 * plain masked softmax only. */
B200_API void attention_fwd_kernel_float16(int64_t rank_q, B200MemRef4D *q, int64_t rank_k, B200MemRef4D *k,
                                           int64_t rank_v, B200MemRef4D *v, int64_t rank_o, B200MemRef4D *out,
                                           float sm_scale, B200_GRID_ARGS);
B200_API void attention_fwd_kernel_float32(int64_t rank_q, B200MemRef4D *q, int64_t rank_k, B200MemRef4D *k,
                                           int64_t rank_v, B200MemRef4D *v, int64_t rank_o, B200MemRef4D *out,
                                           float sm_scale, B200_GRID_ARGS);

/* ---- seam 2: runtime ---------------------------------------------------------
 * qcom_hexagon_backend/bin/runtime/include/HexagonCAPI.h:26-68.  `isVtcm`
 * selected the 8 MiB on-chip scratch on Hexagon; here every allocation is HBM
 * and the flag is accepted and ignored.  Alignment: any power of two up to 2048
 * (tile buffers ask for 2048).  alloc never returns NULL for a valid request on
 * a working device; on failure it returns NULL and records the error instead of
 * aborting the process.
 * alloc_2d is the indirect-tensor form (bin/runtime/src/HexagonCAPI.cpp:89-94,
 * src/HexagonBuffer.cpp:89-113): one device allocation of numBlocks blocks at a
 * stride of blockSize rounded up to the alignment, and the RETURN VALUE IS A
 * TABLE of numBlocks block addresses (table[i] = block i), not the storage.  The
 * table is pinned host memory mapped into the device's address space: host code
 * and kernels may both index it.  free_2d takes the table and releases both. */
B200_API void *hexagon_runtime_alloc_1d(size_t bytes, uint64_t alignment, bool isVtcm);
B200_API void hexagon_runtime_free_1d(void *ptr);
B200_API void *hexagon_runtime_alloc_2d(size_t numBlocks, size_t blockSize, uint64_t alignment,
                                        bool isVtcm);
B200_API void hexagon_runtime_free_2d(void *ptr);
B200_API void hexagon_runtime_copy(void *dst, void *src, size_t nbytes, bool isDstVtcm,
                                   bool isSrcVtcm);
/* Tile-pointer alias of a contiguous buffer (HexagonCAPI.h:34-37; impl
 * bin/runtime/src/HexagonCAPI.cpp:113-126).  build_crouton returns a device table of
 * nbytes/2048 pointers, entry i = source + i*2048 (nbytes must be a positive multiple of 2048,
 * otherwise NULL with the error recorded, where the reference asserts);
 * get_contiguous_memref maps such a table back to its source, NULL for any other pointer.
 * The table is released with hexagon_runtime_free_1d, which leaves the source untouched. */
B200_API void *hexagon_runtime_build_crouton(void *source, size_t nbytes);
B200_API void *hexagon_runtime_get_contiguous_memref(void *source);
/* Residency (HexagonCAPI.h:39-57; impl bin/runtime/src/HexagonCAPI.cpp:132-206).
 * One immutable scope per process; requests before scope entry fail; a weight
 * is identified by its source address and exact (bytes, alignment) descriptor
 * and the same device address is returned on every later request.  The
 * resident copy of a weight is a device buffer that stays allocated until the
 * process exits. */
B200_API int32_t hexagon_runtime_resident_scope_enter_v2(uint64_t scopeLow64, uint64_t scopeHigh64);
B200_API void *hexagon_runtime_workspace_resident_v2(uint64_t key, uint32_t bytes,
                                                     uint32_t alignment, uint32_t instance);
B200_API void *hexagon_runtime_weight_resident_v2(uint64_t src, uint32_t bytes, uint32_t alignment);
B200_API void *hexagon_runtime_weight_resident_ddr_v2(uint64_t src, uint32_t bytes,
                                                      uint32_t alignment);
B200_API int32_t hexagon_runtime_resident_free_v2(void *ptr, uint32_t bytes);
/* Engine lock (HexagonCAPI.h:59-68).  SMs are not a single locked engine;
 * kept so that compiled callers link, and they do nothing. */
B200_API void hexagon_runtime_hmx_ensure(void);
B200_API void hexagon_runtime_hmx_unlock(void);
/* ---- seam 2: the engine and layout leaves ---------------------------------------------------
 * The 29 leaves of qcom_hexagon_backend/bin/runtime/hmx/include/HMXAPI.h:53-293 (table
 * include/hexagon/Conversion/HmxToLLVM/HmxLeafSignatures.h:85-137) under their own names, with
 * the reference's argument order and meaning.  One deviation: the reference passes every buffer
 * as a 32-bit address (HMXAPI.h:11-15); here the ADDRESS arguments are uintptr_t and carry 64-bit
 * DEVICE addresses (a host address is refused with an error).  Each leaf enqueues a small kernel
 * on the calling thread's stream.  Tile image: element (r, c) of a 32 x 32 fp16 tile at byte
 * 128*(r>>1) + 4*c + 2*(r&1) (hmx/src/HMXLayout.c:9-14).  Engine leaves act on one 32 x 32
 * accumulator (fp32 here) and four bias sets: acc_clear; mma adds n_croutons activation tiles
 * times weight tiles (consecutive 2 KiB tiles at act_addr / wt_addr); acc_store converts with the
 * loaded set (scale, output bias; bias_init_unit writes the identity), writes one fp16 tile and
 * clears the accumulator.  Packs read a row-major source (the _T forms a row-major [n][k]
 * transpose input), zero-fill what is out of range, round an f32 source to fp16 after "+0.0";
 * the bulk forms cover consecutive tiles at dst_addr + t*2048; the tail forms read only
 * valid_rows x valid_cols of the tile.  Unpacks write rows tile_row*32 + 2*block_j, +1 (bulk:
 * n_pairs pairs from 0) of a row of read-out tiles; the f32 forms widen exactly and add an f32
 * residual when has_res is non-zero.  The library's own GEMM kernels do not call these: TMA's
 * swizzle, tcgen05 with TMEM accumulators and the fused read-out take their place there. */
B200_API void hmx_bias_init_unit_f16(uintptr_t bias_addr);
B200_API void hmx_bias_load_f16(uintptr_t bias_addr, unsigned set);
B200_API void hmx_acc_clear_f16(void);
B200_API void hmx_acc_store_f16(uintptr_t dst_addr, unsigned set);
B200_API void hmx_mma_f16(uintptr_t act_addr, uintptr_t wt_addr, unsigned n_croutons);
B200_API void hmx_pack_act_f16(uintptr_t dst_addr, uintptr_t src_addr, unsigned src_rows, unsigned src_cols,
    unsigned src_stride, unsigned tile_row, unsigned tile_col);
B200_API void hmx_pack_weight_f16(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n, unsigned
    src_stride, unsigned k_tile, unsigned n_tile);
B200_API void hmx_pack_act_f16_bulk(uintptr_t dst_addr, uintptr_t src_addr, unsigned src_rows, unsigned
    src_cols, unsigned src_stride, unsigned tile_row, unsigned tile_col_start, unsigned n_col_tiles);
B200_API void hmx_pack_weight_f16_bulk(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n,
    unsigned src_stride, unsigned k_tile_start, unsigned n_tile, unsigned n_k_tiles);
B200_API void hmx_pack_act_f32(uintptr_t dst_addr, uintptr_t src_addr, unsigned src_rows, unsigned src_cols,
    unsigned src_stride, unsigned tile_row, unsigned tile_col);
B200_API void hmx_pack_weight_f32(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n, unsigned
    src_stride, unsigned k_tile, unsigned n_tile);
B200_API void hmx_pack_act_f32_bulk(uintptr_t dst_addr, uintptr_t src_addr, unsigned src_rows, unsigned
    src_cols, unsigned src_stride, unsigned tile_row, unsigned tile_col_start, unsigned n_col_tiles);
B200_API void hmx_pack_weight_f32_bulk(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n,
    unsigned src_stride, unsigned k_tile_start, unsigned n_tile, unsigned n_k_tiles);
B200_API void hmx_pack_weight_f16_T(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n, unsigned
    src_stride, unsigned k_tile, unsigned n_tile);
B200_API void hmx_pack_weight_f16_T_bulk(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n,
    unsigned src_stride, unsigned k_tile_start, unsigned n_tile, unsigned n_k_tiles);
B200_API void hmx_pack_weight_f32_T(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n, unsigned
    src_stride, unsigned k_tile, unsigned n_tile);
B200_API void hmx_pack_weight_f32_T_bulk(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n,
    unsigned src_stride, unsigned k_tile_start, unsigned n_tile, unsigned n_k_tiles);
B200_API void hmx_pack_act_tail_f16(uintptr_t dst_addr, uintptr_t src_addr, unsigned src_rows, unsigned
    src_cols, unsigned src_stride, unsigned tile_row, unsigned tile_col, unsigned valid_rows, unsigned
    valid_cols);
B200_API void hmx_pack_weight_tail_f16(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n,
    unsigned src_stride, unsigned k_tile, unsigned n_tile, unsigned valid_rows, unsigned valid_cols);
B200_API void hmx_pack_act_tail_f32(uintptr_t dst_addr, uintptr_t src_addr, unsigned src_rows, unsigned
    src_cols, unsigned src_stride, unsigned tile_row, unsigned tile_col, unsigned valid_rows, unsigned
    valid_cols);
B200_API void hmx_pack_weight_tail_f32(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n,
    unsigned src_stride, unsigned k_tile, unsigned n_tile, unsigned valid_rows, unsigned valid_cols);
B200_API void hmx_pack_weight_tail_f16_T(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n,
    unsigned src_stride, unsigned k_tile, unsigned n_tile, unsigned valid_rows, unsigned valid_cols);
B200_API void hmx_pack_weight_tail_f32_T(uintptr_t dst_addr, uintptr_t src_addr, unsigned k, unsigned n,
    unsigned src_stride, unsigned k_tile, unsigned n_tile, unsigned valid_rows, unsigned valid_cols);
B200_API void hmx_unpack_acc_f16(uintptr_t dst_addr, uintptr_t src_ar_addr, unsigned dst_rows, unsigned
    dst_cols, unsigned dst_stride, unsigned tile_row, unsigned block_j);
B200_API void hmx_unpack_acc_f16_bulk(uintptr_t dst_addr, uintptr_t src_ar_addr, unsigned dst_rows, unsigned
    dst_cols, unsigned dst_stride, unsigned tile_row, unsigned n_pairs);
B200_API void hmx_unpack_acc_f32(uintptr_t dst_addr, uintptr_t res_addr, unsigned has_res, uintptr_t
    src_ar_addr, unsigned dst_rows, unsigned dst_cols, unsigned dst_stride, unsigned res_stride, unsigned
    tile_row, unsigned block_j);
B200_API void hmx_unpack_acc_f32_bulk(uintptr_t dst_addr, uintptr_t res_addr, unsigned has_res, uintptr_t
    src_ar_addr, unsigned dst_rows, unsigned dst_cols, unsigned dst_stride, unsigned res_stride, unsigned
    tile_row, unsigned n_pairs);
B200_API void hmx_unpack_acc_tail_f16(uintptr_t dst_addr, uintptr_t src_ar_addr, unsigned dst_rows, unsigned
    dst_cols, unsigned dst_stride, unsigned tile_row, unsigned block_j, unsigned valid_rows, unsigned
    valid_cols);
B200_API void hmx_unpack_acc_tail_f32(uintptr_t dst_addr, uintptr_t res_addr, unsigned has_res, uintptr_t
    src_ar_addr, unsigned dst_rows, unsigned dst_cols, unsigned dst_stride, unsigned res_stride, unsigned
    tile_row, unsigned block_j, unsigned valid_rows, unsigned valid_cols);

/* Read-out executor (bin/runtime/include/HmxVectorExecutor.h:86-156): a resident host thread
 * runs `fn` on groups of accumulator rows while the calling thread continues.  The descriptor has
 * the reference's six fields in its order (pointers are 64-bit here, so 32 bytes instead of 24).
 * configure returns 0, -1 (fn is NULL), -2 (numThreads other than 1 was asked for; one thread is
 * used and the executor works), -3 (the thread would not start).  publish has one producer, never
 * blocks and returns the number of batches accepted: fewer than `count` only when the 16-slot ring
 * (15 usable) is full — THE CALLER MUST READ OUT THE REST ITSELF — and 0 before configure or after
 * shutdown.  `fn` is called once per batch (count = 1), in publish order.  drain returns when every
 * accepted batch has been read out; shutdown drains and releases the thread.  Inside this
 * library's own GEMM kernels the split these calls implement is done by the epilogue warps. */
typedef struct {
  uint32_t rowStart;  /* first m-row in `ar` */
  uint32_t rowCount;  /* rows in the group (G) */
  uint32_t validRows; /* rows valid in the last row of the group */
  uint32_t nCroutons; /* n-tiles per row */
  void *ar;           /* accumulator array */
  void *dst;          /* row-major destination, already offset to rowStart */
} B200HmxReadoutBatch;
typedef void (*B200HmxReadoutFn)(const B200HmxReadoutBatch *batch, uint32_t count);
#define B200_HMX_EXEC_OK 0
#define B200_HMX_EXEC_ERR_NULL_FN (-1)
#define B200_HMX_EXEC_ERR_THREADS (-2)
#define B200_HMX_EXEC_ERR_CREATE (-3)
B200_API int32_t hexagon_runtime_hmx_exec_configure(B200HmxReadoutFn fn, int32_t numThreads);
B200_API uint32_t hexagon_runtime_hmx_exec_publish(const B200HmxReadoutBatch *batches, uint32_t count);
B200_API void hexagon_runtime_hmx_exec_drain(void);
B200_API void hexagon_runtime_hmx_exec_shutdown(void);
/* Batches the executor thread has run since the library was loaded (diagnostic counter, the
 * `batchesRun` of the reference's executor). */
B200_API uint64_t b200mlir_hmx_exec_batches_run(void);
/* Asynchronous copies (bin/runtime/include/RuntimeDMA.h:39-51).  A refused
 * start returns 0xFFFFFFFF and sets *status = -1; waiting on that token
 * returns at once.  Strides, width in bytes. */
B200_API uint32_t hexagon_runtime_dma_start(void *src, int srcAS, void *dst, int dstAS,
                                            uint32_t length, bool bypassCacheSrc,
                                            bool bypassCacheDst, int *status);
B200_API uint32_t hexagon_runtime_dma2d_start(void *src, int srcAS, void *dst, int dstAS,
                                              uint32_t width, uint32_t height,
                                              uint32_t srcStride, uint32_t dstStride,
                                              bool bypassCacheSrc, bool bypassCacheDst,
                                              bool isOrdered, uint32_t cacheAllocationPolicy,
                                              int *status);
B200_API void hexagon_runtime_dma_wait(uint32_t token);

/* Contract of a registered weight (explicit, or implicit through w8a16_matmul while option
 * "enableWeightResident" is 1, the default): the library identifies the weight by its SOURCE
 * ADDRESS, as the reference's runtime does (bin/runtime/src/HexagonCAPI.cpp:167-169, no content
 * hash).  From registration until b200mlir_w8a16_unregister_weight the bytes at that address must
 * not change and the buffer must stay alive: a buffer freed and re-used for another [K,N] weight,
 * or updated in place, would be multiplied with the stale image.  Unregister before freeing or
 * rewriting a weight (or call with enableWeightResident = 0, which builds and drops the image per
 * call).  The scales are re-read whenever a call passes a different scales pointer. */
/* ---- weight residency for the GEMMs (replaces the host packer
 * qcom_hexagon_backend/backend/hmx_weight_prepack.py:124-212 and
 * WeightResidentPass, lib/Dialect/Hmx/Transforms/WeightResidentPass.cpp:9-93).
 * Registers a [K,N] int8 weight + fp16 scales by source address: the first
 * call builds the pre-swizzled device image once; later w8a16_matmul calls
 * with the same Wq pointer use it without touching the row-major source.
 * Returns 0 or an error code.  `l2_persist` != 0 also asks for an L2
 * persistence window over the image for decode-shaped calls. */
B200_API int b200mlir_w8a16_register_weight(const void *wq, const void *scales, int64_t k,
                                            int64_t n, int l2_persist);
B200_API int b200mlir_w8a16_unregister_weight(const void *wq);
/* w8a16 GEMM that never allocates.  It has no counterpart in the reference.
 *
 * Who needs it: a host that may not call cudaMalloc where it calls this
 * library — an inference server that reserved all device memory up front and
 * treats any later allocation as a fault, a plugin living inside another
 * runtime's memory pool, or code on a latency-critical thread where the
 * implicit synchronisation of cudaMalloc/cudaFree is not acceptable.
 * w8a16_matmul builds and keeps device images of the weights it meets (and its
 * many-row route allocates workspaces); this entry takes a caller-built image
 * and keeps the fp32 partial sums of its split-K kernel in a fixed 4 MiB array
 * inside the library image (every GPU that loads the library holds it until the
 * process exits).
 *
 * Limits: 1 <= M <= 64 and 1 <= N <= 16384 (M*N floats of scratch); larger
 * shapes are rejected with B200MLIR_ERR_UNSUPPORTED.  K and lda multiples of
 * 8; `a` and `image` 16-byte aligned.  All pointers are DEVICE pointers owned
 * by the caller; `cuda_stream` is the stream to enqueue on (NULL = default).
 *
 * `image` is the pre-swizzled weight, (ceil(N/32) * ceil(K/16) * 512) bytes
 * laid out [strip = n/32][kstep = k/16][lane 0..31][16 bytes]: with g = lane/4,
 * t = lane%4, byte 4*j + e (j, e in 0..3) holds q[k][n] + 128 for
 * n = 32*strip + 8*j + g and k = 16*kstep + {2t, 2t+1, 2t+8, 2t+9}[e]; positions
 * outside [K, N] hold 128.  `scales` is fp16 [N]; C = f16(sum * scales[n]).
 *
 * The first call on each device looks up the array's device address and sets
 * kernel attributes; make that first call before any stream capture begins.
 * Every call uses the same array: it is cleared at the start of each call, and
 * two calls that overlap on the GPU (different streams, or two threads) race
 * on it and corrupt each other's sums — serialise them.  The partial sums of a
 * column are added with atomic adds in the order the CTAs arrive, so the fp32
 * sum order — and with it the last bit of a result — can differ from call to
 * call; results agree with w8a16_matmul within the w8a16 tolerance (1e-2), not
 * bit for bit.
 * Returns 0 or an error code (message through b200mlir_last_error). */
B200_API int b200mlir_w8a16_matmul_static_scratch(const void *a, int64_t lda, const void *image,
                                                  const void *scales, void *c, int64_t ldc,
                                                  int64_t m, int64_t n, int64_t k,
                                                  void *cuda_stream);
/* Row-major fp16 [K,N] -> the reference's weight tile image [Nt,Kt,16,32,2]
 * and back-compatible activation/accumulator images (device or host pointers).
 * (hmx_pack_weight_f16_bulk / hmx_pack_act_f16_bulk / hmx_unpack_acc_f16_bulk,
 * hmx/include/HMXAPI.h:81-106,231-262) */
B200_API int b200mlir_pack_weight_f16(const void *src, void *dst, int64_t k, int64_t n,
                                      int64_t src_stride);
B200_API int b200mlir_pack_act_f16(const void *src, void *dst, int64_t rows, int64_t cols,
                                   int64_t src_stride);
B200_API int b200mlir_unpack_acc_f16(const void *tiles, void *dst, int64_t rows, int64_t cols,
                                     int64_t dst_stride);

/* ---- dispatch and tile search (replaces
 * qcom_hexagon_backend/backend/hmx_search.py and the legality predicate
 * include/hexagon/Dialect/Hmx/Transforms/HmxTarget.h:195-222,341-383) --------- */
/* Number of hand-written GEMM variants and a JSON description of variant i. */
B200_API int b200mlir_gemm_variant_count(void);
B200_API int b200mlir_gemm_variant_info(int variant, char *json, int cap);
/* Verdict of one variant on one shape: "ok" or a rejection reason
 * ("min-rows", "tile-alignment", "smem-budget", "tmem-budget", ...).  Returns
 * 1 when legal, 0 when refused, <0 on a bad variant index. */
B200_API int b200mlir_gemm_variant_verdict(int variant, int64_t m, int64_t n, int64_t k,
                                           char *reason, int cap);
/* JSON record of what the dispatcher would run for this shape and why
 * (plan / reason vocabulary of
 * include/hexagon/Dialect/Hmx/Transforms/HmxManifest.h:81-100). */
B200_API int b200mlir_gemm_explain(int64_t m, int64_t n, int64_t k, char *json, int cap);
/* How `matmul` treats an fp16 GEMM whose three tensors are host memory: returns 1 when it is cut
 * into row panels of A and column panels of B that go up, are multiplied and come back down
 * concurrently (panels4 = {panel rows, panel columns, row panels, column panels}; edges on
 * multiples of 256, at most 16 panels each way), 0 when it is staged whole (small problems, or
 * K or N not a multiple of 8).  Pure: needs no device. */
B200_API int b200mlir_host_gemm_plan(int64_t m, int64_t n, int64_t k, int64_t *panels4);
/* Search the variant list for one shape on the current device: enumerate,
 * refuse illegal ones, order by modelled lower bound, measure each with one
 * discarded launch + timed launches (3 repetitions, q50/q20/q80), verify the
 * first repetition against `expected` checks, crown only past max(3*CV, 15%),
 * void the round if the canary drifted.  Result cached by (M,N,K,dtype,gpu,
 * build).  Writes a JSON report; returns the champion variant or <0. */
B200_API int b200mlir_gemm_autotune(int64_t m, int64_t n, int64_t k, char *json, int cap);
/* The verdict stage alone, on measurements supplied by the caller instead of
 * the device — the reference tests its search loop the same way, with a fake
 * launcher (qcom_hexagon_backend/test/test_hmx_search_loop_contract.py:134-158).
 * times_us[3*v + {0,1,2}] = {q50, q20, q80} of variant v (a non-finite or
 * non-positive q50 means the candidate failed); canary = {q50, q20, q80} or
 * NULL; canary_reference_q50 <= 0 or NaN = no reference yet.  Returns the
 * champion variant or -1. */
B200_API int b200mlir_gemm_search_scripted(int64_t m, int64_t n, int64_t k, const double *times_us,
                                           int n_variants, int control_variant,
                                           const double *canary, double canary_reference_q50,
                                           char *json, int cap);
B200_API int b200mlir_autotune_cache_load(const char *path);
B200_API int b200mlir_autotune_cache_save(const char *path);
B200_API void b200mlir_autotune_cache_clear(void);

/* Benchmark protocol of the generated wrapper
 * (backend/hexagon_launcher_base.py:114-159;
 * test/utils/dsp/include/hexagon_benchmark.h:57-72): the caller's thunk is run
 * once and discarded, then `iterations` times between two CUDA events on the
 * library's stream.  *mean_us receives the mean per call. */
typedef void (*b200mlir_thunk)(void *user);
B200_API int b200mlir_benchmark(b200mlir_thunk fn, void *user, int iterations, double *mean_us);

/* The generated wrapper's timed section together with its report
 * (backend/hexagon_launcher_base.py:153-192): one discarded call, `iterations` timed
 * calls, then perf.txt at `path` (NULL: no file) — the Test_Info block of
 * test/utils/dsp/include/test_report.h:43-66 followed by "PerfPcycles:<n>", both from
 * the same pass, which backend/hmx_search.py:1074-1092 parses.  Cycles are SM clock
 * cycles per call (two stamps on the stream; time x rated clock if they land on
 * different SMs). */
B200_API int b200mlir_benchmark_report(b200mlir_thunk fn, void *user, int iterations, const char *name,
                                       const char *path, double *mean_us, long long *mean_cycles);
/* result: 0 Pass, 1 Fail, other Unknown; cycles < 0 omits the PerfPcycles line. */
B200_API int b200mlir_perf_report_save(const char *path, const char *name, double perf, const char *units,
                                       int result, long long cycles);

/* Synthetic inputs for the harness: fills `dst` (device or host pointer; n elements of dtype id
 * 1 = float16, 2 = float32, 4 = int8, the ids of the raw tensor files below) from a counter-based
 * generator (Philox4x32-10 keyed by `seed`; element i is drawn from its index alone).  dist 0:
 * uniform [p0, p1); 1: normal(mean p0, sigma p1) as a sum of twelve uniforms (tails end at six
 * sigma); 2: integers uniform in [p0, p1].  The same stream is implemented on the CPU beside the
 * oracle, so a CPU check and this library see identical bytes for one seed.  No counterpart in
 * the reference, whose tests draw their inputs in Python. */
B200_API int b200mlir_fill_random(void *dst, int32_t dtype_id, int64_t n, uint64_t seed, int dist, double p0,
                                  double p1);
/* Self-test of the bounded device wait every kernel here relies on: a one-CTA kernel waits, with a
 * budget of `limit_us` microseconds, on a barrier nothing arrives at; the wait gives up and the
 * kernel returns.  Returns 0 when that happened; b200mlir_device_status() then reports site 90
 * (and clears the word), exactly as after a real expiry.  The reference refuses instead of
 * hanging in the same way (bin/runtime/include/RuntimeDMA.h:19-37). */
B200_API int b200mlir_selftest_bounded_wait(int limit_us);

/* Raw tensor files of the reference's device harness
 * (test/utils/dsp/include/tensor.h:219-259; dtype ids :26-38; host reader
 * backend/hexagon_executor.py:200-216).  Output files: u32 dtype id, i64 rank,
 * i64 dims[rank], data.  Input files: data only.  `data` / `dst` may be host or device
 * pointers; rank <= 8. */
B200_API int b200mlir_dtype_size(int32_t dtype_id);
B200_API int b200mlir_tensor_dump(const char *path, int32_t dtype_id, int64_t rank, const int64_t *dims,
                                  const void *data);
B200_API int b200mlir_tensor_file_info(const char *path, int32_t *dtype_id, int64_t *rank, int64_t *dims,
                                       int64_t *data_bytes);
B200_API int b200mlir_tensor_load(const char *path, int has_header, void *dst, int64_t bytes);

/* Manifest of the matmuls dispatched since the last reset, in the vocabulary of
 * include/hexagon/Dialect/Hmx/Transforms/HmxManifest.h:81-111: plan "full-hmx"
 * (tensor cores, whole tiles) / "hmx-tail" (tensor cores, edge tiles) / "hvx"
 * (CUDA-core path) and the canonical reason; `detail` is this library's own wording.
 * Returns the length of the JSON text. */
B200_API int b200mlir_manifest_json(char *json, int cap);
B200_API void b200mlir_manifest_reset(void);

#ifdef __cplusplus
}
#endif
#endif /* B200MLIR_CAPI_H */
