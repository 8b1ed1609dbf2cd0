// The 29 engine and layout leaves of seam 2 (qcom_hexagon_backend/bin/runtime/hmx/include/HMXAPI.h:53-293,
// table include/hexagon/Conversion/HmxToLLVM/HmxLeafSignatures.h:85-137) under their own names.
//
// The reference's leaves take 32-bit addresses ("addresses, not pointers", HMXAPI.h:11-15), which
// cannot carry a 64-bit device address; these twins keep every name, the argument order and the
// argument meaning, and widen only the address arguments to uintptr_t.  Addresses are DEVICE
// addresses (from hexagon_runtime_alloc_* or any CUDA allocation); each leaf enqueues a small
// kernel on the calling thread's stream and returns.  A host address is refused with an error
// (b200mlir_last_error) instead of being dereferenced on the device.
//
// They exist for hosts whose compiled kernels call the leaves one tile at a time.  The library's
// own GEMM kernels do not go through them: there the packs are TMA's swizzle, the engine is
// tcgen05 with accumulators in TMEM and the read-out is fused (gemm_tcgen05*.cu).
//
// Tile image: element (r, c) of a 32 x 32 fp16 tile at byte 128*(r>>1) + 4*c + 2*(r&1)
// (hmx/src/HMXLayout.c:9-14), the same for activation, weight and accumulator read-out tiles.
// Engine state (HMXAPI.c:22-55): one 32 x 32 accumulator, held here as fp32 in device memory,
// and four 256-byte bias sets of which only the identity conversion (scale 1.0, bias 0) exists
// in the reference.
#include <mutex>

#include "common.h"

namespace b200 {
namespace {

constexpr int kTile = 32, kTileElems = 1024;

__device__ __forceinline__ int tile_elem(int r, int c) { return 64 * (r >> 1) + 2 * c + (r & 1); }

// ---- pack: row-major (or transposed) source -> consecutive tiles --------------------------------
// Tile t of the call covers logical tile (tile_row + (ADV_ROW ? t : 0), tile_col + (ADV_ROW ? 0 : t)).
// Logical element (R, C) = (32*tr + r, 32*tc + c) reads src[R*stride + C], or src[C*stride + R] for a
// transposed source; out of range (R >= rows, C >= cols, r >= valid_rows, c >= valid_cols) is zero.
template <bool SRC_F32, bool TRANSPOSED>
__global__ void __launch_bounds__(256)
leaf_pack_kernel(__half *__restrict__ dst, const void *__restrict__ src, unsigned rows, unsigned cols, unsigned stride,
                 unsigned tile_row, unsigned tile_col, int adv_row, unsigned valid_rows, unsigned valid_cols) {
  const unsigned t = blockIdx.x;
  const unsigned tr = tile_row + (adv_row ? t : 0u), tc = tile_col + (adv_row ? 0u : t);
  __half *tile = dst + (size_t)t * kTileElems;
  for (int e = threadIdx.x; e < kTileElems; e += 256) {
    const int r = e >> 5, c = e & 31;
    const unsigned R = tr * kTile + r, C = tc * kTile + c;
    __half v = __float2half_rn(0.0f);
    if (R < rows && C < cols && (unsigned)r < valid_rows && (unsigned)c < valid_cols) {
      const size_t idx = TRANSPOSED ? (size_t)C * stride + R : (size_t)R * stride + C;
      if (SRC_F32) {
        // the engine's conversion folded into the pack: "+0.0" (so -0 becomes +0), then round to
        // nearest even (HMXLayout.c:257-264)
        v = __float2half_rn(__fadd_rn(reinterpret_cast<const float *>(src)[idx], 0.0f));
      } else {
        v = reinterpret_cast<const __half *>(src)[idx];
      }
    }
    tile[tile_elem(r, c)] = v;
  }
}

// ---- unpack: a row of read-out tiles -> row-major rows --------------------------------------------
// Rows tile_row*32 + 2*j, +1 for j in [pair0, pair0 + n_pairs); columns [0, cols_limit); column
// `col` comes from tile col/32 of the row (tile 0 only in the bounds-safe single-tile form).
template <bool DST_F32>
__global__ void __launch_bounds__(256)
leaf_unpack_kernel(void *__restrict__ dst, const float *__restrict__ res, int has_res, const __half *__restrict__ ar,
                   unsigned dst_rows, unsigned cols_limit, unsigned dst_stride, unsigned res_stride, unsigned tile_row,
                   unsigned pair0, unsigned n_pairs, unsigned valid_rows) {
  const unsigned total = 2u * n_pairs * cols_limit;
  for (unsigned i = blockIdx.x * 256 + threadIdx.x; i < total; i += gridDim.x * 256) {
    const unsigned col = i % cols_limit, rr = i / cols_limit;
    const unsigned r_in_tile = 2u * pair0 + rr;  // row inside the 32-row tile
    const unsigned row = tile_row * kTile + r_in_tile;
    if (r_in_tile >= valid_rows || row >= dst_rows) continue;
    const __half v = ar[(size_t)(col >> 5) * kTileElems + tile_elem((int)r_in_tile, (int)(col & 31))];
    if (DST_F32) {
      float f = __half2float(v);  // x1.0 widening, exact (HMXLayout.c:876-882)
      if (has_res) f += res[(size_t)row * res_stride + col];
      reinterpret_cast<float *>(dst)[(size_t)row * dst_stride + col] = f;
    } else {
      reinterpret_cast<__half *>(dst)[(size_t)row * dst_stride + col] = v;
    }
  }
}

// ---- engine ---------------------------------------------------------------------------------------
struct Engine {
  float *acc = nullptr;      // [32][32] fp32
  uint32_t *bias = nullptr;  // 4 sets x 64 words
  int device = -1;
};
Engine g_engine;
std::mutex g_engine_mu;

int engine_ready() {
  B200_TRY(ensure_ready());
  std::lock_guard<std::mutex> lk(g_engine_mu);
  if (g_engine.acc) return 0;
  B200_CUDA(cudaMalloc(&g_engine.acc, kTileElems * sizeof(float)));
  B200_CUDA(cudaMalloc(&g_engine.bias, 4 * 64 * sizeof(uint32_t)));
  B200_CUDA(cudaMemsetAsync(g_engine.acc, 0, kTileElems * sizeof(float), ctx().stream));
  B200_CUDA(cudaMemsetAsync(g_engine.bias, 0, 4 * 64 * sizeof(uint32_t), ctx().stream));
  g_engine.device = ctx().device;
  return 0;
}

__global__ void bias_unit_kernel(uint32_t *w) {
  // lower words: scale = fp16 1.0 in [15:0], output bias 0; upper words 0 (HMXAPI.c:18-28)
  const int ch = threadIdx.x;
  if (ch < 32) w[ch] = 0x00003C00u;
  else if (ch < 64) w[ch] = 0u;
}
__global__ void bias_load_kernel(uint32_t *sets, const uint32_t *src, unsigned set) {
  if (threadIdx.x < 64) sets[(set & 3u) * 64 + threadIdx.x] = src[threadIdx.x];
}
__global__ void acc_clear_kernel(float *acc) { acc[threadIdx.x] = 0.0f; }

// acc[m][n] += sum over the call's tiles t and kk of act_t(m, kk) * wt_t(kk, n): fp16 products are
// exact in fp32, the sums are fp32 in ascending k (the engine's wide accumulator, HMXAPI.c:47-55)
__global__ void __launch_bounds__(1024)
mma_kernel(float *__restrict__ acc, const __half *__restrict__ act, const __half *__restrict__ wt, unsigned n_tiles) {
  __shared__ __half a_s[kTileElems], w_s[kTileElems];
  const int m = threadIdx.x >> 5, n = threadIdx.x & 31;
  float sum = acc[threadIdx.x];
  for (unsigned t = 0; t < n_tiles; ++t) {
    __syncthreads();
    a_s[threadIdx.x] = act[(size_t)t * kTileElems + threadIdx.x];
    w_s[threadIdx.x] = wt[(size_t)t * kTileElems + threadIdx.x];
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kTile; ++kk)
      sum += __half2float(a_s[tile_elem(m, kk)]) * __half2float(w_s[tile_elem(kk, n)]);
  }
  acc[threadIdx.x] = sum;
}

// read-out: fp16(acc * scale + bias) with the loaded set's per-column scale and output bias (the
// identity set in the reference), stored in the tile image; the accumulator is cleared (fused form)
__global__ void __launch_bounds__(1024)
acc_store_kernel(float *__restrict__ acc, const uint32_t *__restrict__ bias_set, __half *__restrict__ dst) {
  const int r = threadIdx.x >> 5, c = threadIdx.x & 31;
  const uint32_t lo = bias_set[c];
  const float scale = __half2float(__ushort_as_half((unsigned short)(lo & 0xffffu)));
  const float obias = __half2float(__ushort_as_half((unsigned short)(lo >> 16)));
  dst[tile_elem(r, c)] = __float2half_rn(acc[threadIdx.x] * scale + obias);
  acc[threadIdx.x] = 0.0f;
}

bool dev_addr(const char *leaf, const char *what, uintptr_t a) {
  if (a != 0 && is_device_ptr((const void *)a)) return true;
  set_error(B200MLIR_ERR_BAD_ARG, "%s: %s must be a device address (got %p)", leaf, what, (void *)a);
  return false;
}

template <bool F32, bool T>
void pack(const char *leaf, uintptr_t dst, uintptr_t src, unsigned rows, unsigned cols, unsigned stride, unsigned tile_row,
          unsigned tile_col, unsigned n_tiles, int adv_row, unsigned valid_rows = kTile, unsigned valid_cols = kTile) {
  clear_error();
  if (ensure_ready() || n_tiles == 0) return;
  if (!dev_addr(leaf, "dst_addr", dst) || !dev_addr(leaf, "src_addr", src)) return;
  leaf_pack_kernel<F32, T><<<n_tiles, 256, 0, ctx().stream>>>((__half *)dst, (const void *)src, rows, cols, stride, tile_row,
                                                             tile_col, adv_row, valid_rows, valid_cols);
  check_launch(leaf);
}

template <bool F32>
void unpack(const char *leaf, uintptr_t dst, uintptr_t res, unsigned has_res, uintptr_t ar, unsigned dst_rows,
            unsigned cols_limit, unsigned dst_stride, unsigned res_stride, unsigned tile_row, unsigned pair0,
            unsigned n_pairs, unsigned valid_rows = kTile) {
  clear_error();
  if (ensure_ready() || n_pairs == 0 || cols_limit == 0) return;
  if (!dev_addr(leaf, "dst_addr", dst) || !dev_addr(leaf, "src_ar_addr", ar)) return;
  if (has_res && !dev_addr(leaf, "res_addr", res)) return;
  const unsigned total = 2u * n_pairs * cols_limit;
  unsigned blocks = (total + 255) / 256;
  if (blocks > 1024) blocks = 1024;
  leaf_unpack_kernel<F32><<<blocks, 256, 0, ctx().stream>>>((void *)dst, (const float *)res, has_res ? 1 : 0, (const __half *)ar,
                                                           dst_rows, cols_limit, dst_stride, res_stride, tile_row, pair0,
                                                           n_pairs, valid_rows);
  check_launch(leaf);
}

// pairs of the tile row that lie inside dst_rows (the bulk forms stop at the first pair past the end)
unsigned clamp_pairs(unsigned dst_rows, unsigned tile_row, unsigned n_pairs) {
  const unsigned base = tile_row * kTile;
  unsigned n = base < dst_rows ? (dst_rows - base + 1u) / 2u : 0u;
  if (n > 16u) n = 16u;
  return n < n_pairs ? n : n_pairs;
}
unsigned min_u(unsigned a, unsigned b) { return a < b ? a : b; }

}  // namespace
}  // namespace b200

using namespace b200;
#define LEAF __attribute__((visibility("default")))

extern "C" {

// ---- bias / accumulator / multiply-accumulate (HMXAPI.h:53-66) ------------------------------------
LEAF void hmx_bias_init_unit_f16(uintptr_t bias_addr) {
  clear_error();
  if (ensure_ready() || !dev_addr("hmx_bias_init_unit_f16", "bias_addr", bias_addr)) return;
  bias_unit_kernel<<<1, 64, 0, ctx().stream>>>((uint32_t *)bias_addr);
  check_launch("hmx_bias_init_unit_f16");
}
LEAF void hmx_bias_load_f16(uintptr_t bias_addr, unsigned set) {
  clear_error();
  if (engine_ready() || !dev_addr("hmx_bias_load_f16", "bias_addr", bias_addr)) return;
  bias_load_kernel<<<1, 64, 0, ctx().stream>>>(g_engine.bias, (const uint32_t *)bias_addr, set);
  check_launch("hmx_bias_load_f16");
}
LEAF void hmx_acc_clear_f16(void) {
  clear_error();
  if (engine_ready()) return;
  acc_clear_kernel<<<1, 1024, 0, ctx().stream>>>(g_engine.acc);
  check_launch("hmx_acc_clear_f16");
}
LEAF void hmx_acc_store_f16(uintptr_t dst_addr, unsigned set) {
  clear_error();
  if (engine_ready() || !dev_addr("hmx_acc_store_f16", "dst_addr", dst_addr)) return;
  acc_store_kernel<<<1, 1024, 0, ctx().stream>>>(g_engine.acc, g_engine.bias + (set & 3u) * 64, (__half *)dst_addr);
  check_launch("hmx_acc_store_f16");
}
LEAF void hmx_mma_f16(uintptr_t act_addr, uintptr_t wt_addr, unsigned n_croutons) {
  clear_error();
  if (engine_ready() || n_croutons == 0) return;
  if (!dev_addr("hmx_mma_f16", "act_addr", act_addr) || !dev_addr("hmx_mma_f16", "wt_addr", wt_addr)) return;
  mma_kernel<<<1, 1024, 0, ctx().stream>>>(g_engine.acc, (const __half *)act_addr, (const __half *)wt_addr, n_croutons);
  check_launch("hmx_mma_f16");
}

// ---- packs (HMXAPI.h:81-212) ------------------------------------------------------------------------
LEAF void hmx_pack_act_f16(uintptr_t dst, uintptr_t src, unsigned rows, unsigned cols, unsigned stride, unsigned tile_row,
                           unsigned tile_col) {
  pack<false, false>("hmx_pack_act_f16", dst, src, rows, cols, stride, tile_row, tile_col, 1, 0);
}
LEAF void hmx_pack_weight_f16(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride, unsigned k_tile,
                              unsigned n_tile) {
  pack<false, false>("hmx_pack_weight_f16", dst, src, k, n, stride, k_tile, n_tile, 1, 1);
}
LEAF void hmx_pack_act_f16_bulk(uintptr_t dst, uintptr_t src, unsigned rows, unsigned cols, unsigned stride,
                                unsigned tile_row, unsigned tile_col_start, unsigned n_col_tiles) {
  pack<false, false>("hmx_pack_act_f16_bulk", dst, src, rows, cols, stride, tile_row, tile_col_start, n_col_tiles, 0);
}
LEAF void hmx_pack_weight_f16_bulk(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride,
                                   unsigned k_tile_start, unsigned n_tile, unsigned n_k_tiles) {
  pack<false, false>("hmx_pack_weight_f16_bulk", dst, src, k, n, stride, k_tile_start, n_tile, n_k_tiles, 1);
}
LEAF void hmx_pack_act_f32(uintptr_t dst, uintptr_t src, unsigned rows, unsigned cols, unsigned stride, unsigned tile_row,
                           unsigned tile_col) {
  pack<true, false>("hmx_pack_act_f32", dst, src, rows, cols, stride, tile_row, tile_col, 1, 0);
}
LEAF void hmx_pack_weight_f32(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride, unsigned k_tile,
                              unsigned n_tile) {
  pack<true, false>("hmx_pack_weight_f32", dst, src, k, n, stride, k_tile, n_tile, 1, 1);
}
LEAF void hmx_pack_act_f32_bulk(uintptr_t dst, uintptr_t src, unsigned rows, unsigned cols, unsigned stride,
                                unsigned tile_row, unsigned tile_col_start, unsigned n_col_tiles) {
  pack<true, false>("hmx_pack_act_f32_bulk", dst, src, rows, cols, stride, tile_row, tile_col_start, n_col_tiles, 0);
}
LEAF void hmx_pack_weight_f32_bulk(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride,
                                   unsigned k_tile_start, unsigned n_tile, unsigned n_k_tiles) {
  pack<true, false>("hmx_pack_weight_f32_bulk", dst, src, k, n, stride, k_tile_start, n_tile, n_k_tiles, 1);
}
// transposed source: src is row-major [n][k], W[k, n] = src[n*stride + k]
LEAF void hmx_pack_weight_f16_T(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride, unsigned k_tile,
                                unsigned n_tile) {
  pack<false, true>("hmx_pack_weight_f16_T", dst, src, k, n, stride, k_tile, n_tile, 1, 1);
}
LEAF void hmx_pack_weight_f16_T_bulk(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride,
                                     unsigned k_tile_start, unsigned n_tile, unsigned n_k_tiles) {
  pack<false, true>("hmx_pack_weight_f16_T_bulk", dst, src, k, n, stride, k_tile_start, n_tile, n_k_tiles, 1);
}
LEAF void hmx_pack_weight_f32_T(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride, unsigned k_tile,
                                unsigned n_tile) {
  pack<true, true>("hmx_pack_weight_f32_T", dst, src, k, n, stride, k_tile, n_tile, 1, 1);
}
LEAF void hmx_pack_weight_f32_T_bulk(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride,
                                     unsigned k_tile_start, unsigned n_tile, unsigned n_k_tiles) {
  pack<true, true>("hmx_pack_weight_f32_T_bulk", dst, src, k, n, stride, k_tile_start, n_tile, n_k_tiles, 1);
}
// bounds-safe single tiles: only valid_rows x valid_cols of the tile are read, the rest is zero
LEAF void hmx_pack_act_tail_f16(uintptr_t dst, uintptr_t src, unsigned rows, unsigned cols, unsigned stride,
                                unsigned tile_row, unsigned tile_col, unsigned valid_rows, unsigned valid_cols) {
  pack<false, false>("hmx_pack_act_tail_f16", dst, src, rows, cols, stride, tile_row, tile_col, 1, 0, valid_rows, valid_cols);
}
LEAF void hmx_pack_weight_tail_f16(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride, unsigned k_tile,
                                   unsigned n_tile, unsigned valid_rows, unsigned valid_cols) {
  pack<false, false>("hmx_pack_weight_tail_f16", dst, src, k, n, stride, k_tile, n_tile, 1, 1, valid_rows, valid_cols);
}
LEAF void hmx_pack_act_tail_f32(uintptr_t dst, uintptr_t src, unsigned rows, unsigned cols, unsigned stride,
                                unsigned tile_row, unsigned tile_col, unsigned valid_rows, unsigned valid_cols) {
  pack<true, false>("hmx_pack_act_tail_f32", dst, src, rows, cols, stride, tile_row, tile_col, 1, 0, valid_rows, valid_cols);
}
LEAF void hmx_pack_weight_tail_f32(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride, unsigned k_tile,
                                   unsigned n_tile, unsigned valid_rows, unsigned valid_cols) {
  pack<true, false>("hmx_pack_weight_tail_f32", dst, src, k, n, stride, k_tile, n_tile, 1, 1, valid_rows, valid_cols);
}
LEAF void hmx_pack_weight_tail_f16_T(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride,
                                     unsigned k_tile, unsigned n_tile, unsigned valid_rows, unsigned valid_cols) {
  pack<false, true>("hmx_pack_weight_tail_f16_T", dst, src, k, n, stride, k_tile, n_tile, 1, 1, valid_rows, valid_cols);
}
LEAF void hmx_pack_weight_tail_f32_T(uintptr_t dst, uintptr_t src, unsigned k, unsigned n, unsigned stride,
                                     unsigned k_tile, unsigned n_tile, unsigned valid_rows, unsigned valid_cols) {
  pack<true, true>("hmx_pack_weight_tail_f32_T", dst, src, k, n, stride, k_tile, n_tile, 1, 1, valid_rows, valid_cols);
}

// ---- read-outs (HMXAPI.h:231-293) -------------------------------------------------------------------
LEAF void hmx_unpack_acc_f16(uintptr_t dst, uintptr_t ar, unsigned dst_rows, unsigned dst_cols, unsigned dst_stride,
                             unsigned tile_row, unsigned block_j) {
  unpack<false>("hmx_unpack_acc_f16", dst, 0, 0, ar, dst_rows, dst_cols, dst_stride, 0, tile_row, block_j, 1);
}
LEAF void hmx_unpack_acc_f16_bulk(uintptr_t dst, uintptr_t ar, unsigned dst_rows, unsigned dst_cols, unsigned dst_stride,
                                  unsigned tile_row, unsigned n_pairs) {
  unpack<false>("hmx_unpack_acc_f16_bulk", dst, 0, 0, ar, dst_rows, dst_cols, dst_stride, 0, tile_row, 0,
                clamp_pairs(dst_rows, tile_row, n_pairs));
}
LEAF void hmx_unpack_acc_f32(uintptr_t dst, uintptr_t res, unsigned has_res, uintptr_t ar, unsigned dst_rows,
                             unsigned dst_cols, unsigned dst_stride, unsigned res_stride, unsigned tile_row,
                             unsigned block_j) {
  unpack<true>("hmx_unpack_acc_f32", dst, res, has_res, ar, dst_rows, dst_cols, dst_stride, res_stride, tile_row, block_j, 1);
}
LEAF void hmx_unpack_acc_f32_bulk(uintptr_t dst, uintptr_t res, unsigned has_res, uintptr_t ar, unsigned dst_rows,
                                  unsigned dst_cols, unsigned dst_stride, unsigned res_stride, unsigned tile_row,
                                  unsigned n_pairs) {
  unpack<true>("hmx_unpack_acc_f32_bulk", dst, res, has_res, ar, dst_rows, dst_cols, dst_stride, res_stride, tile_row, 0,
               clamp_pairs(dst_rows, tile_row, n_pairs));
}
// single-tile, bounds-safe: columns below min(valid_cols, 32, dst_cols) of rows below valid_rows
LEAF void hmx_unpack_acc_tail_f16(uintptr_t dst, uintptr_t ar, unsigned dst_rows, unsigned dst_cols, unsigned dst_stride,
                                  unsigned tile_row, unsigned block_j, unsigned valid_rows, unsigned valid_cols) {
  unpack<false>("hmx_unpack_acc_tail_f16", dst, 0, 0, ar, dst_rows, min_u(min_u(valid_cols, kTile), dst_cols), dst_stride, 0,
                tile_row, block_j, 1, valid_rows);
}
LEAF void hmx_unpack_acc_tail_f32(uintptr_t dst, uintptr_t res, unsigned has_res, uintptr_t ar, unsigned dst_rows,
                                  unsigned dst_cols, unsigned dst_stride, unsigned res_stride, unsigned tile_row,
                                  unsigned block_j, unsigned valid_rows, unsigned valid_cols) {
  unpack<true>("hmx_unpack_acc_tail_f32", dst, res, has_res, ar, dst_rows, min_u(min_u(valid_cols, kTile), dst_cols),
               dst_stride, res_stride, tile_row, block_j, 1, valid_rows);
}

}  // extern "C"
