// Pieces shared by the 1-CTA and the 2-CTA tensor-core GEMM kernels: the kernel
// parameter block, the tile walk, the fused epilogues and the tensor-map helper.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include <mutex>

#include "common.h"

namespace b200 {
namespace {

constexpr int GROUP_M = 8;  // default height, in tiles, of the band the tile walk sweeps (option gemmGroupM)

struct TcParams {
  void *c;
  const void *res;
  int64_t ldc, ldres;
  int m, n, k;
  int m_blocks, n_blocks, num_tiles, k_blocks;
  int group_m;
  int seg_kb;  // K-looped form: k-blocks per segment
  void *push_recv[kMaxPushRanks];  // EPI_PUSH16: receive buffers, by owner rank
  int push_rank, push_rows;
  int *status;
  int res_mod = 1, res_rem = 0;  // EPI_F16_RES16: residual only in 256-row blocks b with b % res_mod == res_rem
};

__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int group_m, int &m_blk,
                                            int &n_blk) {
  // A division costs the lone producer thread about 300 clocks, and on a small problem its first
  // load waits for this: the first band needs none, and a band height that is a power of two
  // (the default, 8) needs only shifts.
  const int per_group = group_m * n_blocks;
  const int group = tile < per_group ? 0 : tile / per_group;
  const int first_m = group * group_m;
  const int gsz = min(m_blocks - first_m, group_m);
  const int in_group = tile - group * per_group;
  if ((gsz & (gsz - 1)) == 0) {
    const int sh = __ffs(gsz) - 1;
    m_blk = first_m + (in_group & (gsz - 1));
    n_blk = in_group >> sh;
  } else {
    m_blk = first_m + in_group % gsz;
    n_blk = in_group / gsz;
  }
}

__device__ __forceinline__ __half silu_h(__half x) {
  __half e = __float2half_rn(__expf(-__half2float(x)));
  __half d = __float2half_rn(1.0f + __half2float(e));
  return __float2half_rn(__fdividef(__half2float(x), __half2float(d)));
}

// {d0, d1} += {f32(f16(a0)), f32(f16(a1))}: one packed rounding, two widenings, one packed add
// (the K-looped read-out: every segment is rounded to fp16 before it joins the fp32 running sum)
__device__ __forceinline__ void add_rounded2(float &d0, float &d1, float a0, float a1) {
  const float2 f = __half22float2(__floats2half2_rn(a0, a1));
  asm("{\n\t.reg .b64 ra, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\t"
      "add.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "+f"(d0), "+f"(d1)
      : "f"(f.x), "f"(f.y));
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}


// The fp16 residual of one 32-column chunk of a row.  A read-out thread owns a row, so these are
// four lone 16-byte loads whose latency nothing else of the chunk hides: they are issued one chunk
// ahead (the first before the wait for the accumulators), and the chunk's store finds them landed.
struct ResChunk {
  uint4 v[8];  // four vectors of 8 fp16 values, or eight of 4 fp32 values (the fp32 read-out's residual)
};
template <int EPI>
__device__ __forceinline__ void residual_prefetch(ResChunk &rc, int row, int col0, bool row_ok, const TcParams &p) {
  if (EPI == EPI_F32_RES) {
    const float *rp = reinterpret_cast<const float *>(p.res) + (int64_t)row * p.ldres + col0;
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      if (p.res && row_ok && col0 + v * 4 < p.n)
        rc.v[v] = __ldg(reinterpret_cast<const uint4 *>(rp + v * 4));
      else
        rc.v[v] = make_uint4(0u, 0u, 0u, 0u);
    }
    return;
  }
  if (EPI != EPI_F16_RES16) return;
  const __half *rp = reinterpret_cast<const __half *>(p.res) + (int64_t)row * p.ldres + col0;
  if (p.res_mod > 1 && (row >> 8) % p.res_mod != p.res_rem) row_ok = false;  // another rank adds it here: + 0 is exact
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    if (row_ok && col0 + v * 8 < p.n)
      rc.v[v] = __ldg(reinterpret_cast<const uint4 *>(rp + v * 8));
    else
      rc.v[v] = make_uint4(0u, 0u, 0u, 0u);
  }
}

// One 32-column chunk of one accumulator row: r (and r2 for the SwiGLU pair) hold the
// fp32 accumulators of columns [col0, col0+32) of `row`; rc the chunk's residual (EPI_F16_RES16).
template <int EPI>
__device__ __forceinline__ void epilogue_store_chunk(const uint32_t (&r)[32], const uint32_t (&r2)[32], int row,
                                                     int col0, const TcParams &p, const ResChunk &rc) {
  if (EPI == EPI_F16 || EPI == EPI_F16_RES16 || EPI == EPI_SWIGLU) {
    __half *cp = reinterpret_cast<__half *>(p.c) + (int64_t)row * p.ldc + col0;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      if (col0 + v * 8 >= p.n) break;  // N is a multiple of 8
      uint4 o;
      uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
      if (EPI == EPI_F16) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          ow[j] = pack_h2(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
      } else if (EPI == EPI_F16_RES16) {
        // f16(f32(f16(acc)) + f32(res)): the engine reads out fp16, the residual is added wide
        const uint4 rv = rc.v[v];
        const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 t = __half22float2(__floats2half2_rn(__uint_as_float(r[v * 8 + 2 * j]),
                                                      __uint_as_float(r[v * 8 + 2 * j + 1])));
          float2 rr = __half22float2(rh[j]);
          ow[j] = pack_h2(t.x + rr.x, t.y + rr.y);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __half g0 = __float2half_rn(__uint_as_float(r[v * 8 + 2 * j]));
          __half g1 = __float2half_rn(__uint_as_float(r[v * 8 + 2 * j + 1]));
          __half u0 = __float2half_rn(__uint_as_float(r2[v * 8 + 2 * j]));
          __half u1 = __float2half_rn(__uint_as_float(r2[v * 8 + 2 * j + 1]));
          ow[j] = pack_h2(__half2float(silu_h(g0)) * __half2float(u0),
                          __half2float(silu_h(g1)) * __half2float(u1));
        }
      }
      *reinterpret_cast<uint4 *>(cp + v * 8) = o;
    }
  } else if (EPI == EPI_PUSH16) {
    // the row's owner holds [world][rows][N]; this rank fills slot push_rank (stores cross NVLink)
    const int owner = row / p.push_rows;
    const int lr = row - owner * p.push_rows;
    __half *cp = reinterpret_cast<__half *>(p.push_recv[owner]) +
                 ((int64_t)p.push_rank * p.push_rows + lr) * p.ldc + col0;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      if (col0 + v * 8 >= p.n) break;  // N is a multiple of 8
      uint4 o;
      uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        ow[j] = pack_h2(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
      *reinterpret_cast<uint4 *>(cp + v * 8) = o;
    }
  } else if (EPI == EPI_I32) {
    int32_t *cp = reinterpret_cast<int32_t *>(p.c) + (int64_t)row * p.ldc + col0;
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      if (col0 + v * 4 >= p.n) break;  // N is a multiple of 4
      *reinterpret_cast<int4 *>(cp + v * 4) =
          make_int4((int)r[v * 4], (int)r[v * 4 + 1], (int)r[v * 4 + 2], (int)r[v * 4 + 3]);
    }
  } else if (EPI == EPI_F32_RES) {
    float *cp = reinterpret_cast<float *>(p.c) + (int64_t)row * p.ldc + col0;
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      if (col0 + v * 4 >= p.n) break;  // N is a multiple of 8
      float4 o;
      float *of = reinterpret_cast<float *>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        of[j] = __half2float(__float2half_rn(__uint_as_float(r[v * 4 + j])));
      if (p.res) {  // fetched a chunk ahead (zeros where there is none: the sum is then exact)
        const uint4 rv = rc.v[v];
        o.x += __uint_as_float(rv.x); o.y += __uint_as_float(rv.y); o.z += __uint_as_float(rv.z); o.w += __uint_as_float(rv.w);
      }
      *reinterpret_cast<float4 *>(cp + v * 4) = o;
    }
  }
}

template <int EPI>
__device__ __forceinline__ void epilogue_store_chunk(const uint32_t (&r)[32], const uint32_t (&r2)[32], int row,
                                                     int col0, const TcParams &p) {
  static_assert(EPI != EPI_F16_RES16 && EPI != EPI_F32_RES, "the residual is passed in, fetched a chunk ahead");
  ResChunk none;
  epilogue_store_chunk<EPI>(r, r2, row, col0, p, none);
}

// Fills the EPI_PUSH16 part of the kernel parameters.
inline void set_push_params(TcParams &p, const GemmArgs &g) {
  for (int i = 0; i < kMaxPushRanks; ++i) p.push_recv[i] = g.push ? g.push->recv[i] : nullptr;
  p.push_rank = g.push ? g.push->rank : 0;
  p.push_rows = g.push ? (int)g.push->rows_per_rank : 1;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// 2-D row-major tensor [outer, inner] with row pitch ld elements; box {box_inner, box_outer}.
int make_map_2d(CUtensorMap *map, const void *base, CUtensorMapDataType dt, int elem_bytes,
                int64_t inner, int64_t outer, int64_t ld, int box_inner, int box_outer) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(B200MLIR_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (cuuint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(B200MLIR_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}


}  // namespace
}  // namespace b200
