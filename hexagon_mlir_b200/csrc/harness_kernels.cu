// Harness pieces that run on the device: the synthetic-input generator and the self-test of
// the bounded device wait.
#include "common.h"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

// ---- synthetic inputs ------------------------------------------------------------------------
// Philox4x32-10, stateless: element i takes word (i & 3) of the block with counter
// (i >> 2, stream, lane) and key = seed, so every element is drawn independently of launch
// geometry and the host twins of this loop produce the same bytes.  Multiplies and adds are the
// explicitly unfused intrinsics: a contraction into an FMA would change the last bit.
__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ float fill_value(int64_t i, uint32_t k0, uint32_t k1, int dist, float p0, float p1) {
  uint32_t w[4];
  if (dist == 1) {  // Irwin-Hall: twelve 20-bit uniforms, exact integer sum
    uint32_t sum = 0;
#pragma unroll
    for (uint32_t j = 0; j < 3; ++j) {
      philox4x32_10((uint32_t)((uint64_t)i), (uint32_t)((uint64_t)i >> 32), j, 1u, k0, k1, w);
      sum += (w[0] >> 12) + (w[1] >> 12) + (w[2] >> 12) + (w[3] >> 12);
    }
    const float z = __fsub_rn(__fmul_rn(__uint2float_rn(sum), 9.5367431640625e-07f), 6.0f);
    return __fadd_rn(p0, __fmul_rn(p1, z));
  }
  philox4x32_10((uint32_t)((uint64_t)i >> 2), (uint32_t)((uint64_t)i >> 34), 0u, 0u, k0, k1, w);
  const uint32_t x = w[i & 3];
  if (dist == 2) {
    const int lo = (int)p0, hi = (int)p1;
    return (float)(lo + (int)(x % (uint32_t)(hi - lo + 1)));
  }
  const float u = __fmul_rn(__uint2float_rn(x >> 8), 5.9604644775390625e-08f);
  return __fadd_rn(p0, __fmul_rn(u, __fsub_rn(p1, p0)));
}

__global__ void fill_random_kernel(void *dst, int dtype_id, int64_t n, uint32_t k0, uint32_t k1, int dist, float p0,
                                   float p1) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = fill_value(i, k0, k1, dist, p0, p1);
    if (dtype_id == 1) reinterpret_cast<__half *>(dst)[i] = __float2half_rn(v);
    else if (dtype_id == 2) reinterpret_cast<float *>(dst)[i] = v;
    else reinterpret_cast<int8_t *>(dst)[i] = (int8_t)(int)v;
  }
}

// ---- bounded-wait self-test ------------------------------------------------------------------
// One thread waits on an mbarrier that nothing ever arrives at, with a clock budget of
// `limit_cycles`; the wait gives up, records {site, detail} in the status word and the kernel
// returns.  This is the expiry path of every wait in the GEMM, w8a16 and attention kernels
// (same function, same status word), exercised without making any of them misbehave.
constexpr int kSelfTestSite = 90;
constexpr int kSelfTestDetail = 7;
__global__ void bounded_wait_selftest_kernel(int *status, long long limit_cycles, int *returned) {
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ int abort_flag;
  const uint32_t bar = ptx::smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = ptx::mbar_wait(bar, 0, &abort_flag, status, kSelfTestSite, kSelfTestDetail, limit_cycles);
  __syncthreads();
  // bit 0: the waiter saw its wait expire; bit 1: the wait claimed success (must not happen);
  // bit 2: another warp of the CTA sees the abort flag the expired wait raised, as the kernels' roles do
  if (threadIdx.x == 0) atomicOr(returned, (abort_flag ? 1 : 0) | (ok ? 2 : 0));
  if (threadIdx.x == 32 && abort_flag) atomicOr(returned, 4);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200mlir_fill_random(void *dst, int32_t dtype_id, int64_t n, uint64_t seed, int dist, double p0, double p1) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!dst || n < 0 || (dtype_id != 1 && dtype_id != 2 && dtype_id != 4) || dist < 0 || dist > 2)
    return set_error(B200MLIR_ERR_BAD_ARG, "fill_random: dtype id 1 (f16), 2 (f32) or 4 (int8); dist 0, 1 or 2");
  if (dist == 2 && !((int)p1 >= (int)p0)) return set_error(B200MLIR_ERR_BAD_ARG, "fill_random: empty integer range");
  if (n == 0) return 0;
  Context &c = ctx();
  const size_t esz = dtype_id == 1 ? 2 : dtype_id == 2 ? 4 : 1;
  void *dev = dst;
  const bool host = !is_device_ptr(dst);
  if (host) B200_CUDA(cudaMallocAsync(&dev, (size_t)n * esz, c.stream));
  const int64_t want = (n + 255) / 256;
  const unsigned grid = (unsigned)(want < (int64_t)c.sm_count * 16 ? want : (int64_t)c.sm_count * 16);
  fill_random_kernel<<<grid, 256, 0, c.stream>>>(dev, dtype_id, n, (uint32_t)seed, (uint32_t)(seed >> 32), dist,
                                                 (float)p0, (float)p1);
  int rc = check_launch("fill_random");
  if (host) {
    cudaError_t e = cudaMemcpyAsync(dst, dev, (size_t)n * esz, cudaMemcpyDeviceToHost, c.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c.stream);
    cudaFreeAsync(dev, c.stream);
    if (rc == 0 && e != cudaSuccess) rc = set_error(B200MLIR_ERR_CUDA, "fill_random: %s", cudaGetErrorString(e));
  }
  return rc;
}

int b200mlir_selftest_bounded_wait(int limit_us) {
  clear_error();
  B200_TRY(ensure_ready());
  if (limit_us < 1 || limit_us > 100000)
    return set_error(B200MLIR_ERR_BAD_ARG, "selftest: limit between 1 us and 100 ms");
  Context &c = ctx();
  int clock_khz = 0;
  B200_CUDA(cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, c.device));
  const long long cycles = (long long)limit_us * (clock_khz > 0 ? clock_khz : 1965000) / 1000;
  int *d_ret = c.d_status + 16;  // a spare word of the 256-byte status block
  B200_CUDA(cudaMemsetAsync(d_ret, 0, sizeof(int), c.stream));
  bounded_wait_selftest_kernel<<<1, 64, 0, c.stream>>>(c.d_status, cycles, d_ret);
  B200_TRY(check_launch("bounded_wait_selftest"));
  int h = -1;
  B200_CUDA(cudaMemcpyAsync(&h, d_ret, sizeof(int), cudaMemcpyDeviceToHost, c.stream));
  B200_CUDA(cudaStreamSynchronize(c.stream));
  if (h != 5) return set_error(B200MLIR_ERR_CUDA, "selftest: the wait returned %d (expected an expiry)", h);
  return 0;
}

}  // extern "C"
