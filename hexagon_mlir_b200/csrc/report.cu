// Host tooling formats of the reference, so that its harness can drive this library
// unchanged: raw tensor files, the perf.txt report, and the matmul manifest.
//
//  * tensor files: inputs are raw element data; outputs carry a header
//    {u32 dtype id, i64 rank, i64 dims[rank]} before the data
//    (test/utils/dsp/include/tensor.h:219-259, ids :26-38; host reader
//    backend/hexagon_executor.py:200-216).
//  * perf.txt: a "Test_Info: {...}" block written by TestReport::save
//    (test/utils/dsp/include/test_report.h:43-66) followed by an appended
//    "PerfPcycles:<n>" line taken from the same timed pass
//    (backend/hexagon_launcher_base.py:155-192; parser backend/hmx_search.py:1074-1092).
//  * manifest: per-matmul {plan, reason} records in the reference's vocabulary
//    (include/hexagon/Dialect/Hmx/Transforms/HmxManifest.h:81-111).
#include <cstdio>
#include <cstring>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "common.h"

namespace b200 {
namespace {

const int kDtypeSize[] = {1, 2, 4, 8, 1, 2, 4, 8, 1, 2, 4};  // Bool, Half, Float, Double, Int8..Int64, UInt8..UInt32
constexpr int kDtypeCount = 11;
constexpr int64_t kMaxRank = 8;

int put_string(const std::string &s, char *buf, int cap) {
  if (buf && cap > 0) {
    size_t n = s.size() < (size_t)cap - 1 ? s.size() : (size_t)cap - 1;
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return (int)s.size();
}

struct FileCloser {
  FILE *f;
  ~FileCloser() {
    if (f) fclose(f);
  }
};

// ---- manifest ------------------------------------------------------------------------------
struct ManifestRow {
  int64_t m, n, k;
  int epilogue, variant;
  std::string plan, reason, detail, name;
  long long count;
};
std::mutex g_manifest_mu;
std::vector<ManifestRow> g_manifest;
constexpr size_t kManifestCap = 256;

const char *epilogue_name(int e) {
  switch (e) {
    case EPI_F16: return "f16";
    case EPI_F32_RES: return "f32+residual";
    case EPI_KLOOP_F16: return "kloop-f16";
    case EPI_F16_RES16: return "f16+residual";
    case EPI_SWIGLU: return "swiglu";
  }
  return "?";
}

// stamps the SM clock counter and the SM it was read on
__global__ void stamp_kernel(long long *out) {
  unsigned smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  out[0] = clock64();
  out[1] = (long long)smid;
}

}  // namespace

// Called by the GEMM dispatcher for every launch it plans.
void manifest_record(const GemmArgs &g, int variant, const std::string &why) {
  ManifestRow r;
  r.m = g.m; r.n = g.n; r.k = g.k;
  r.epilogue = g.epilogue;
  r.variant = variant;
  r.detail = why;
  r.count = 1;
  if (variant >= 0) {
    const TcVariantInfo &i = tc_variant_info(variant);
    r.name = i.name;
    const bool whole = g.m % i.bm == 0 && g.n % i.bn == 0 && g.k % i.bk == 0;
    r.plan = whole ? "full-hmx" : "hmx-tail";            // edge tiles: TMA zero fill + masked stores
    r.reason = whole ? "selected-aligned" : "selected-tail";
  } else {
    r.name = "simt64x64";
    r.plan = "hvx";
    if (why.find("min-rows") != std::string::npos) r.reason = "min-rows";
    else if (why.find("tile-alignment") != std::string::npos) r.reason = "tile-alignment";
    else if (why.find("budget") != std::string::npos) r.reason = "vtcm-budget";
    else if (why.find("option") != std::string::npos) r.reason = "library-call";
    else r.reason = "unsupported-layout";
  }
  std::lock_guard<std::mutex> lk(g_manifest_mu);
  for (auto &e : g_manifest)
    if (e.m == r.m && e.n == r.n && e.k == r.k && e.epilogue == r.epilogue && e.variant == r.variant &&
        e.detail == r.detail) {
      ++e.count;
      return;
    }
  if (g_manifest.size() < kManifestCap) g_manifest.push_back(r);
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200mlir_dtype_size(int32_t dtype_id) {
  return dtype_id >= 0 && dtype_id < kDtypeCount ? kDtypeSize[dtype_id] : 0;
}

int b200mlir_tensor_dump(const char *path, int32_t dtype_id, int64_t rank, const int64_t *dims, const void *data) {
  clear_error();
  const int esz = b200mlir_dtype_size(dtype_id);
  if (!path || !esz || rank < 0 || rank > kMaxRank || (rank > 0 && !dims))
    return set_error(B200MLIR_ERR_BAD_ARG, "tensor_dump: bad path / dtype id %d / rank %lld", (int)dtype_id,
                     (long long)rank);
  int64_t elems = 1;
  for (int64_t i = 0; i < rank; ++i) {
    if (dims[i] < 0) return set_error(B200MLIR_ERR_BAD_ARG, "tensor_dump: negative extent");
    elems *= dims[i];
  }
  const size_t bytes = (size_t)elems * esz;
  if (bytes && !data) return set_error(B200MLIR_ERR_BAD_ARG, "tensor_dump: null data");
  std::vector<uint8_t> host;
  const void *src = data;
  if (bytes && is_device_ptr(data)) {
    B200_TRY(ensure_ready());
    host.resize(bytes);
    B200_CUDA(cudaStreamSynchronize(ctx().stream));
    B200_CUDA(cudaMemcpy(host.data(), data, bytes, cudaMemcpyDeviceToHost));
    src = host.data();
  }
  FileCloser fc{fopen(path, "wb")};
  if (!fc.f) return set_error(B200MLIR_ERR_BAD_ARG, "tensor_dump: cannot open %s", path);
  bool ok = fwrite(&dtype_id, sizeof(int32_t), 1, fc.f) == 1 && fwrite(&rank, sizeof(int64_t), 1, fc.f) == 1;
  if (ok && rank > 0) ok = fwrite(dims, sizeof(int64_t), (size_t)rank, fc.f) == (size_t)rank;
  if (ok && bytes) ok = fwrite(src, 1, bytes, fc.f) == bytes;
  if (!ok) return set_error(B200MLIR_ERR_BAD_ARG, "tensor_dump: short write to %s", path);
  return 0;
}

int b200mlir_tensor_file_info(const char *path, int32_t *dtype_id, int64_t *rank, int64_t *dims, int64_t *data_bytes) {
  clear_error();
  if (!path) return set_error(B200MLIR_ERR_BAD_ARG, "tensor_file_info: null path");
  FileCloser fc{fopen(path, "rb")};
  if (!fc.f) return set_error(B200MLIR_ERR_BAD_ARG, "tensor_file_info: cannot open %s", path);
  int32_t id = -1;
  int64_t rk = -1, d[kMaxRank];
  if (fread(&id, sizeof(int32_t), 1, fc.f) != 1 || fread(&rk, sizeof(int64_t), 1, fc.f) != 1)
    return set_error(B200MLIR_ERR_BAD_ARG, "tensor_file_info: %s: truncated header", path);
  if (!b200mlir_dtype_size(id) || rk < 0 || rk > kMaxRank)
    return set_error(B200MLIR_ERR_BAD_ARG, "tensor_file_info: %s: dtype id %d / rank %lld not understood", path,
                     (int)id, (long long)rk);
  if (rk > 0 && fread(d, sizeof(int64_t), (size_t)rk, fc.f) != (size_t)rk)
    return set_error(B200MLIR_ERR_BAD_ARG, "tensor_file_info: %s: truncated shape", path);
  int64_t elems = 1;
  for (int64_t i = 0; i < rk; ++i) {
    if (d[i] < 0) return set_error(B200MLIR_ERR_BAD_ARG, "tensor_file_info: %s: negative extent", path);
    elems *= d[i];
  }
  const long header = ftell(fc.f);
  fseek(fc.f, 0, SEEK_END);
  const long total = ftell(fc.f);
  const int64_t want = elems * b200mlir_dtype_size(id);
  if (total - header != want)
    return set_error(B200MLIR_ERR_BAD_ARG, "tensor_file_info: %s: %ld data bytes, shape needs %lld", path,
                     total - header, (long long)want);
  if (dtype_id) *dtype_id = id;
  if (rank) *rank = rk;
  if (dims)
    for (int64_t i = 0; i < rk; ++i) dims[i] = d[i];
  if (data_bytes) *data_bytes = want;
  return 0;
}

// has_header != 0: an output file (header skipped); 0: an input file (raw data only).
int b200mlir_tensor_load(const char *path, int has_header, void *dst, int64_t bytes) {
  clear_error();
  if (!path || bytes < 0 || (bytes && !dst)) return set_error(B200MLIR_ERR_BAD_ARG, "tensor_load: bad arguments");
  int64_t rank = 0;
  if (has_header) B200_TRY(b200mlir_tensor_file_info(path, nullptr, &rank, nullptr, nullptr));
  FileCloser fc{fopen(path, "rb")};
  if (!fc.f) return set_error(B200MLIR_ERR_BAD_ARG, "tensor_load: cannot open %s", path);
  if (has_header) fseek(fc.f, (long)(4 + 8 + 8 * rank), SEEK_SET);
  std::vector<uint8_t> host;
  void *sink = dst;
  const bool dev = bytes && is_device_ptr(dst);
  if (dev) {
    host.resize((size_t)bytes);
    sink = host.data();
  }
  if (bytes && fread(sink, 1, (size_t)bytes, fc.f) != (size_t)bytes)
    return set_error(B200MLIR_ERR_BAD_ARG, "tensor_load: %s: unexpected end of file", path);
  if (dev) {
    B200_TRY(ensure_ready());
    B200_CUDA(cudaMemcpy(dst, host.data(), (size_t)bytes, cudaMemcpyHostToDevice));
  }
  return 0;
}

// result: 0 Pass, 1 Fail, anything else Unknown.  cycles < 0: no PerfPcycles line.
int b200mlir_perf_report_save(const char *path, const char *name, double perf, const char *units, int result,
                              long long cycles) {
  clear_error();
  if (!path || !name || !units) return set_error(B200MLIR_ERR_BAD_ARG, "perf_report_save: null argument");
  FileCloser fc{fopen(path, "w")};
  if (!fc.f) return set_error(B200MLIR_ERR_BAD_ARG, "perf_report_save: cannot open %s", path);
  const char *res = result == 0 ? "Pass" : result == 1 ? "Fail" : "Unknown";
  fprintf(fc.f, "Test_Info: {\n\tName:%s\n\tResult:%s\n\tPerf:%f\n\tUnits:%s\n}\n", name, res, perf, units);
  if (cycles >= 0) fprintf(fc.f, "PerfPcycles:%llu\n", (unsigned long long)cycles);
  return 0;
}

// The generated wrapper's timed section with its report: one discarded call, `iterations`
// timed calls, mean microseconds and mean SM cycles from the same pass, written to `path`
// (NULL: not written).  The cycle count is the difference of two SM clock stamps taken on
// the stream around the loop when both land on one SM, else time x the rated SM clock.
int b200mlir_benchmark_report(b200mlir_thunk fn, void *user, int iterations, const char *name, const char *path,
                              double *mean_us, long long *mean_cycles) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!fn || iterations < 1 || !name)
    return set_error(B200MLIR_ERR_BAD_ARG, "benchmark_report: null thunk / name, or iterations < 1");
  cudaStream_t s = ctx().stream;
  long long *stamps = nullptr;
  B200_CUDA(cudaMalloc(&stamps, 4 * sizeof(long long)));
  cudaEvent_t e0, e1;
  B200_CUDA(cudaEventCreate(&e0));
  B200_CUDA(cudaEventCreate(&e1));
  fn(user);  // discarded (hexagon_launcher_base.py:114-153)
  cudaStreamSynchronize(s);
  cudaEventRecord(e0, s);
  stamp_kernel<<<1, 1, 0, s>>>(stamps);
  for (int i = 0; i < iterations; ++i) fn(user);
  stamp_kernel<<<1, 1, 0, s>>>(stamps + 2);
  cudaEventRecord(e1, s);
  cudaError_t e = cudaEventSynchronize(e1);
  float ms = 0;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  long long h[4] = {0, 0, 0, 1};
  if (e == cudaSuccess) e = cudaMemcpy(h, stamps, sizeof(h), cudaMemcpyDeviceToHost);
  cudaFree(stamps);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (e != cudaSuccess) return set_error(B200MLIR_ERR_CUDA, "benchmark_report: %s", cudaGetErrorString(e));
  const double us = (double)ms * 1000.0 / iterations;
  long long cyc;
  if (h[1] == h[3] && h[2] > h[0]) {
    cyc = (h[2] - h[0]) / iterations;
  } else {
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx().device);
    cyc = (long long)(us * 1e-3 * khz);
  }
  if (mean_us) *mean_us = us;
  if (mean_cycles) *mean_cycles = cyc;
  char msg[256];
  const int code = b200mlir_last_error(msg, (int)sizeof(msg));  // an error recorded by the thunk's calls
  if (path) B200_TRY(b200mlir_perf_report_save(path, name, us, "us", code ? 1 : 0, cyc));
  if (code) return set_error(code, "%s", msg);
  return 0;
}

void b200mlir_manifest_reset(void) {
  std::lock_guard<std::mutex> lk(g_manifest_mu);
  g_manifest.clear();
}

int b200mlir_manifest_json(char *json, int cap) {
  std::ostringstream os;
  {
    std::lock_guard<std::mutex> lk(g_manifest_mu);
    os << "{\"matmuls\":[";
    for (size_t i = 0; i < g_manifest.size(); ++i) {
      const ManifestRow &r = g_manifest[i];
      os << (i ? "," : "") << "{\"plan\":\"" << r.plan << "\",\"reason\":\"" << r.reason << "\",\"detail\":\""
         << r.detail << "\",\"shape_mnk\":[" << r.m << "," << r.n << "," << r.k << "],\"epilogue\":\""
         << epilogue_name(r.epilogue) << "\",\"variant\":" << r.variant << ",\"name\":\"" << r.name
         << "\",\"launches\":" << r.count << "}";
    }
    os << "]}";
  }
  return put_string(os.str(), json, cap);
}

}  // extern "C"
