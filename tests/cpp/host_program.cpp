// A host program with no Python in it: plain C++ against include/b200mlir_capi.h, device memory
// through the runtime seam (hexagon_runtime_alloc_1d / _copy), the kernel entry points through
// their generated-wrapper convention.  One process per GPU: the parent forks `world` ranks, rank 0
// draws the tensor-parallel group's id and passes it down pipes, every rank runs
//   1. matmul            (fp16, checked against a CPU loop in this file)
//   2. mlp_block_tp_float16 over its shard of the hidden dimension (ncclAllReduce inside the call)
//   3. (two ranks or more) a host-buffer matmul whose A every rank holds: each rank uploads its row
//      slab of every panel and the slabs travel GPU to GPU inside the call
// and compares with the unsharded block / sampled rows computed on the CPU.  Exit code 0 when every rank agrees.
//   usage: host_program <world>
#include <sys/wait.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "b200mlir_capi.h"

typedef _Float16 f16;

static uint32_t g_state = 12345u;
static float uniform() {  // xorshift32: the same numbers in every rank
  g_state ^= g_state << 13; g_state ^= g_state >> 17; g_state ^= g_state << 5;
  return (float)(g_state >> 8) * (1.0f / 16777216.0f) * 2.0f - 1.0f;
}
static void fill(std::vector<f16> &v, float scale) { for (auto &e : v) e = (f16)(uniform() * scale); }

static int fail(int rank, const char *what) {
  char msg[512];
  int code = b200mlir_last_error(msg, sizeof(msg));
  fprintf(stderr, "rank %d: %s failed (code %d: %s)\n", rank, what, code, msg);
  return 1;
}

struct DevBuf {
  void *p = nullptr;
  explicit DevBuf(size_t bytes) { p = hexagon_runtime_alloc_1d(bytes, 256, false); }
  ~DevBuf() { if (p) hexagon_runtime_free_1d(p); }
};
static void up(void *dst, const void *src, size_t n) { hexagon_runtime_copy(dst, const_cast<void *>(src), n, false, false); }
static void down(void *dst, const void *src, size_t n) { hexagon_runtime_copy(dst, const_cast<void *>(src), n, false, false); }

static B200MemRef2D m2(void *p, int64_t r, int64_t c) { B200MemRef2D d; d.allocated = d.aligned = p; d.offset = 0; d.sizes[0] = r; d.sizes[1] = c; d.strides[0] = c; d.strides[1] = 1; return d; }
static B200MemRef1D m1(void *p, int64_t n) { B200MemRef1D d; d.allocated = d.aligned = p; d.offset = 0; d.sizes[0] = n; d.strides[0] = 1; return d; }

static void cpu_gemm(const f16 *a, const f16 *b, f16 *c, int m, int n, int k, int lda, int ldb, int ldc) {
  std::vector<float> acc(n);
  for (int i = 0; i < m; ++i) {
    std::fill(acc.begin(), acc.end(), 0.0f);
    for (int kk = 0; kk < k; ++kk) { const float av = (float)a[(size_t)i * lda + kk]; for (int j = 0; j < n; ++j) acc[j] += av * (float)b[(size_t)kk * ldb + j]; }
    for (int j = 0; j < n; ++j) c[(size_t)i * ldc + j] = (f16)acc[j];
  }
}
static double max_abs_rel(const std::vector<f16> &got, const std::vector<f16> &want) {
  double err = 0, ref = 1e-30;
  for (size_t i = 0; i < got.size(); ++i) { err = std::fmax(err, std::fabs((double)got[i] - (double)want[i])); ref = std::fmax(ref, std::fabs((double)want[i])); }
  return err / ref;
}

static int run_rank(int rank, int world, int id_read_fd, const std::vector<int> &id_write_fds) {
  if (b200mlir_init(rank) != 0) return fail(rank, "b200mlir_init");
  // ---- 1. matmul -----------------------------------------------------------------------------
  const int M = 384, N = 512, K = 320;
  std::vector<f16> a((size_t)M * K), b((size_t)K * N), c((size_t)M * N), want((size_t)M * N);
  fill(a, 1.0f); fill(b, 1.0f);
  cpu_gemm(a.data(), b.data(), want.data(), M, N, K, K, N, N);
  {
    DevBuf da(a.size() * 2), db(b.size() * 2), dc(c.size() * 2);
    if (!da.p || !db.p || !dc.p) return fail(rank, "alloc_1d");
    up(da.p, a.data(), a.size() * 2); up(db.p, b.data(), b.size() * 2);
    B200MemRef2D A = m2(da.p, M, K), B = m2(db.p, K, N), C = m2(dc.p, M, N);
    matmul(2, &A, 2, &B, 2, &C, 1, 1, 1, 0, 0, 0);
    char buf[8];
    if (b200mlir_last_error(buf, sizeof(buf)) != 0) return fail(rank, "matmul");
    down(c.data(), dc.p, c.size() * 2);
    if (b200mlir_device_status() != 0) return fail(rank, "device status after matmul");
  }
  const double e1 = max_abs_rel(c, want);
  printf("rank %d: matmul %dx%dx%d max-abs-rel %.2e\n", rank, M, N, K, e1);
  if (!(e1 <= 1e-2)) return 1;

  // ---- 2. the tensor-parallel group and the MLP block -----------------------------------------
  if (world > 1) {
    unsigned char id[128];
    if (rank == 0) {
      if (b200mlir_tp_unique_id(id) != 0) return fail(rank, "tp_unique_id");
      for (int fd : id_write_fds) if (write(fd, id, sizeof(id)) != (ssize_t)sizeof(id)) return 1;
    } else if (read(id_read_fd, id, sizeof(id)) != (ssize_t)sizeof(id)) {
      return 1;
    }
    if (b200mlir_tp_init(id, rank, world) != 0) return fail(rank, "tp_init");
  }
  int r = -1, w = -1;
  const int on = b200mlir_tp_info(&r, &w);
  if ((world > 1) != (on == 1) || r != (world > 1 ? rank : 0) || w != world) { fprintf(stderr, "rank %d: tp_info says %d %d %d\n", rank, on, r, w); return 1; }

  const int T = 512, D = 512, F = 1024;  // F / world columns per rank; two 256-row chunks of the down projection
  std::vector<f16> x((size_t)T * D), gain(D), wg((size_t)D * F), wu((size_t)D * F), wd((size_t)F * D);
  fill(x, 1.0f); for (auto &g : gain) g = (f16)(1.0f + 0.25f * uniform()); fill(wg, 0.05f); fill(wu, 0.05f); fill(wd, 0.05f);
  // the unsharded block on the CPU: rmsnorm -> gate/up -> silu(gate)*up -> down -> + x
  std::vector<f16> h((size_t)T * D), g1((size_t)T * F), u1((size_t)T * F), act((size_t)T * F), y((size_t)T * D), ref((size_t)T * D);
  for (int t = 0; t < T; ++t) {
    float ss = 0; for (int d = 0; d < D; ++d) { const float v = (float)x[(size_t)t * D + d]; ss += v * v; }
    const float inv = 1.0f / std::sqrt(ss / D + 1e-6f);
    for (int d = 0; d < D; ++d) h[(size_t)t * D + d] = (f16)((float)x[(size_t)t * D + d] * inv * (float)gain[d]);
  }
  cpu_gemm(h.data(), wg.data(), g1.data(), T, F, D, D, F, F);
  cpu_gemm(h.data(), wu.data(), u1.data(), T, F, D, D, F, F);
  for (size_t i = 0; i < act.size(); ++i) {
    const float g = (float)g1[i];
    const f16 e = (f16)std::exp(-g), den = (f16)(1.0f + (float)e), s = (f16)(g / (float)den);
    act[i] = (f16)((float)s * (float)u1[i]);
  }
  cpu_gemm(act.data(), wd.data(), y.data(), T, D, F, F, D, D);
  for (size_t i = 0; i < ref.size(); ++i) ref[i] = (f16)((float)y[i] + (float)x[i]);

  const int lo = rank * F / world, hi = (rank + 1) * F / world, fl = hi - lo;
  std::vector<f16> wg_s((size_t)D * fl), wu_s((size_t)D * fl);
  for (int d = 0; d < D; ++d) { memcpy(&wg_s[(size_t)d * fl], &wg[(size_t)d * F + lo], fl * 2); memcpy(&wu_s[(size_t)d * fl], &wu[(size_t)d * F + lo], fl * 2); }
  std::vector<f16> out((size_t)T * D);
  {
    DevBuf dx(x.size() * 2), dg(D * 2), dwg(wg_s.size() * 2), dwu(wu_s.size() * 2), dwd((size_t)fl * D * 2), dout(out.size() * 2);
    if (!dx.p || !dg.p || !dwg.p || !dwu.p || !dwd.p || !dout.p) return fail(rank, "alloc_1d");
    up(dx.p, x.data(), x.size() * 2); up(dg.p, gain.data(), D * 2); up(dwg.p, wg_s.data(), wg_s.size() * 2);
    up(dwu.p, wu_s.data(), wu_s.size() * 2); up(dwd.p, &wd[(size_t)lo * D], (size_t)fl * D * 2);
    B200MemRef2D X = m2(dx.p, T, D), WG = m2(dwg.p, D, fl), WU = m2(dwu.p, D, fl), WD = m2(dwd.p, fl, D), O = m2(dout.p, T, D);
    B200MemRef1D G = m1(dg.p, D);
    for (int chunks = 1; chunks <= 2; ++chunks) {
      mlp_block_tp_float16(2, &X, 1, &G, 2, &WG, 2, &WU, 2, &WD, 2, &O, 1e-6f, chunks, 1, 1, 1, 0, 0, 0);
      char buf[8];
      if (b200mlir_last_error(buf, sizeof(buf)) != 0) return fail(rank, "mlp_block_tp_float16");
      if (b200mlir_synchronize() != 0) return fail(rank, "synchronize");
      down(out.data(), dout.p, out.size() * 2);
      if (b200mlir_device_status() != 0) return fail(rank, "device status after the block");
      const double e2 = max_abs_rel(out, ref);
      printf("rank %d of %d: mlp block (chunks %d) max-abs-rel %.2e\n", rank, world, chunks, e2);
      if (!(e2 <= 1e-2)) return 1;
    }
  }
  // ---- 3. host-buffer matmul, A replicated over the ranks ---------------------------------------
  if (world > 1) {
    const int M3 = 8192, K3 = 2048, N3 = 4096;
    std::vector<f16> a3((size_t)M3 * K3), b3((size_t)K3 * N3), c3((size_t)M3 * N3);
    g_state = 777u;
    fill(a3, 1.0f);  // the same A on every rank
    g_state = 1000u + (uint32_t)rank;
    fill(b3, 1.0f);  // this rank's column block of B
    int64_t panels[4] = {0, 0, 0, 0};
    if (b200mlir_host_gemm_plan(M3, N3, K3, panels) != 1 || panels[2] < 2) { fprintf(stderr, "rank %d: host_gemm_plan\n", rank); return 1; }
    B200MemRef2D A3 = m2(a3.data(), M3, K3), B3 = m2(b3.data(), K3, N3), C3 = m2(c3.data(), M3, N3);
    b200mlir_set_option("replicatedOperandA", 1.0);
    matmul(2, &A3, 2, &B3, 2, &C3, 1, 1, 1, 0, 0, 0);
    b200mlir_set_option("replicatedOperandA", 0.0);
    char buf[8];
    if (b200mlir_last_error(buf, sizeof(buf)) != 0) return fail(rank, "matmul with a replicated A");
    if (b200mlir_device_status() != 0) return fail(rank, "device status after the host-buffer matmul");
    double e3 = 0;
    std::vector<f16> got(N3), want(N3);
    for (int i = 0; i < 16; ++i) {  // sampled rows, one in every panel
      const int row = i * (M3 / 16) + 37 * i % (M3 / 16);
      cpu_gemm(&a3[(size_t)row * K3], b3.data(), want.data(), 1, N3, K3, K3, N3, N3);
      memcpy(got.data(), &c3[(size_t)row * N3], (size_t)N3 * 2);
      e3 = std::fmax(e3, max_abs_rel(got, want));
    }
    const int mode = b200mlir_tp_slab_exchange_mode();
    printf("rank %d of %d: host-buffer matmul, replicated A, %lld x %lld panels, slabs by %s, max-abs-rel %.2e\n", rank, world,
           (long long)panels[2], (long long)panels[3], mode == 1 ? "copy engines" : mode == 2 ? "ncclAllGather" : "nothing", e3);
    if (!(e3 <= 1e-2) || mode == 0) return 1;
  }
  if (b200mlir_tp_shutdown() != 0) return fail(rank, "tp_shutdown");
  return 0;
}

int main(int argc, char **argv) {
  const int world = argc > 1 ? atoi(argv[1]) : 1;
  if (world < 1 || world > 8) { fprintf(stderr, "usage: host_program <world 1..8>\n"); return 2; }
  std::vector<int> rd(world, -1), wr;
  for (int r = 1; r < world; ++r) { int p[2]; if (pipe(p) != 0) return 2; rd[r] = p[0]; wr.push_back(p[1]); }
  std::vector<pid_t> kids;
  for (int r = 0; r < world; ++r) {
    pid_t pid = fork();
    if (pid == 0) {
      const int rc = run_rank(r, world, rd[r], wr);
      fflush(stdout);
      fflush(stderr);
      _exit(rc);
    }
    kids.push_back(pid);
  }
  int bad = 0;
  for (pid_t k : kids) { int st = 0; waitpid(k, &st, 0); bad |= !(WIFEXITED(st) && WEXITSTATUS(st) == 0); }
  printf(bad ? "FAILED\n" : "all ranks ok\n");
  return bad;
}
