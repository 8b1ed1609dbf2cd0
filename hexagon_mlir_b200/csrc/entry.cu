// Seam 1: the kernel entry points, in the calling convention of the reference's
// generated wrapper (backend/hexagon_launcher_base.py:58-60,72-74;
// backend/triton_hexagon_launcher.py:241-252).  Validates descriptors, stages
// host tensors through device memory, and hands device pointers to the
// dispatcher.  Nothing here computes on the CPU.
#include <algorithm>
#include <cstdlib>
#include <functional>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.h"

namespace b200 {
namespace {

// Host tensors are copied to stream-ordered device temporaries and back.
class Stager {
 public:
  ~Stager() { release(); }
  // Returns a device pointer for `p` (p itself when it already is one).
  int in(const void *p, size_t bytes, const void **dev) {
    if (!p || bytes == 0 || is_device_ptr(p)) {
      *dev = p;
      return 0;
    }
    void *d = nullptr;
    B200_CUDA(cudaMallocAsync(&d, bytes, ctx().stream));
    items_.push_back({d, nullptr, 0});
    B200_CUDA(cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, ctx().stream));
    *dev = d;
    return 0;
  }
  int out(void *p, size_t bytes, void **dev, bool preload = false) {
    if (!p || bytes == 0 || is_device_ptr(p)) {
      *dev = p;
      return 0;
    }
    void *d = nullptr;
    B200_CUDA(cudaMallocAsync(&d, bytes, ctx().stream));
    items_.push_back({d, p, bytes});
    if (preload) B200_CUDA(cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, ctx().stream));
    *dev = d;
    host_out_ = true;
    return 0;
  }
  // Copy results back and wait when any tensor lived on the host.
  int finish() {
    for (auto &it : items_)
      if (it.host) B200_CUDA(cudaMemcpyAsync(it.host, it.dev, it.bytes, cudaMemcpyDeviceToHost, ctx().stream));
    int rc = 0;
    if (!items_.empty()) {
      cudaError_t e = cudaStreamSynchronize(ctx().stream);
      if (e != cudaSuccess) rc = set_error(B200MLIR_ERR_CUDA, "stream sync failed: %s", cudaGetErrorString(e));
    }
    release();
    return rc;
  }

 private:
  struct Item {
    void *dev;
    void *host;
    size_t bytes;
  };
  void release() {
    for (auto &it : items_) cudaFreeAsync(it.dev, ctx().stream);
    items_.clear();
  }
  std::vector<Item> items_;
  bool host_out_ = false;
};

struct View2 {
  void *p;
  int64_t rows, cols, ld;
  size_t span(size_t esz) const { return rows > 0 && cols > 0 ? ((size_t)(rows - 1) * ld + cols) * esz : 0; }
};
struct View1 {
  void *p;
  int64_t n;
};

int view2(const char *what, int64_t rank, const B200MemRef2D *d, size_t esz, View2 *v) {
  if (rank != 2 || !d)
    return set_error(B200MLIR_ERR_BAD_ARG, "%s: expected a rank-2 memref descriptor (got rank %lld)", what, (long long)rank);
  if (d->sizes[0] < 0 || d->sizes[1] < 0)
    return set_error(B200MLIR_ERR_BAD_ARG, "%s: negative extent", what);
  const bool empty = d->sizes[0] == 0 || d->sizes[1] == 0;
  if (!empty && d->sizes[1] > 1 && d->strides[1] != 1)
    return set_error(B200MLIR_ERR_BAD_ARG, "%s: innermost stride must be 1 (dense rows)", what);
  if (!empty && d->sizes[0] > 1 && d->strides[0] < d->sizes[1])
    return set_error(B200MLIR_ERR_BAD_ARG, "%s: row stride %lld below row length %lld", what,
                     (long long)d->strides[0], (long long)d->sizes[1]);
  if (!d->aligned && d->sizes[0] * d->sizes[1] != 0)
    return set_error(B200MLIR_ERR_BAD_ARG, "%s: null data pointer", what);
  v->p = (char *)d->aligned + d->offset * (int64_t)esz;
  v->rows = d->sizes[0];
  v->cols = d->sizes[1];
  v->ld = d->sizes[0] > 1 ? d->strides[0] : d->sizes[1];
  if (v->ld < v->cols) v->ld = v->cols;
  return 0;
}

int view1(const char *what, int64_t rank, const B200MemRef1D *d, size_t esz, View1 *v) {
  if (rank != 1 || !d)
    return set_error(B200MLIR_ERR_BAD_ARG, "%s: expected a rank-1 memref descriptor (got rank %lld)", what, (long long)rank);
  if (d->sizes[0] < 0) return set_error(B200MLIR_ERR_BAD_ARG, "%s: negative extent", what);
  if (d->sizes[0] > 1 && d->strides[0] != 1)
    return set_error(B200MLIR_ERR_BAD_ARG, "%s: stride must be 1", what);
  if (!d->aligned && d->sizes[0] != 0) return set_error(B200MLIR_ERR_BAD_ARG, "%s: null data pointer", what);
  v->p = (char *)d->aligned + d->offset * (int64_t)esz;
  v->n = d->sizes[0];
  return 0;
}

inline bool not_first_program(int px, int py, int pz) { return (px | py | pz) != 0; }

int check_grid(int nx, int ny, int nz, int px, int py, int pz) {
  if (nx < 1 || ny < 1 || nz < 1 || px < 0 || py < 0 || pz < 0 || px >= nx || py >= ny || pz >= nz)
    return set_error(B200MLIR_ERR_BAD_ARG, "program id (%d,%d,%d) outside grid (%d,%d,%d)", px, py, pz, nx, ny, nz);
  return 0;
}

// fp16 GEMM whose three tensors live in host memory, large enough that the PCIe transfers
// dominate: A is cut into row panels and B into column panels, panels go up in the order
// A0 B0 A1 B1 ..., the strips of C that a panel completes are computed as soon as it has landed and go
// back down on a third stream while later panels are still on their way up.  The link is
// full duplex, so the call approaches max(bytes up, bytes down) / link rate instead of their sum.
constexpr size_t kPipelineMinBytes = 96u << 20;

// Which host-buffer fp16 GEMMs take the pipelined path, and their panels: about 1024 rows of A and
// 1024 columns of B per panel, at most 16 of each, counted separately (a narrow column block — one
// rank's share of a wide B — still gets a fine-grained pipeline over A); panel edges on multiples
// of 256 (whole tiles of the widest variant).
struct HostGemmPlan {
  bool pipelined;
  int64_t pm, pn, PM, PN;  // panel height / width, panel counts
};
HostGemmPlan host_gemm_plan(int64_t M, int64_t N, int64_t K) {
  HostGemmPlan h{};
  h.pipelined = K > 0 && std::min(M, N) >= 1024 && std::max(M, N) >= 4096 && K % 8 == 0 && N % 8 == 0 &&
                (size_t)(M * K + K * N + M * N) * 2 >= kPipelineMinBytes;
  if (!h.pipelined) return h;
  const int64_t P_m = std::max<int64_t>(2, std::min<int64_t>(16, M / 1024));
  const int64_t P_n = std::max<int64_t>(1, std::min<int64_t>(16, N / 1024));
  h.pm = ((M + P_m - 1) / P_m + 255) / 256 * 256;
  h.pn = ((N + P_n - 1) / P_n + 255) / 256 * 256;
  h.PM = (M + h.pm - 1) / h.pm;
  h.PN = (N + h.pn - 1) / h.pn;
  return h;
}

int matmul_host_pipelined(const View2 &A, const View2 &B, const View2 &C) {
  const int64_t M = A.rows, K = A.cols, N = B.cols;
  const HostGemmPlan hp = host_gemm_plan(M, N, K);
  const int64_t pm = hp.pm, pn = hp.pn, PM = hp.PM, PN = hp.PN;
  // option replicatedOperandA inside a tensor-parallel group: a collective call — every rank
  // enters with the same M and K (its own B and C column block)
  const int world = ctx().opt.replicated_operand_a != 0 ? tp_world() : 1;
  cudaStream_t s_in, s_out, s_ag = nullptr, s = ctx().stream;
  B200_TRY(copy_streams(&s_in, &s_out));
  const size_t a_bytes = (size_t)M * K * 2, b_bytes = (size_t)K * N * 2, c_bytes = (size_t)M * N * 2;
  // The slabs travel between the GPUs by copy engines into windows the ranks map from each other
  // (no kernel, so nothing competes with the strip GEMMs for SMs); where the machine gives no such
  // mapping, by ncclAllGather on the communicator's stream.
  SlabExchange xc;
  if (world > 1) {
    B200_TRY(tp_slab_exchange_begin(a_bytes, &xc));
    B200_TRY(tp_comm_stream(&s_ag));
    if (xc.a) s_ag = xc.push;
  }
  void *base = nullptr;
  const size_t a_staged = xc.a ? 0 : a_bytes;  // A lives in the exchange window when there is one
  B200_TRY(staging_workspace(a_staged + b_bytes + c_bytes + 512, &base));
  __half *dA = xc.a ? (__half *)xc.a : (__half *)base;
  __half *dB = (__half *)((char *)base + ((a_staged + 255) & ~(size_t)255));
  __half *dC = (__half *)((char *)dB + ((b_bytes + 255) & ~(size_t)255));
  std::vector<cudaEvent_t> ev;
  const bool debug = getenv("B200MLIR_DEBUG") != nullptr;  // timed events, and a timeline printed at the end
  std::vector<std::pair<const char *, cudaEvent_t>> marks;
  auto new_event = [&](cudaEvent_t *e) -> cudaError_t {
    cudaError_t r = cudaEventCreateWithFlags(e, debug ? cudaEventDefault : cudaEventDisableTiming);
    if (r == cudaSuccess) ev.push_back(*e);
    return r;
  };
  int rc = 0;
  cudaError_t e = cudaSuccess;
  std::vector<cudaEvent_t> a_up(PM), b_up(PN);
  cudaEvent_t start, done;
#define PIPE_CUDA(expr)                                                                      \
  if (rc == 0 && (e = (expr)) != cudaSuccess)                                                 \
  rc = set_error(B200MLIR_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e))
  // the copy streams start after whatever the caller queued before this call
  cudaEvent_t t0 = nullptr;
  if (debug) { cudaEventCreate(&t0); cudaEventRecord(t0, s); }
  PIPE_CUDA(new_event(&start));
  PIPE_CUDA(cudaEventRecord(start, s));
  PIPE_CUDA(cudaStreamWaitEvent(s_in, start, 0));
  PIPE_CUDA(cudaStreamWaitEvent(s_out, start, 0));
  if (s_ag) PIPE_CUDA(cudaStreamWaitEvent(s_ag, start, 0));
  for (int64_t d = 0; d < std::max(PM, PN) && rc == 0; ++d) {
    bool exchanged_by_flags = false;
    if (d < PM) {
      const int64_t r0 = d * pm, rows = std::min(pm, M - r0);
      if (world > 1 && rows % world == 0) {
        // every rank holds the same A: this rank sends up only its slab of the panel over its own
        // PCIe link, and the slabs are exchanged GPU to GPU (an in-place all-gather over NVLink)
        const int64_t slab = rows / world, s0 = r0 + (int64_t)tp_rank() * slab;
        PIPE_CUDA(cudaMemcpy2DAsync(dA + s0 * K, (size_t)K * 2, (const __half *)A.p + s0 * A.ld, (size_t)A.ld * 2,
                                    (size_t)K * 2, (size_t)slab, cudaMemcpyHostToDevice, s_in));
        cudaEvent_t slab_up;
        PIPE_CUDA(new_event(&slab_up));
        PIPE_CUDA(cudaEventRecord(slab_up, s_in));
        PIPE_CUDA(cudaStreamWaitEvent(s_ag, slab_up, 0));
        if (xc.a && d < kExchangePanels) {
          const size_t off = (size_t)s0 * K * 2, bytes = (size_t)slab * K * 2;
          const int me = tp_rank();
          for (int i = 1; i < world; ++i) {  // each rank starts at its right-hand neighbour
            const int peer = (me + i) % world;
            PIPE_CUDA(cudaMemcpyAsync(xc.peer_a[peer] + off, xc.a + off, bytes, cudaMemcpyDefault, s_ag));
            PIPE_CUDA(cudaMemcpyAsync(xc.peer_flags[peer] + d * kMaxPushRanks + me, xc.d_seq, 4, cudaMemcpyDefault, s_ag));
          }
          a_up[d] = slab_up;          // the compute stream waits for this rank's slab by event ...
          exchanged_by_flags = true;  // ... and for the others' by their flags
        } else {
          if (rc == 0) rc = tp_all_gather_bytes(dA + s0 * K, dA + r0 * K, (size_t)slab * K * 2, s_ag);
          PIPE_CUDA(new_event(&a_up[d]));
          PIPE_CUDA(cudaEventRecord(a_up[d], s_ag));
        }
        if (debug) { marks.push_back({"slab up", slab_up}); marks.push_back({"slabs exchanged", a_up[d]}); }
      } else {
        PIPE_CUDA(cudaMemcpy2DAsync(dA + r0 * K, (size_t)K * 2, (const __half *)A.p + r0 * A.ld, (size_t)A.ld * 2,
                                    (size_t)K * 2, (size_t)rows, cudaMemcpyHostToDevice, s_in));
        PIPE_CUDA(new_event(&a_up[d]));
        PIPE_CUDA(cudaEventRecord(a_up[d], s_in));
      }
    }
    if (d < PN) {
      const int64_t c0 = d * pn, cols = std::min(pn, N - c0);
      PIPE_CUDA(cudaMemcpy2DAsync(dB + c0, (size_t)N * 2, (const __half *)B.p + c0, (size_t)B.ld * 2,
                                  (size_t)cols * 2, (size_t)K, cudaMemcpyHostToDevice, s_in));
      PIPE_CUDA(new_event(&b_up[d]));
      PIPE_CUDA(cudaEventRecord(b_up[d], s_in));
      if (debug) marks.push_back({"B panel up", b_up[d]});
    }
    // what panel d completes: the row strip (row panel d x column panels 0..d) and the column
    // strip (row panels 0..d-1 x column panel d); one GEMM and one copy down for each
    for (int strip = 0; strip < 2 && rc == 0; ++strip) {
      int64_t r0, rows, c0, cols;
      if (strip == 0) {
        if (d >= PM) continue;
        r0 = d * pm; rows = std::min(pm, M - r0);
        c0 = 0; cols = std::min((d + 1) * pn, N);
      } else {
        if (d >= PN || d == 0) continue;
        r0 = 0; rows = std::min(d * pm, M);
        c0 = d * pn; cols = std::min(pn, N - c0);
      }
      if (rows <= 0 || cols <= 0) continue;
      if (d < PM) PIPE_CUDA(cudaStreamWaitEvent(s, a_up[d], 0));
      if (d < PN) PIPE_CUDA(cudaStreamWaitEvent(s, b_up[d], 0));
      if (exchanged_by_flags && rc == 0) {
        rc = tp_slab_exchange_wait(xc, (int)d, s);
        exchanged_by_flags = false;  // once per panel: the column strip follows on the same stream
      }
      GemmArgs g;
      g.a = dA + r0 * K; g.b = dB + c0; g.c = dC + r0 * N + c0;
      g.m = rows; g.n = cols; g.k = K;
      g.lda = K; g.ldb = N; g.ldc = N;
      g.epilogue = EPI_F16;
      if (rc == 0) rc = gemm_dispatch(g);
      cudaEvent_t blk;
      PIPE_CUDA(new_event(&blk));
      PIPE_CUDA(cudaEventRecord(blk, s));
      PIPE_CUDA(cudaStreamWaitEvent(s_out, blk, 0));
      PIPE_CUDA(cudaMemcpy2DAsync((__half *)C.p + r0 * C.ld + c0, (size_t)C.ld * 2, dC + r0 * N + c0, (size_t)N * 2,
                                  (size_t)cols * 2, (size_t)rows, cudaMemcpyDeviceToHost, s_out));
      if (debug && rc == 0) {
        cudaEvent_t dn;
        PIPE_CUDA(new_event(&dn));
        PIPE_CUDA(cudaEventRecord(dn, s_out));
        marks.push_back({strip == 0 ? "row strip computed" : "column strip computed", blk});
        marks.push_back({"strip down", dn});
      }
    }
  }
  cudaEvent_t t_up = nullptr, t_mm = nullptr, t_down = nullptr;
  if (debug) {
    cudaEventCreate(&t_up); cudaEventCreate(&t_mm); cudaEventCreate(&t_down);
    cudaEventRecord(t_up, s_in); cudaEventRecord(t_mm, s); cudaEventRecord(t_down, s_out);
  }
  // the caller's stream continues after the last copy down; the call itself waits for it
  PIPE_CUDA(new_event(&done));
  PIPE_CUDA(cudaEventRecord(done, s_out));
  PIPE_CUDA(cudaStreamWaitEvent(s, done, 0));
#undef PIPE_CUDA
  cudaError_t e1 = cudaStreamSynchronize(s_in), e2 = cudaStreamSynchronize(s_out), e3 = cudaStreamSynchronize(s);
  if (s_ag && e1 == cudaSuccess) e1 = cudaStreamSynchronize(s_ag);
  if (debug) {  // B200MLIR_DEBUG: when each of the three streams finished
    float a = 0, b = 0, c = 0;
    cudaEventElapsedTime(&a, t0, t_up); cudaEventElapsedTime(&b, t0, t_mm); cudaEventElapsedTime(&c, t0, t_down);
    fprintf(stderr, "[b200mlir] pipelined host GEMM %lldx%lldx%lld panels %lldx%lld%s: up done %.2f ms, compute done %.2f ms, down done %.2f ms\n",
            (long long)M, (long long)N, (long long)K, (long long)PM, (long long)PN,
            world == 1 ? "" : xc.a ? ", slabs by copy engines" : ", slabs by ncclAllGather", a, b, c);
    if (getenv("B200MLIR_DEBUG")[0] == '2' && tp_rank() == 0)
      for (auto &mk : marks) {
        float t = 0;
        if (cudaEventElapsedTime(&t, t0, mk.second) == cudaSuccess) fprintf(stderr, "[b200mlir]   %8.3f ms  %s\n", t, mk.first);
      }
    cudaEventDestroy(t0); cudaEventDestroy(t_up); cudaEventDestroy(t_mm); cudaEventDestroy(t_down);
  }
  for (cudaEvent_t x : ev) cudaEventDestroy(x);
  if (rc == 0 && (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess))
    rc = set_error(B200MLIR_ERR_CUDA, "pipelined host GEMM: %s",
                   cudaGetErrorString(e1 != cudaSuccess ? e1 : e2 != cudaSuccess ? e2 : e3));
  return rc;
}

int matmul_impl(int epilogue, int64_t ra, B200MemRef2D *a, int64_t rb, B200MemRef2D *b, int64_t rc,
                B200MemRef2D *c, int64_t rr, B200MemRef2D *res) {
  B200_TRY(ensure_ready());
  View2 A, B, C, R{nullptr, 0, 0, 0};
  const size_t c_esz = epilogue == EPI_F32_RES ? 4 : 2;
  B200_TRY(view2("A", ra, a, 2, &A));
  B200_TRY(view2("B", rb, b, 2, &B));
  B200_TRY(view2("C", rc, c, c_esz, &C));
  const bool has_res = epilogue == EPI_F32_RES && rr != 0 && res && res->aligned;
  if (has_res) B200_TRY(view2("residual", rr, res, 4, &R));
  if (A.cols != B.rows || C.rows != A.rows || C.cols != B.cols)
    return set_error(B200MLIR_ERR_BAD_ARG, "matmul: shapes [%lld,%lld]x[%lld,%lld]->[%lld,%lld] do not agree",
                     (long long)A.rows, (long long)A.cols, (long long)B.rows, (long long)B.cols,
                     (long long)C.rows, (long long)C.cols);
  if (has_res && (R.rows != C.rows || R.cols != C.cols))
    return set_error(B200MLIR_ERR_BAD_ARG, "matmul: residual shape differs from C");
  if (C.rows == 0 || C.cols == 0) return 0;
  if (epilogue == EPI_F16 && host_gemm_plan(A.rows, B.cols, A.cols).pipelined && !is_device_ptr(A.p) && !is_device_ptr(B.p) &&
      !is_device_ptr(C.p))
    return matmul_host_pipelined(A, B, C);
  Stager st;
  GemmArgs g;
  B200_TRY(st.in(A.p, A.span(2), &g.a));
  B200_TRY(st.in(B.p, B.span(2), &g.b));
  // C rows may be a strided view into a wider matrix: keep the bytes between rows
  B200_TRY(st.out(C.p, C.span(c_esz), &g.c, C.ld != C.cols));
  if (has_res) B200_TRY(st.in(R.p, R.span(4), &g.res));
  g.m = A.rows; g.n = B.cols; g.k = A.cols;
  g.lda = A.ld; g.ldb = B.ld; g.ldc = C.ld; g.ldres = R.ld;
  g.epilogue = epilogue;
  g.block_k = (int)ctx().opt.kloop_block_k;
  B200_TRY(gemm_dispatch(g));
  return st.finish();
}

// ---- w8a16 resident weights --------------------------------------------------------------
std::mutex g_w_mu;
std::unordered_map<const void *, W8A16Weight> g_weights;

int register_weight_locked(const void *wq, const void *scales, int64_t k, int64_t n, int l2_persist,
                           W8A16Weight **out) {
  auto it = g_weights.find(wq);
  if (it != g_weights.end()) {
    W8A16Weight &e = it->second;
    if (e.k != k || e.n != n)
      return set_error(B200MLIR_ERR_BAD_ARG, "w8a16: weight at %p re-registered with a different shape", wq);
    if (e.scales != scales) {
      // same weight bytes under other scales: the image (scale-free) stays, the device copy of the
      // scales is refreshed and the expanded fp16 weight, which has the scales folded in, is dropped
      cudaError_t ce = cudaMemcpyAsync(e.scales_dev, scales, (size_t)n * 2, cudaMemcpyDefault, ctx().stream);
      if (ce == cudaSuccess) ce = cudaStreamSynchronize(ctx().stream);
      if (ce != cudaSuccess) return set_error(B200MLIR_ERR_CUDA, "w8a16: scales copy failed: %s", cudaGetErrorString(ce));
      if (e.w16) cudaFree(e.w16);
      e.w16 = nullptr;
      e.scales = scales;
    }
    if (l2_persist && !e.l2_persist) {
      e.l2_persist = true;
      l2_window_set(e.image, e.image_bytes);
    }
    if (out) *out = &e;
    return 0;
  }
  Context &c = ctx();
  W8A16Weight w;
  w.src = wq; w.scales = scales; w.k = k; w.n = n; w.l2_persist = l2_persist != 0;
  const int8_t *wq_dev = (const int8_t *)wq;
  void *tmp = nullptr;
  if (!is_device_ptr(wq)) {
    B200_CUDA(cudaMalloc(&tmp, (size_t)k * n));
    B200_CUDA(cudaMemcpyAsync(tmp, wq, (size_t)k * n, cudaMemcpyHostToDevice, c.stream));
    wq_dev = (const int8_t *)tmp;
  }
  int rc = w8a16_build_tmem_image(wq_dev, k, n, &w.image, &w.image_bytes);
  if (rc == 0) {
    cudaError_t e = cudaMalloc(&w.scales_dev, (size_t)n * 2);
    if (e == cudaSuccess) e = cudaMemcpyAsync(w.scales_dev, scales, (size_t)n * 2, cudaMemcpyDefault, c.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c.stream);
    if (e != cudaSuccess) rc = set_error(B200MLIR_ERR_CUDA, "w8a16: scales copy failed: %s", cudaGetErrorString(e));
  }
  if (tmp) cudaFree(tmp);
  if (rc) {
    if (w.image) cudaFree(w.image);
    if (w.scales_dev) cudaFree(w.scales_dev);
    return rc;
  }
  // Decode GEMMs re-read the same image every call: pin as much of it as the device allows in
  // L2.  The window follows the calling thread's stream (b200mlir_set_stream re-applies it).
  if (w.l2_persist) l2_window_set(w.image, w.image_bytes);
  auto ins = g_weights.emplace(wq, w);
  if (out) *out = &ins.first->second;
  return 0;
}

}  // namespace
}  // namespace b200

using namespace b200;

#define ENTER_KERNEL()                                                                     \
  clear_error();                                                                           \
  if (check_grid(num_programs_x, num_programs_y, num_programs_z, pid_x, pid_y, pid_z)) return; \
  if (not_first_program(pid_x, pid_y, pid_z)) return

extern "C" {

void matmul(int64_t ra, B200MemRef2D *a, int64_t rb, B200MemRef2D *b, int64_t rc, B200MemRef2D *c,
            B200_GRID_ARGS) {
  ENTER_KERNEL();
  matmul_impl(EPI_F16, ra, a, rb, b, rc, c, 0, nullptr);
}

void multispan_matmul(int64_t ra, B200MemRef2D *a, int64_t rb, B200MemRef2D *b, int64_t rc, B200MemRef2D *c,
                      B200_GRID_ARGS) {
  // spans are a tiling the caller's kernel expresses; one call covers every span
  ENTER_KERNEL();
  matmul_impl(EPI_F16, ra, a, rb, b, rc, c, 0, nullptr);
}

void klooped_matmul(int64_t ra, B200MemRef2D *a, int64_t rb, B200MemRef2D *b, int64_t rc,
                    B200MemRef2D *c, B200_GRID_ARGS) {
  ENTER_KERNEL();
  matmul_impl(EPI_KLOOP_F16, ra, a, rb, b, rc, c, 0, nullptr);
}

void matmul_f32out(int64_t ra, B200MemRef2D *a, int64_t rb, B200MemRef2D *b, int64_t rc,
                   B200MemRef2D *c32, int64_t rr, B200MemRef2D *res32, B200_GRID_ARGS) {
  ENTER_KERNEL();
  matmul_impl(EPI_F32_RES, ra, a, rb, b, rc, c32, rr, res32);
}

void matmul_i8(int64_t ra, B200MemRef2D *a, int64_t rb, B200MemRef2D *b, int64_t rc, B200MemRef2D *c,
               B200_GRID_ARGS) {
  ENTER_KERNEL();
  if (ensure_ready()) return;
  View2 A, B, C;
  if (view2("A", ra, a, 1, &A) || view2("B", rb, b, 1, &B) || view2("C", rc, c, 4, &C)) return;
  if (A.cols != B.rows || C.rows != A.rows || C.cols != B.cols) {
    set_error(B200MLIR_ERR_BAD_ARG, "matmul_i8: shapes do not agree");
    return;
  }
  if (C.rows == 0 || C.cols == 0) return;
  Stager st;
  const void *da, *db;
  void *dc;
  if (st.in(A.p, A.span(1), &da) || st.in(B.p, B.span(1), &db) || st.out(C.p, C.span(4), &dc, C.ld != C.cols)) return;
  // Tensor cores (kind::i8, exact int32 sums) when the operands meet the TMA alignment and the
  // problem fills a few tiles; B is transposed once into the workspace because both int8 operands
  // are read K-major.  Everything else takes the CUDA-core loop.  Both are exact.
  const int64_t M = A.rows, N = B.cols, K = A.cols;
  const bool tc = ctx().opt.gemm_variant != -2 && M >= 64 && N >= 64 && K >= 64 && N % 4 == 0 && A.ld % 16 == 0 &&
                  C.ld % 4 == 0 && ((uintptr_t)da & 15) == 0 && ((uintptr_t)dc & 15) == 0;
  if (tc) {
    const int64_t ldbt = (K + 15) / 16 * 16;
    void *bt = nullptr;
    if (workspace((size_t)N * ldbt, &bt)) return;
    if (launch_transpose_i8((const int8_t *)db, (int8_t *)bt, K, N, B.ld, ldbt)) return;
    if (launch_gemm_i8_tc((const int8_t *)da, (const int8_t *)bt, (int32_t *)dc, M, N, K, A.ld, ldbt, C.ld)) return;
  } else if (launch_gemm_i8_simt((const int8_t *)da, (const int8_t *)db, (int32_t *)dc, M, N, K, A.ld, B.ld, C.ld)) {
    return;
  }
  st.finish();
}

static void softmax_impl(bool f16, int64_t rx, B200MemRef2D *x, int64_t ry, B200MemRef2D *y) {
  if (ensure_ready()) return;
  const size_t esz = f16 ? 2 : 4;
  View2 X, Y;
  if (view2("x", rx, x, esz, &X) || view2("output", ry, y, esz, &Y)) return;
  if (X.rows != Y.rows || X.cols != Y.cols) {
    set_error(B200MLIR_ERR_BAD_ARG, "softmax: input and output shapes differ");
    return;
  }
  if (X.rows == 0 || X.cols == 0) return;
  Stager st;
  const void *dx;
  void *dy;
  if (st.in(X.p, X.span(esz), &dx) || st.out(Y.p, Y.span(esz), &dy, Y.ld != Y.cols)) return;
  int rc = f16 ? launch_softmax_f16((const __half *)dx, (__half *)dy, X.rows, X.cols, X.ld, Y.ld)
               : launch_softmax_f32((const float *)dx, (float *)dy, X.rows, X.cols, X.ld, Y.ld);
  if (rc) return;
  st.finish();
}

void softmax_kernel_float16(int64_t rx, B200MemRef2D *x, int64_t ry, B200MemRef2D *y, B200_GRID_ARGS) {
  ENTER_KERNEL();
  softmax_impl(true, rx, x, ry, y);
}
void softmax_kernel_float32(int64_t rx, B200MemRef2D *x, int64_t ry, B200MemRef2D *y, B200_GRID_ARGS) {
  ENTER_KERNEL();
  softmax_impl(false, rx, x, ry, y);
}

static void rmsnorm_impl(bool f16, int64_t rx, B200MemRef2D *x, int64_t ry, B200MemRef2D *y, int64_t rw,
                         B200MemRef1D *w) {
  if (ensure_ready()) return;
  const size_t esz = f16 ? 2 : 4;
  View2 X, Y;
  View1 W;
  if (view2("x", rx, x, esz, &X) || view2("y", ry, y, esz, &Y) || view1("weights", rw, w, esz, &W)) return;
  if (X.rows != Y.rows || X.cols != Y.cols || W.n != X.cols) {
    set_error(B200MLIR_ERR_BAD_ARG, "rms_norm: shapes do not agree");
    return;
  }
  if (X.rows == 0 || X.cols == 0) return;
  Stager st;
  const void *dx, *dw;
  void *dy;
  if (st.in(X.p, X.span(esz), &dx) || st.in(W.p, (size_t)W.n * esz, &dw) ||
      st.out(Y.p, Y.span(esz), &dy, Y.ld != Y.cols))
    return;
  const float eps = (float)ctx().opt.rms_eps;
  int rc = f16 ? launch_rmsnorm_f16((const __half *)dx, (const __half *)dw, (__half *)dy, X.rows, X.cols, X.ld,
                                    Y.ld, eps)
               : launch_rmsnorm_f32((const float *)dx, (const float *)dw, (float *)dy, X.rows, X.cols, X.ld,
                                    Y.ld, eps);
  if (rc) return;
  st.finish();
}

void rms_norm_fwd_kernel_float16(int64_t rx, B200MemRef2D *x, int64_t ry, B200MemRef2D *y, int64_t rw,
                                 B200MemRef1D *w, B200_GRID_ARGS) {
  ENTER_KERNEL();
  rmsnorm_impl(true, rx, x, ry, y, rw, w);
}
void rms_norm_fwd_kernel_float32(int64_t rx, B200MemRef2D *x, int64_t ry, B200MemRef2D *y, int64_t rw,
                                 B200MemRef1D *w, B200_GRID_ARGS) {
  ENTER_KERNEL();
  rmsnorm_impl(false, rx, x, ry, y, rw, w);
}

// op: 0 silu f16, 1 silu f32, 2 swiglu f16, 3 add f16
static void ew_impl(int op, int64_t r0, B200MemRef1D *a, int64_t r1, B200MemRef1D *b, int64_t r2,
                    B200MemRef1D *o) {
  if (ensure_ready()) return;
  const size_t esz = op == 1 ? 4 : 2;
  View1 A, B{nullptr, 0}, O;
  if (view1("input 0", r0, a, esz, &A) || view1("output", r2, o, esz, &O)) return;
  if (op >= 2 && view1("input 1", r1, b, esz, &B)) return;
  if (A.n != O.n || (op >= 2 && B.n != A.n)) {
    set_error(B200MLIR_ERR_BAD_ARG, "elementwise: lengths differ");
    return;
  }
  if (A.n == 0) return;
  Stager st;
  const void *da, *db = nullptr;
  void *dout;
  if (st.in(A.p, (size_t)A.n * esz, &da) || (op >= 2 && st.in(B.p, (size_t)B.n * esz, &db)) ||
      st.out(O.p, (size_t)O.n * esz, &dout))
    return;
  int rc = 0;
  switch (op) {
    case 0: rc = launch_silu_f16((const __half *)da, (__half *)dout, A.n); break;
    case 1: rc = launch_silu_f32((const float *)da, (float *)dout, A.n); break;
    case 2: rc = launch_swiglu_f16((const __half *)da, (const __half *)db, (__half *)dout, A.n); break;
    default: rc = launch_add_f16((const __half *)da, (const __half *)db, (__half *)dout, A.n); break;
  }
  if (rc) return;
  st.finish();
}

void silu_kernel_float16(int64_t rx, B200MemRef1D *x, int64_t ry, B200MemRef1D *y, B200_GRID_ARGS) {
  ENTER_KERNEL();
  ew_impl(0, rx, x, 0, nullptr, ry, y);
}
void silu_kernel_float32(int64_t rx, B200MemRef1D *x, int64_t ry, B200MemRef1D *y, B200_GRID_ARGS) {
  ENTER_KERNEL();
  ew_impl(1, rx, x, 0, nullptr, ry, y);
}
void swiglu_kernel_float16(int64_t rg, B200MemRef1D *g, int64_t ru, B200MemRef1D *u, int64_t ro,
                           B200MemRef1D *o, B200_GRID_ARGS) {
  ENTER_KERNEL();
  ew_impl(2, rg, g, ru, u, ro, o);
}
void add_kernel_float16(int64_t rx, B200MemRef1D *x, int64_t ry, B200MemRef1D *y, int64_t ro,
                        B200MemRef1D *o, B200_GRID_ARGS) {
  ENTER_KERNEL();
  ew_impl(3, rx, x, ry, y, ro, o);
}

// ---- attention block ---------------------------------------------------------------------------
struct View4 {
  void *p;
  int64_t z, h, n, d, sz, sh, sn;
  size_t span(size_t esz) const { return (size_t)((z - 1) * sz + (h - 1) * sh + (n - 1) * sn + d) * esz; }
};
static int view4(const char *what, int64_t rank, const B200MemRef4D *m, size_t esz, View4 *v) {
  if (rank != 4 || !m)
    return set_error(B200MLIR_ERR_BAD_ARG, "%s: expected a rank-4 memref descriptor (got rank %lld)", what, (long long)rank);
  for (int i = 0; i < 4; ++i)
    if (m->sizes[i] < 1 || m->strides[i] < 0)
      return set_error(B200MLIR_ERR_BAD_ARG, "%s: extent %d is %lld", what, i, (long long)m->sizes[i]);
  if (m->strides[3] != 1) return set_error(B200MLIR_ERR_BAD_ARG, "%s: innermost stride must be 1", what);
  if (!m->aligned) return set_error(B200MLIR_ERR_BAD_ARG, "%s: null data pointer", what);
  v->p = (char *)m->aligned + m->offset * (int64_t)esz;
  v->z = m->sizes[0], v->h = m->sizes[1], v->n = m->sizes[2], v->d = m->sizes[3];
  v->sn = v->n > 1 ? m->strides[2] : v->d;
  v->sh = v->h > 1 ? m->strides[1] : v->n * v->sn;
  v->sz = v->z > 1 ? m->strides[0] : std::max(v->h * v->sh, v->n * v->sn);
  return 0;
}
static void attention_impl(bool f32, int64_t rq, B200MemRef4D *q, int64_t rk, B200MemRef4D *k, int64_t rv,
                           B200MemRef4D *v, int64_t ro, B200MemRef4D *out, float sm_scale) {
  if (ensure_ready()) return;
  const size_t esz = f32 ? 4 : 2;
  View4 Q, K, V, O;
  if (view4("Q", rq, q, esz, &Q) || view4("K", rk, k, esz, &K) || view4("V", rv, v, esz, &V) ||
      view4("Out", ro, out, esz, &O))
    return;
  for (const View4 *t : {&K, &V, &O})
    if (t->z != Q.z || t->h != Q.h || t->n != Q.n || t->d != Q.d) {
      set_error(B200MLIR_ERR_BAD_ARG, "attention: Q, K, V and Out must have one shape [Z, H, N_CTX, D_HEAD]");
      return;
    }
  for (const View4 *t : {&K, &V})
    if (t->sz != Q.sz || t->sh != Q.sh || t->sn != Q.sn) {
      // the reference kernel takes one stride set for all of its tensors (test_flash_attention.py:31-34)
      set_error(B200MLIR_ERR_BAD_ARG, "attention: Q, K and V must share their strides");
      return;
    }
  Stager st;
  const void *dq, *dk, *dv;
  void *dout;
  if (st.in(Q.p, Q.span(esz), &dq) || st.in(K.p, K.span(esz), &dk) || st.in(V.p, V.span(esz), &dv) ||
      st.out(O.p, O.span(esz), &dout, O.span(esz) != (size_t)(O.z * O.h * O.n * O.d) * esz))
    return;
  if (launch_attention(dq, dk, dv, dout, f32, Q.z, Q.h, Q.n, Q.d, Q.sz, Q.sh, Q.sn, O.sz, O.sh, O.sn, (double)sm_scale,
                       ctx().opt.attention_stage == 3))
    return;
  st.finish();
}

void online_softmax(int64_t rx, B200MemRef2D *x, int64_t ry, B200MemRef2D *y, B200_GRID_ARGS) {
  ENTER_KERNEL();
  softmax_impl(false, rx, x, ry, y);
}
void attention_fwd_kernel_float16(int64_t rq, B200MemRef4D *q, int64_t rk, B200MemRef4D *k, int64_t rv,
                                  B200MemRef4D *v, int64_t ro, B200MemRef4D *out, float sm_scale, B200_GRID_ARGS) {
  ENTER_KERNEL();
  attention_impl(false, rq, q, rk, k, rv, v, ro, out, sm_scale);
}
void attention_fwd_kernel_float32(int64_t rq, B200MemRef4D *q, int64_t rk, B200MemRef4D *k, int64_t rv,
                                  B200MemRef4D *v, int64_t ro, B200MemRef4D *out, float sm_scale, B200_GRID_ARGS) {
  ENTER_KERNEL();
  attention_impl(true, rq, q, rk, k, rv, v, ro, out, sm_scale);
}

int b200mlir_w8a16_register_weight(const void *wq, const void *scales, int64_t k, int64_t n, int l2_persist) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!wq || !scales || k <= 0 || n <= 0)
    return set_error(B200MLIR_ERR_BAD_ARG, "w8a16 register: null pointer or empty shape");
  std::lock_guard<std::mutex> lk(g_w_mu);
  return register_weight_locked(wq, scales, k, n, l2_persist, nullptr);
}

int b200mlir_w8a16_unregister_weight(const void *wq) {
  clear_error();
  std::lock_guard<std::mutex> lk(g_w_mu);
  auto it = g_weights.find(wq);
  if (it == g_weights.end()) return set_error(B200MLIR_ERR_BAD_ARG, "w8a16 unregister: unknown weight");
  cudaStreamSynchronize(ctx().stream);
  if (it->second.l2_persist) l2_window_clear(it->second.image);
  cudaFree(it->second.image);
  cudaFree(it->second.w16);
  cudaFree(it->second.scales_dev);
  g_weights.erase(it);
  return 0;
}

void w8a16_matmul(int64_t ra, B200MemRef2D *a, int64_t rw, B200MemRef2D *wq, int64_t rs, B200MemRef1D *s,
                  int64_t rc, B200MemRef2D *c, B200_GRID_ARGS) {
  ENTER_KERNEL();
  if (ensure_ready()) return;
  View2 A, W, C;
  View1 S;
  if (view2("A", ra, a, 2, &A) || view2("Wq", rw, wq, 1, &W) || view1("scales", rs, s, 2, &S) ||
      view2("C", rc, c, 2, &C))
    return;
  if (A.cols != W.rows || C.rows != A.rows || C.cols != W.cols || S.n != W.cols) {
    set_error(B200MLIR_ERR_BAD_ARG, "w8a16_matmul: shapes do not agree");
    return;
  }
  if (W.ld != W.cols) {
    set_error(B200MLIR_ERR_BAD_ARG, "w8a16_matmul: the weight must be dense row-major");
    return;
  }
  if (C.rows == 0 || C.cols == 0) return;
  const bool resident = ctx().opt.enable_weight_resident != 0;
  W8A16Weight local, *w = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_w_mu);
    if (resident) {
      if (register_weight_locked(W.p, S.p, W.rows, W.cols, 0, &w)) return;
      if (A.rows > (int64_t)ctx().opt.w8a16_expand_rows && !w->w16 &&
          w8a16_expand_f16(w->image, (const __half *)w->scales_dev, w->k, w->n, &w->w16))
        return;
      local = *w;
    }
  }
  Stager st;
  void *tmp_w = nullptr;
  if (!resident) {
    // residency off: the image is rebuilt for this call and dropped afterwards
    const void *dw, *ds;
    if (st.in(W.p, (size_t)W.rows * W.cols, &dw) || st.in(S.p, (size_t)S.n * 2, &ds)) return;
    local.k = W.rows; local.n = W.cols; local.scales_dev = const_cast<void *>(ds);
    if (w8a16_build_tmem_image((const int8_t *)dw, W.rows, W.cols, &local.image, &local.image_bytes)) return;
    tmp_w = local.image;
  }
  const void *da;
  void *dc;
  int rcode = st.in(A.p, A.span(2), &da);
  if (!rcode) rcode = st.out(C.p, C.span(2), &dc, C.ld != C.cols);
  if (!rcode) rcode = launch_w8a16((const __half *)da, local, (__half *)dc, A.rows, A.ld, C.ld);
  if (!rcode) rcode = st.finish();
  if (tmp_w) {
    cudaStreamSynchronize(ctx().stream);
    cudaFree(tmp_w);
  }
}

// Phase stamps of the most recent MLP block on this thread (option mlpPhaseTiming): events after
// the block's start, RMSNorm, gate/up GEMM, down GEMM and, in the tensor-parallel entry, the collective.
struct PhaseStamps {
  cudaEvent_t ev[5] = {};
  int n = 0;
  void mark(int i) {
    if (ctx().opt.mlp_phase_timing == 0) return;
    if (!ev[i] && cudaEventCreate(&ev[i]) != cudaSuccess) return;
    cudaEventRecord(ev[i], ctx().stream);
    if (i + 1 > n) n = i + 1;
    if (i == 0) n = 1;
  }
};
static thread_local PhaseStamps t_phases;

// rmsnorm -> gate/up GEMM with SwiGLU read-out -> down GEMM.  The down GEMM either writes
// `out` (with the residual when asked) or, given push targets, stores its fp16 partial rows
// into the receive slots of the ranks that own them.
// `down_chunks` > 1 cuts the DOWN projection (only) into that many token chunks and calls
// `after_chunk(first row, rows, device address of the chunk's output rows)` after each one's
// launch: the tensor-parallel entry starts the chunk's collective there.  RMSNorm and the gate/up
// GEMM always cover all tokens (cut into chunks they would fill the SM pairs worse; the down
// projection's 256 x 256 tiles divide evenly over token halves).
typedef std::function<int(int64_t, int64_t, void *)> ChunkHook;
static void mlp_block_impl(int64_t rx, B200MemRef2D *x, int64_t rg, B200MemRef1D *gain, int64_t rwg,
                           B200MemRef2D *wg, int64_t rwu, B200MemRef2D *wu, int64_t rwd, B200MemRef2D *wd,
                           int64_t ro, B200MemRef2D *out, float eps, int add_residual, const PushTargets *push,
                           int down_chunks = 1, const ChunkHook *after_chunk = nullptr, int res_mod = 1,
                           int res_rem = 0) {
  if (ensure_ready()) return;
  View2 X, WG, WU, WD, O{nullptr, 0, 0, 0};
  View1 G;
  if (view2("x", rx, x, 2, &X) || view1("gain", rg, gain, 2, &G) || view2("Wg", rwg, wg, 2, &WG) ||
      view2("Wu", rwu, wu, 2, &WU) || view2("Wd", rwd, wd, 2, &WD) || (!push && view2("out", ro, out, 2, &O)))
    return;
  const int64_t T = X.rows, D = X.cols, F = WG.cols;
  if (G.n != D || WG.rows != D || WU.rows != D || WU.cols != F || WD.rows != F || WD.cols != D ||
      (!push && (O.rows != T || O.cols != D)) || WU.ld != WG.ld) {
    set_error(B200MLIR_ERR_BAD_ARG, "mlp_block: shapes do not agree");
    return;
  }
  if (T == 0 || D == 0) return;
  Stager st;
  const void *dx, *dg, *dwg, *dwu, *dwd;
  void *dout = nullptr;
  if (st.in(X.p, X.span(2), &dx) || st.in(G.p, (size_t)D * 2, &dg) || st.in(WG.p, WG.span(2), &dwg) ||
      st.in(WU.p, WU.span(2), &dwu) || st.in(WD.p, WD.span(2), &dwd) ||
      (!push && st.out(O.p, O.span(2), &dout, O.ld != O.cols)))
    return;
  void *h = nullptr, *act = nullptr;
  if (workspace((size_t)T * D * 2, &h) || workspace2((size_t)T * F * 2, &act)) return;
  t_phases.mark(0);
  // 1. h = rmsnorm(x) * gain
  if (launch_rmsnorm_f16((const __half *)dx, (const __half *)dg, (__half *)h, T, D, X.ld, D, eps)) return;
  // 2. act = silu(h·Wg) * (h·Wu), fused in the GEMM epilogue
  GemmArgs g1;
  g1.a = h; g1.b = dwg; g1.b2 = dwu; g1.c = act;
  g1.m = T; g1.n = F; g1.k = D; g1.lda = D; g1.ldb = WG.ld; g1.ldc = F;
  g1.epilogue = EPI_SWIGLU;
  t_phases.mark(1);
  if (gemm_dispatch(g1)) return;
  t_phases.mark(2);
  // 3. out = act·Wd (+ x through the f32 residual read-out), or the partial rows pushed to their owners
  GemmArgs g2;
  g2.a = act; g2.b = dwd; g2.c = dout;
  g2.m = T; g2.n = D; g2.k = F; g2.lda = F; g2.ldb = WD.ld; g2.ldc = push ? D : O.ld;
  if (push) {
    g2.epilogue = EPI_PUSH16;
    g2.push = push;
  } else if (add_residual) {
    g2.epilogue = EPI_F16_RES16;
    g2.res = dx;
    g2.ldres = X.ld;
    g2.res_mod = res_mod;  // tensor-parallel callers: the ranks take turns, by 256-row block, in adding x
    g2.res_rem = res_rem;
  }
  if (push || down_chunks <= 1) {
    if (gemm_dispatch(g2)) return;
    t_phases.mark(3);
    if (after_chunk && (*after_chunk)(0, T, dout)) return;
  } else {
    // token chunks on multiples of 256 rows (whole tiles of the pair kernel)
    int64_t step = ((T + down_chunks - 1) / down_chunks + 255) / 256 * 256;
    for (int64_t r0 = 0; r0 < T; r0 += step) {
      const int64_t rows = std::min(step, T - r0);
      GemmArgs gc = g2;
      gc.a = (const __half *)act + r0 * F;
      gc.c = (__half *)dout + r0 * g2.ldc;
      if (gc.res) gc.res = (const __half *)dx + r0 * X.ld;
      gc.m = rows;
      if (gemm_dispatch(gc)) return;
      if (after_chunk && (*after_chunk)(r0, rows, gc.c)) return;
    }
    t_phases.mark(3);
  }
  st.finish();
}

void mlp_block_float16(int64_t rx, B200MemRef2D *x, int64_t rg, B200MemRef1D *gain, int64_t rwg,
                       B200MemRef2D *wg, int64_t rwu, B200MemRef2D *wu, int64_t rwd, B200MemRef2D *wd,
                       int64_t ro, B200MemRef2D *out, float eps, int add_residual, B200_GRID_ARGS) {
  ENTER_KERNEL();
  const int mod = (int)ctx().opt.mlp_residual_mod, rem = (int)ctx().opt.mlp_residual_rem;
  mlp_block_impl(rx, x, rg, gain, rwg, wg, rwu, wu, rwd, wd, ro, out, eps, add_residual, nullptr, 1, nullptr,
                 mod > 1 ? mod : 1, mod > 1 ? rem : 0);
}

// The tensor-parallel block with the sum over ranks inside the call: every rank computes the
// partial output of its shard of the hidden dimension (each carries the residual of its share of the 256-row blocks, so the sum is
// the finished block) and the partials are added with ncclAllReduce.  `chunks` > 1 cuts the down
// projection into that many token chunks; the all-reduce of a chunk runs on a second stream while
// the next chunk's GEMM is computed.  Device tensors only (the collective works on `out` in place).
void mlp_block_tp_float16(int64_t rx, B200MemRef2D *x, int64_t rg, B200MemRef1D *gain, int64_t rwg,
                          B200MemRef2D *wg, int64_t rwu, B200MemRef2D *wu, int64_t rwd, B200MemRef2D *wd,
                          int64_t ro, B200MemRef2D *out, float eps, int chunks, B200_GRID_ARGS) {
  ENTER_KERNEL();
  if (ensure_ready()) return;
  const int world = tp_world();
  if (world == 1) {
    mlp_block_impl(rx, x, rg, gain, rwg, wg, rwu, wu, rwd, wd, ro, out, eps, 1, nullptr);
    return;
  }
  View2 X, O;
  if (view2("x", rx, x, 2, &X) || view2("out", ro, out, 2, &O)) return;
  if (X.rows != O.rows || X.cols != O.cols || O.ld != O.cols) {
    set_error(B200MLIR_ERR_BAD_ARG, "mlp_block_tp: out must be a dense [T, D] tensor of x's shape");
    return;
  }
  if (!is_device_ptr(X.p) || !is_device_ptr(O.p)) {
    set_error(B200MLIR_ERR_BAD_ARG, "mlp_block_tp: x and out must be device tensors (the all-reduce works on out in place)");
    return;
  }
  const int64_t D = X.cols;
  if (X.rows == 0 || D == 0) return;
  if (chunks < 1) chunks = 1;
  if (chunks > 16) chunks = 16;
  cudaStream_t s = ctx().stream, sc = nullptr;
  if (chunks > 1 && tp_comm_stream(&sc)) return;
  cudaEvent_t ev[16] = {}, done[16] = {};
  int used = 0;
  ChunkHook hook = [&](int64_t, int64_t rows, void *dst) -> int {
    if (chunks == 1) {
      int rc = tp_all_reduce_f16(dst, (size_t)rows * D, s);
      t_phases.mark(4);
      return rc;
    }
    // fork: this chunk's collective on the side stream, after the chunk's GEMM
    if (used >= 16) return set_error(B200MLIR_ERR_BAD_ARG, "mlp_block_tp: too many chunks");
    if (cudaEventCreateWithFlags(&ev[used], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&done[used], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventRecord(ev[used], s) != cudaSuccess || cudaStreamWaitEvent(sc, ev[used], 0) != cudaSuccess) {
      ++used;
      return set_error(B200MLIR_ERR_CUDA, "mlp_block_tp: event plumbing failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    int rc = tp_all_reduce_f16(dst, (size_t)rows * D, sc);
    if (rc == 0) cudaEventRecord(done[used], sc);
    ++used;
    return rc;
  };
  // every rank's partial carries the residual of ITS 256-row blocks (block b: rank b % world), so
  // the sum holds x once and no rank's read-out pays for all of it
  mlp_block_impl(rx, x, rg, gain, rwg, wg, rwu, wu, rwd, wd, ro, out, eps, 1, nullptr, chunks, &hook, world, tp_rank());
  for (int i = 0; i < used; ++i) {  // join: the caller's stream continues after every chunk's collective
    if (done[i]) cudaStreamWaitEvent(s, done[i], 0);
    if (ev[i]) cudaEventDestroy(ev[i]);
    if (done[i]) cudaEventDestroy(done[i]);
  }
}

// The tensor-parallel block with the sum over ranks done by this library's own kernel through
// the NVSwitch's multicast addresses, overlapped with the math: `out` is this rank's [T, D] view
// at the start of a symmetric buffer whose multicast address is `mc_buf` and which holds 16 flag
// words at element `flags_elem_offset` (see b200mlir_tp_allreduce_multimem_sync_float16).  The
// down projection is cut into `chunks` token chunks; as soon as a chunk's GEMM has been issued its
// all-reduce is launched on a second stream, where it runs beside the next chunk's GEMM: the
// kernel uses no shared memory and few registers, so its CTAs fit on the SMs the persistent GEMM
// occupies.  Both rendezvous of the ranks are inside that launch (bounded waits).  With one chunk
// the rendezvous are the library's one-warp barrier launches around the plain all-reduce.
void mlp_block_tp_multicast_float16(int64_t rx, B200MemRef2D *x, int64_t rg, B200MemRef1D *gain, int64_t rwg,
                                    B200MemRef2D *wg, int64_t rwu, B200MemRef2D *wu, int64_t rwd, B200MemRef2D *wd,
                                    int64_t ro, B200MemRef2D *out, void *mc_buf, void *const *peer_bufs,
                                    int64_t flags_elem_offset, void *state, int rank, int world, float eps, int chunks,
                                    B200_GRID_ARGS) {
  ENTER_KERNEL();
  if (ensure_ready()) return;
  View2 X, O;
  if (view2("x", rx, x, 2, &X) || view2("out", ro, out, 2, &O)) return;
  const int64_t T = X.rows, D = X.cols;
  if (O.rows != T || O.cols != D || O.ld != D || !is_device_ptr(X.p) || !is_device_ptr(O.p) || !mc_buf || !state ||
      !peer_bufs || world < 2 || world > kMaxPushRanks || rank < 0 || rank >= world || flags_elem_offset < T * D ||
      peer_bufs[rank] != O.p) {
    set_error(B200MLIR_ERR_BAD_ARG,
              "mlp_block_tp_multicast: dense device [T, D] out at the start of the symmetric buffer, its multicast "
              "address, flag words behind the data, 2 <= world <= %d", kMaxPushRanks);
    return;
  }
  if (T == 0 || D == 0) return;
  if (chunks < 1) chunks = 1;
  if (chunks > 16) chunks = 16;
  // every chunk a multiple of 256 rows (whole tiles) whose rows divide over the ranks
  int64_t step = ((T + chunks - 1) / chunks + 255) / 256 * 256;
  if (chunks > 1 && (T % step != 0 || step % world != 0)) {
    chunks = 1;
    step = T;
  }
  if (T % world != 0 || (D % 8) != 0) {
    set_error(B200MLIR_ERR_BAD_ARG, "mlp_block_tp_multicast: tokens divisible by the world size, width a multiple of 8");
    return;
  }
  cudaStream_t s = ctx().stream, sc = nullptr;
  if (chunks > 1 && tp_comm_stream(&sc)) return;
  cudaEvent_t ev[16] = {}, done = nullptr;
  int used = 0;
  ChunkHook hook = [&](int64_t r0, int64_t rows, void *) -> int {
    const int64_t mine = rows / world;  // this rank sums rows [r0 + rank * mine, + mine) of the chunk
    const int64_t off = (r0 + (int64_t)rank * mine) * D, cnt = mine * D;
    if (chunks == 1) {
      // one chunk: the library's barrier launches around the plain all-reduce (measured faster than
      // both rendezvous inside the launch: a system-scope fence per CTA costs more than a launch)
      int rc = launch_rank_barrier(peer_bufs, flags_elem_offset, 0, rank, world, state);
      if (rc == 0) rc = launch_allreduce_multimem(mc_buf, mc_buf, off, cnt);
      if (rc == 0) rc = launch_rank_barrier(peer_bufs, flags_elem_offset, 1, rank, world, state);
      t_phases.mark(4);
      return rc;
    }
    if (cudaEventCreateWithFlags(&ev[used], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventRecord(ev[used], s) != cudaSuccess || cudaStreamWaitEvent(sc, ev[used], 0) != cudaSuccess) {
      ++used;
      return set_error(B200MLIR_ERR_CUDA, "mlp_block_tp_multicast: event plumbing failed: %s",
                       cudaGetErrorString(cudaGetLastError()));
    }
    ++used;
    return launch_allreduce_multimem_sync(mc_buf, peer_bufs, off, cnt, flags_elem_offset, rank, world, state, sc);
  };
  mlp_block_impl(rx, x, rg, gain, rwg, wg, rwu, wu, rwd, wd, ro, out, eps, 1, nullptr, chunks, &hook, world, rank);
  if (chunks > 1) {  // join: the caller's stream continues after the last chunk's all-reduce
    if (cudaEventCreateWithFlags(&done, cudaEventDisableTiming) == cudaSuccess && cudaEventRecord(done, sc) == cudaSuccess)
      cudaStreamWaitEvent(s, done, 0);
    if (done) cudaEventDestroy(done);
  }
  for (int i = 0; i < used; ++i)
    if (ev[i]) cudaEventDestroy(ev[i]);
}

static int fill_push(PushTargets *pt, void *const *peer_recv, int world, int rank, int64_t rows) {
  if (!peer_recv || world < 1 || world > kMaxPushRanks || rank < 0 || rank >= world || rows < 1 || rows % world)
    return set_error(B200MLIR_ERR_BAD_ARG, "tensor-parallel push: world 1..%d, rank inside it, rows divisible by world",
                     kMaxPushRanks);
  for (int i = 0; i < world; ++i) {
    if (!peer_recv[i]) return set_error(B200MLIR_ERR_BAD_ARG, "tensor-parallel push: receive pointer %d is null", i);
    pt->recv[i] = peer_recv[i];
  }
  pt->world = world;
  pt->rank = rank;
  pt->rows_per_rank = rows / world;
  return 0;
}

void mlp_block_push_float16(int64_t rx, B200MemRef2D *x, int64_t rg, B200MemRef1D *gain, int64_t rwg,
                            B200MemRef2D *wg, int64_t rwu, B200MemRef2D *wu, int64_t rwd, B200MemRef2D *wd,
                            void *const *peer_recv, int world, int rank, float eps, B200_GRID_ARGS) {
  ENTER_KERNEL();
  PushTargets pt;
  if (!x || fill_push(&pt, peer_recv, world, rank, x->sizes[0])) return;
  mlp_block_impl(rx, x, rg, gain, rwg, wg, rwu, wu, rwd, wd, 0, nullptr, eps, 0, &pt);
}

int b200mlir_tp_reduce_rows_float16(const void *recv, const void *residual, int64_t ldres, void *const *peer_out,
                                    int world, int rank, int64_t rows_per_rank, int64_t cols) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!recv || !peer_out || !is_device_ptr(recv))
    return set_error(B200MLIR_ERR_BAD_ARG, "tp_reduce_rows: device buffers required");
  return launch_reduce_rows_push((const __half *)recv, (const __half *)residual, ldres, peer_out, world, rank,
                                 rows_per_rank, cols);
}

int b200mlir_tp_allreduce_multimem_float16(const void *mc_in, void *mc_out, int64_t elem_offset, int64_t count) {
  clear_error();
  return launch_allreduce_multimem(mc_in, mc_out, elem_offset, count);
}

int b200mlir_tp_allreduce_multimem_sync_float16(void *mc_buf, void *const *peer_bufs, int64_t elem_offset, int64_t count,
                                                int64_t flags_elem_offset, int rank, int world, void *state,
                                                int exit_rendezvous) {
  clear_error();
  return launch_allreduce_multimem_sync(mc_buf, peer_bufs, elem_offset, count, flags_elem_offset, rank, world, state,
                                        nullptr, exit_rendezvous ? 1 : 0);
}

int b200mlir_tp_barrier(void *const *peer_bufs, int64_t flags_elem_offset, int slot, int rank, int world, void *state) {
  clear_error();
  return launch_rank_barrier(peer_bufs, flags_elem_offset, slot, rank, world, state);
}

int b200mlir_host_gemm_plan(int64_t m, int64_t n, int64_t k, int64_t *panels4) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  const HostGemmPlan h = host_gemm_plan(m, n, k);
  if (h.pipelined && panels4) {
    panels4[0] = h.pm;
    panels4[1] = h.pn;
    panels4[2] = h.PM;
    panels4[3] = h.PN;
  }
  return h.pipelined ? 1 : 0;
}

int b200mlir_mlp_phase_times(double *us, int cap) {
  clear_error();
  if (!us || cap < 1) {
    set_error(B200MLIR_ERR_BAD_ARG, "mlp_phase_times: null buffer");
    return -1;
  }
  PhaseStamps &ph = t_phases;
  if (ph.n < 2) return 0;
  int out = 0;
  cudaError_t e = cudaEventSynchronize(ph.ev[ph.n - 1]);
  for (int i = 1; e == cudaSuccess && i < ph.n && out < cap; ++i, ++out) {
    float ms = 0;
    e = cudaEventElapsedTime(&ms, ph.ev[i - 1], ph.ev[i]);
    us[out] = (double)ms * 1000.0;
  }
  if (e != cudaSuccess) {
    set_error(B200MLIR_ERR_CUDA, "mlp_phase_times: %s", cudaGetErrorString(e));
    return -1;
  }
  return out;
}

int b200mlir_pack_weight_f16(const void *src, void *dst, int64_t k, int64_t n, int64_t ld) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!src || !dst || k <= 0 || n <= 0 || ld < n) return set_error(B200MLIR_ERR_BAD_ARG, "pack_weight: bad argument");
  Stager st;
  const void *ds;
  void *dd;
  const size_t out_bytes = (size_t)((k + 31) / 32) * ((n + 31) / 32) * 2048;
  B200_TRY(st.in(src, ((size_t)(k - 1) * ld + n) * 2, &ds));
  B200_TRY(st.out(dst, out_bytes, &dd));
  B200_TRY(launch_pack_weight_f16((const uint16_t *)ds, (uint16_t *)dd, k, n, ld));
  return st.finish();
}

int b200mlir_pack_act_f16(const void *src, void *dst, int64_t rows, int64_t cols, int64_t ld) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!src || !dst || rows <= 0 || cols <= 0 || ld < cols) return set_error(B200MLIR_ERR_BAD_ARG, "pack_act: bad argument");
  Stager st;
  const void *ds;
  void *dd;
  const size_t out_bytes = (size_t)((rows + 31) / 32) * ((cols + 31) / 32) * 2048;
  B200_TRY(st.in(src, ((size_t)(rows - 1) * ld + cols) * 2, &ds));
  B200_TRY(st.out(dst, out_bytes, &dd));
  B200_TRY(launch_pack_act_f16((const uint16_t *)ds, (uint16_t *)dd, rows, cols, ld));
  return st.finish();
}

int b200mlir_unpack_acc_f16(const void *tiles, void *dst, int64_t rows, int64_t cols, int64_t ld) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!tiles || !dst || rows <= 0 || cols <= 0 || ld < cols) return set_error(B200MLIR_ERR_BAD_ARG, "unpack_acc: bad argument");
  Stager st;
  const void *ds;
  void *dd;
  const size_t in_bytes = (size_t)((rows + 31) / 32) * ((cols + 31) / 32) * 2048;
  B200_TRY(st.in(tiles, in_bytes, &ds));
  B200_TRY(st.out(dst, ((size_t)(rows - 1) * ld + cols) * 2, &dd, ld != cols));
  B200_TRY(launch_unpack_acc_f16((const uint16_t *)ds, (uint16_t *)dd, rows, cols, ld));
  return st.finish();
}

}  // extern "C"
