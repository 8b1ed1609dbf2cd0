// Context, error recording, options and the hexagon_runtime_* seam
// (qcom_hexagon_backend/bin/runtime/include/HexagonCAPI.h:26-68,
//  bin/runtime/include/RuntimeDMA.h:39-51) answered on a CUDA device.
#include <cstdarg>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.h"

namespace b200 {

static thread_local int t_err_code = 0;
static thread_local char t_err_msg[512] = {0};
std::atomic<int64_t> g_launches{0};

int set_error(int code, const char *fmt, ...) {
  t_err_code = code;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err_msg, sizeof(t_err_msg), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() {
  t_err_code = 0;
  t_err_msg[0] = 0;
}

Context &ctx() {
  static Context c;
  return c;
}

static std::mutex g_mu;

// ---- the calling thread's stream, and the L2 persistence window it carries ------------------
static thread_local cudaStream_t t_stream = nullptr;
static thread_local uint64_t t_window_gen = 0;       // generation of the window last applied by this thread ...
static thread_local cudaStream_t t_window_stream = nullptr;  // ... and the stream it was applied to
StreamSlot::operator cudaStream_t() const { return t_stream; }
StreamSlot &StreamSlot::operator=(cudaStream_t s) {
  t_stream = s;
  return *this;
}

// An access-policy window is an attribute of ONE stream, and the set-aside L2 size is a device
// limit: the library keeps one window (the most recently registered persisting weight), raises
// the limit and never lowers it, and re-applies the window whenever a thread's stream is not the
// one that carries the current generation.
struct L2Window {
  const void *base = nullptr;
  size_t bytes = 0;
  size_t limit = 0;     // cudaLimitPersistingL2CacheSize as set by this library
  uint64_t gen = 0;     // bumped by every change
};
static L2Window g_window;

void l2_window_apply() {
  const void *base;
  size_t bytes;
  uint64_t gen;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    base = g_window.base;
    bytes = g_window.bytes;
    gen = g_window.gen;
  }
  if (gen == 0 || (t_window_gen == gen && t_window_stream == t_stream)) return;
  cudaStreamAttrValue attr = {};
  attr.accessPolicyWindow.base_ptr = const_cast<void *>(base);
  attr.accessPolicyWindow.num_bytes = base ? bytes : 0;  // zero bytes switches the window off
  attr.accessPolicyWindow.hitRatio = 1.0f;
  attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
  attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
  if (cudaStreamSetAttribute(t_stream, cudaStreamAttributeAccessPolicyWindow, &attr) != cudaSuccess)
    cudaGetLastError();  // a hint; not having it is not an error
  t_window_gen = gen;
  t_window_stream = t_stream;
}

int l2_window_set(const void *base, size_t bytes) {
  Context &c = ctx();
  if (c.persisting_l2_max == 0) return 0;
  size_t want = bytes < c.persisting_l2_max ? bytes : c.persisting_l2_max;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (want > g_window.limit) {
      if (cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, want) != cudaSuccess) {
        cudaGetLastError();
        return 0;
      }
      g_window.limit = want;
    }
    g_window.base = base;
    g_window.bytes = want;
    ++g_window.gen;
  }
  l2_window_apply();
  return 0;
}

void l2_window_clear(const void *base) {
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_window.base != base) return;
    g_window.base = nullptr;
    g_window.bytes = 0;
    ++g_window.gen;
  }
  l2_window_apply();
}

static int init_locked(int device) {
  Context &c = ctx();
  if (c.ready && c.device == device) return 0;
  // The status word, the workspaces, the copy streams, registered weights and the kernels'
  // cached attributes all belong to the first device: one device per process.
  if (c.ready)
    return set_error(B200MLIR_ERR_BAD_ARG, "already initialised on device %d; one device per process (asked for %d)",
                     c.device, device);
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return set_error(B200MLIR_ERR_NO_DEVICE, "no CUDA device: %s",
                     e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  if (device < 0 || device >= count)
    return set_error(B200MLIR_ERR_BAD_ARG, "device %d out of range (have %d)", device, count);
  B200_CUDA(cudaSetDevice(device));
  cudaDeviceProp p;
  B200_CUDA(cudaGetDeviceProperties(&p, device));
  if (p.major != 10)
    return set_error(B200MLIR_ERR_NO_DEVICE,
                     "device %d is sm_%d%d; this library is built for sm_100a only", device,
                     p.major, p.minor);
  c.device = device;
  c.sm_count = p.multiProcessorCount;
  c.cc_major = p.major;
  c.cc_minor = p.minor;
  c.l2_bytes = (size_t)p.l2CacheSize;
  c.persisting_l2_max = (size_t)p.persistingL2CacheMaxSize;
  c.gpu_name = p.name;
  if (!c.d_status) {
    B200_CUDA(cudaMalloc(&c.d_status, 256));
    B200_CUDA(cudaMemset(c.d_status, 0, 256));
  }
  c.ready = true;
  return 0;
}

int ensure_ready() {
  Context &c = ctx();
  if (c.ready) {
    // A host thread that calls in for the first time has no current context yet, and the
    // driver-API calls made here (tensor-map encoding) need one: bind the device's primary context.
    static thread_local bool t_bound = false;
    int cur = -1;
    if (!t_bound || (cudaGetDevice(&cur) == cudaSuccess && cur != c.device)) {
      cudaSetDevice(c.device);
      cudaFree(nullptr);
      t_bound = true;
    }
    return 0;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  return init_locked(dev);
}

int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return set_error(B200MLIR_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  count_launch();
  return 0;
}

// Grow-only workspaces (two for kernels' intermediates, one for staged host tensors).  Growing frees and reallocates, so it must not
// happen inside a stream capture: callers warm up once outside any capture.
struct Arena {
  void *p = nullptr;
  size_t cap = 0;
};
static Arena g_ws[4];

static int ws_get(int which, size_t bytes, void **out) {
  Arena &a = g_ws[which];
  if (bytes > a.cap) {
    size_t want = ((bytes + (1u << 20) - 1) >> 20) << 20;
    if (a.p) {
      B200_CUDA(cudaStreamSynchronize(ctx().stream));
      B200_CUDA(cudaFree(a.p));
      a.p = nullptr;
      a.cap = 0;
    }
    B200_CUDA(cudaMalloc(&a.p, want));
    a.cap = want;
  }
  *out = a.p;
  return 0;
}
int workspace(size_t bytes, void **out) { return ws_get(0, bytes, out); }
int workspace2(size_t bytes, void **out) { return ws_get(1, bytes, out); }
int staging_workspace(size_t bytes, void **out) { return ws_get(2, bytes, out); }
int splitk_workspace(size_t bytes, void **out) {
  const bool fresh = bytes > g_ws[3].cap;
  B200_TRY(ws_get(3, bytes, out));
  // the tile counters at its start must read zero before the first launch that uses them
  // (every launch leaves them at zero again)
  if (fresh) B200_CUDA(cudaMemsetAsync(g_ws[3].p, 0, g_ws[3].cap, ctx().stream));
  return 0;
}

int copy_streams(cudaStream_t *in, cudaStream_t *out) {
  static cudaStream_t s_in = nullptr, s_out = nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!s_in) B200_CUDA(cudaStreamCreateWithFlags(&s_in, cudaStreamNonBlocking));
  if (!s_out) B200_CUDA(cudaStreamCreateWithFlags(&s_out, cudaStreamNonBlocking));
  *in = s_in;
  *out = s_out;
  return 0;
}

bool is_device_ptr(const void *p) {
  if (!p) return false;
  cudaPointerAttributes at;
  cudaError_t e = cudaPointerGetAttributes(&at, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

// ---- residency bookkeeping -----------------------------------------------------------
struct Resident {
  void *ptr = nullptr;
  uint32_t bytes = 0;
  uint32_t align = 0;
  bool freed = false;
};
struct ResidentState {
  bool entered = false;
  uint64_t lo = 0, hi = 0;
  std::map<std::pair<uint64_t, uint32_t>, Resident> workspaces;  // (key, instance)
  std::unordered_map<uint64_t, Resident> weights;                // source address
  std::unordered_map<void *, Resident *> by_ptr;
};
static ResidentState g_res;

static bool supported_alignment(uint32_t a) {
  return a != 0 && (a & (a - 1)) == 0 && a <= 2048;
}

static void *resident_alloc(uint32_t bytes, uint32_t align) {
  void *p = nullptr;
  // cudaMalloc returns >= 256-byte aligned memory; over-allocate for more.
  size_t extra = align > 256 ? align : 0;
  if (cudaMalloc(&p, (size_t)bytes + extra) != cudaSuccess) {
    set_error(B200MLIR_ERR_CUDA, "resident allocation of %u bytes failed: %s", bytes,
              cudaGetErrorString(cudaGetLastError()));
    return nullptr;
  }
  uintptr_t u = (uintptr_t)p;
  if (extra) u = (u + align - 1) & ~(uintptr_t)(align - 1);
  return (void *)u;
}

// ---- copy tokens ---------------------------------------------------------------------
struct CopyRing {
  static constexpr int kSlots = 128;  // the reference ring holds 128 descriptors
  cudaEvent_t ev[kSlots] = {};
  uint32_t token_of[kSlots] = {};
  bool used[kSlots] = {};
  uint32_t next = 0;
  cudaStream_t stream = nullptr;
};
static CopyRing g_ring;

}  // namespace b200

using namespace b200;

extern "C" {

int b200mlir_init(int device) {
  clear_error();
  std::lock_guard<std::mutex> lk(g_mu);
  return init_locked(device);
}

int b200mlir_set_stream(void *s) {
  clear_error();
  B200_TRY(ensure_ready());
  ctx().stream = (cudaStream_t)s;  // this thread's stream from now on
  l2_window_apply();               // the persistence window travels with the stream in use
  return 0;
}

int b200mlir_synchronize(void) {
  clear_error();
  B200_TRY(ensure_ready());
  B200_CUDA(cudaStreamSynchronize(ctx().stream));
  return 0;
}

int b200mlir_last_error(char *buf, int cap) {
  if (buf && cap > 0) {
    strncpy(buf, t_err_msg, (size_t)cap - 1);
    buf[cap - 1] = 0;
  }
  return t_err_code;
}

const char *b200mlir_version(void) { return "b200mlir 0.1 (sm_100a)"; }

int64_t b200mlir_launch_count(void) { return g_launches.load(); }
void b200mlir_reset_launch_count(void) { g_launches.store(0); }

int b200mlir_device_status(void) {
  clear_error();
  if (ensure_ready()) return -1;
  int h[2] = {0, 0};
  if (cudaStreamSynchronize(ctx().stream) != cudaSuccess ||
      cudaMemcpy(h, ctx().d_status, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) {
    set_error(B200MLIR_ERR_CUDA, "reading the device status word failed: %s",
              cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  if (h[0] != 0) {
    set_error(B200MLIR_ERR_DEVICE_WAIT, "a bounded device wait expired (site %d, detail %d)",
              h[0], h[1]);
    cudaMemset(ctx().d_status, 0, 256);
    // a kernel that gave up may have left arrival counters of the split-K workspace non-zero
    if (g_ws[3].p) cudaMemset(g_ws[3].p, 0, g_ws[3].cap < (1u << 20) ? g_ws[3].cap : (1u << 20));
  }
  return h[0];
}

static double *option_slot(const char *name) {
  Options &o = ctx().opt;
  if (!name) return nullptr;
  if (!strcmp(name, "rmsNormEpsilon")) return &o.rms_eps;
  if (!strcmp(name, "iterations")) return &o.iterations;
  if (!strcmp(name, "enableWeightResident")) return &o.enable_weight_resident;
  if (!strcmp(name, "gemmVariant")) return &o.gemm_variant;
  if (!strcmp(name, "kloopBlockK")) return &o.kloop_block_k;
  if (!strcmp(name, "kloopPairs")) return &o.kloop_pairs;
  if (!strcmp(name, "w8a16Variant")) return &o.w8a16_variant;
  if (!strcmp(name, "enablePDL")) return &o.enable_pdl;
  if (!strcmp(name, "gemmGroupM")) return &o.gemm_group_m;
  if (!strcmp(name, "w8a16DependentLaunch")) return &o.w8a16_dependent_launch;
  if (!strcmp(name, "gemmDependentLaunch")) return &o.gemm_dependent_launch;
  if (!strcmp(name, "attentionTiles")) return &o.attention_tiles;
  if (!strcmp(name, "mlpResidualMod")) return &o.mlp_residual_mod;
  if (!strcmp(name, "mlpResidualRem")) return &o.mlp_residual_rem;
  if (!strcmp(name, "attentionSplits")) return &o.attention_splits;
  if (!strcmp(name, "attentionStage")) return &o.attention_stage;
  if (!strcmp(name, "w8a16ExpandRows")) return &o.w8a16_expand_rows;
  if (!strcmp(name, "rowKernelWalk")) return &o.row_kernel_walk;
  if (!strcmp(name, "replicatedOperandA")) return &o.replicated_operand_a;
  if (!strcmp(name, "mlpPhaseTiming")) return &o.mlp_phase_timing;
  return nullptr;
}

int b200mlir_set_option(const char *name, double value) {
  clear_error();
  double *s = option_slot(name);
  if (!s) return set_error(B200MLIR_ERR_BAD_ARG, "unknown option '%s'", name ? name : "(null)");
  *s = value;
  return 0;
}

int b200mlir_get_option(const char *name, double *value) {
  clear_error();
  double *s = option_slot(name);
  if (!s || !value)
    return set_error(B200MLIR_ERR_BAD_ARG, "unknown option '%s'", name ? name : "(null)");
  *value = *s;
  return 0;
}

// ---- seam 2: alloc / copy ----------------------------------------------------------------
// cudaMalloc aligns to 256 bytes; the lowering keeps the op's requested alignment on every
// on-chip allocation and tile buffers ask for 2048 (HexagonMemToLLVMPass.cpp:538-542), so
// larger alignments are served by over-allocating and remembering the base.
static std::unordered_map<void *, void *> g_alias;      // tile-pointer table -> its contiguous source
static std::unordered_map<void *, void *> g_aligned;    // aligned pointer handed out -> cudaMalloc base
static std::unordered_map<void *, void *> g_tables;     // block-pointer table (pinned host) -> device block storage

static void *alloc_aligned(size_t bytes, uint64_t alignment, const char *what) {
  if (bytes == 0 || alignment == 0 || (alignment & (alignment - 1)) != 0 || alignment > 2048) {
    set_error(B200MLIR_ERR_BAD_ARG, "%s: bytes=%zu alignment=%llu unsupported (a power of two up to 2048)", what,
              bytes, (unsigned long long)alignment);
    return nullptr;
  }
  const size_t extra = alignment > 256 ? (size_t)alignment : 0;
  void *base = nullptr;
  if (cudaMalloc(&base, bytes + extra) != cudaSuccess) {
    set_error(B200MLIR_ERR_CUDA, "%s(%zu) failed: %s", what, bytes, cudaGetErrorString(cudaGetLastError()));
    return nullptr;
  }
  if (!extra) return base;
  void *p = (void *)(((uintptr_t)base + alignment - 1) & ~(uintptr_t)(alignment - 1));
  if (p != base) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_aligned[p] = base;
  }
  return p;
}

static void free_aligned(void *p) {
  void *base = p;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_aligned.find(p);
    if (it != g_aligned.end()) {
      base = it->second;
      g_aligned.erase(it);
    }
  }
  if (base && cudaFree(base) != cudaSuccess)
    set_error(B200MLIR_ERR_CUDA, "free failed: %s", cudaGetErrorString(cudaGetLastError()));
}

void *hexagon_runtime_alloc_1d(size_t bytes, uint64_t alignment, bool isVtcm) {
  clear_error();
  if (ensure_ready()) return nullptr;
  (void)isVtcm;
  return alloc_aligned(bytes, alignment, "alloc_1d");
}

void hexagon_runtime_free_1d(void *ptr) {
  clear_error();
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_alias.erase(ptr);  // freeing a tile-pointer table ends the alias, not the source
  }
  free_aligned(ptr);
}

// The indirect-tensor form (bin/runtime/src/HexagonCAPI.cpp:89-94, src/HexagonBuffer.cpp:89-113):
// ONE allocation holding numBlocks blocks at a stride of blockSize rounded up to the alignment,
// and the call returns a TABLE of the block addresses, not the storage.  The reference's table
// is ordinary memory of the processor that also runs the kernel; here it is pinned host memory
// mapped into the device's address space, so host code and kernels index the same pointer.
void *hexagon_runtime_alloc_2d(size_t numBlocks, size_t blockSize, uint64_t alignment,
                               bool isVtcm) {
  clear_error();
  if (ensure_ready()) return nullptr;
  (void)isVtcm;
  if (numBlocks == 0 || blockSize == 0) {
    set_error(B200MLIR_ERR_BAD_ARG, "alloc_2d: zero-sized request");
    return nullptr;
  }
  if (alignment == 0 || (alignment & (alignment - 1)) != 0 || alignment > 2048) {
    set_error(B200MLIR_ERR_BAD_ARG, "alloc_2d: alignment %llu unsupported", (unsigned long long)alignment);
    return nullptr;
  }
  const size_t stride = (blockSize + alignment - 1) / alignment * alignment;
  if (stride > SIZE_MAX / numBlocks) {
    set_error(B200MLIR_ERR_BAD_ARG, "alloc_2d: %zu blocks of %zu bytes overflow", numBlocks, blockSize);
    return nullptr;
  }
  void *storage = alloc_aligned(stride * numBlocks, alignment, "alloc_2d");
  if (!storage) return nullptr;
  void **table = nullptr;
  if (cudaHostAlloc((void **)&table, numBlocks * sizeof(void *), cudaHostAllocMapped | cudaHostAllocPortable) !=
      cudaSuccess) {
    set_error(B200MLIR_ERR_CUDA, "alloc_2d: block table: %s", cudaGetErrorString(cudaGetLastError()));
    free_aligned(storage);
    return nullptr;
  }
  for (size_t i = 0; i < numBlocks; ++i) table[i] = (char *)storage + i * stride;
  std::lock_guard<std::mutex> lk(g_mu);
  g_tables[table] = storage;
  return table;
}

void hexagon_runtime_free_2d(void *ptr) {
  clear_error();
  void *storage = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_tables.find(ptr);
    if (it == g_tables.end()) {
      set_error(B200MLIR_ERR_BAD_ARG, "free_2d: not a table returned by alloc_2d");
      return;
    }
    storage = it->second;
    g_tables.erase(it);
  }
  cudaFreeHost(ptr);
  free_aligned(storage);
}

void hexagon_runtime_copy(void *dst, void *src, size_t nbytes, bool, bool) {
  clear_error();
  if (ensure_ready()) return;
  if (!dst || !src) {
    set_error(B200MLIR_ERR_BAD_ARG, "copy: null pointer");
    return;
  }
  if (nbytes == 0) return;
  cudaError_t e = cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDefault, ctx().stream);
  if (e == cudaSuccess && !(is_device_ptr(dst) && is_device_ptr(src)))
    e = cudaStreamSynchronize(ctx().stream);  // host side must observe completion
  if (e != cudaSuccess) set_error(B200MLIR_ERR_CUDA, "copy failed: %s", cudaGetErrorString(e));
}

// Buffer alias (bin/runtime/include/HexagonCAPI.h:34-37, src/HexagonCAPI.cpp:113-126): a table of
// pointers to the 2048-byte tiles of a contiguous buffer, and the way back from the table.
void *hexagon_runtime_build_crouton(void *source, size_t nbytes) {
  clear_error();
  if (ensure_ready()) return nullptr;
  if (!source || nbytes == 0 || nbytes % 2048 != 0) {
    set_error(B200MLIR_ERR_BAD_ARG, "build_crouton: size must be a positive multiple of 2048 bytes");
    return nullptr;
  }
  const size_t n = nbytes / 2048;
  std::vector<void *> host(n);
  for (size_t i = 0; i < n; ++i) host[i] = (char *)source + i * 2048;
  void *table = nullptr;
  cudaError_t e = cudaMalloc(&table, n * sizeof(void *));
  if (e == cudaSuccess) e = cudaMemcpy(table, host.data(), n * sizeof(void *), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    if (table) cudaFree(table);
    set_error(B200MLIR_ERR_CUDA, "build_crouton: %s", cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_alias[table] = source;
  return table;
}

void *hexagon_runtime_get_contiguous_memref(void *table) {
  clear_error();
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_alias.find(table);
  if (it == g_alias.end()) {
    set_error(B200MLIR_ERR_BAD_ARG, "get_contiguous_memref: not a table built by build_crouton");
    return nullptr;
  }
  return it->second;
}

// ---- seam 2: residency ---------------------------------------------------------------------
int32_t hexagon_runtime_resident_scope_enter_v2(uint64_t lo, uint64_t hi) {
  clear_error();
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_res.entered) {
    g_res.entered = true;
    g_res.lo = lo;
    g_res.hi = hi;
    return 0;
  }
  if (g_res.lo == lo && g_res.hi == hi) return 0;
  set_error(B200MLIR_ERR_SCOPE, "resident scope already entered with a different id");
  return -1;
}

void *hexagon_runtime_workspace_resident_v2(uint64_t key, uint32_t bytes, uint32_t alignment,
                                            uint32_t instance) {
  clear_error();
  if (ensure_ready()) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_res.entered) {
    set_error(B200MLIR_ERR_SCOPE, "workspace_resident before resident_scope_enter");
    return nullptr;
  }
  if (bytes == 0 || !supported_alignment(alignment)) {
    set_error(B200MLIR_ERR_BAD_ARG, "workspace_resident: bytes=%u alignment=%u unsupported", bytes,
              alignment);
    return nullptr;
  }
  auto k = std::make_pair(key, instance);
  auto it = g_res.workspaces.find(k);
  if (it != g_res.workspaces.end()) {
    if (it->second.bytes != bytes || it->second.align != alignment) {
      set_error(B200MLIR_ERR_BAD_ARG,
                "workspace_resident: key reused with a different (bytes, alignment) descriptor");
      return nullptr;
    }
    it->second.freed = false;
    return it->second.ptr;
  }
  void *p = resident_alloc(bytes, alignment);
  if (!p) return nullptr;
  Resident &r = g_res.workspaces[k];
  r.ptr = p;
  r.bytes = bytes;
  r.align = alignment;
  g_res.by_ptr[p] = &r;
  return p;
}

static void *weight_resident(uint64_t src, uint32_t bytes, uint32_t alignment) {
  clear_error();
  if (ensure_ready()) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_res.entered) {
    set_error(B200MLIR_ERR_SCOPE, "weight_resident before resident_scope_enter");
    return nullptr;
  }
  if (src == 0 || bytes == 0 || !supported_alignment(alignment)) {
    set_error(B200MLIR_ERR_BAD_ARG, "weight_resident: src/bytes/alignment unsupported");
    return nullptr;
  }
  auto it = g_res.weights.find(src);
  if (it != g_res.weights.end()) {
    if (it->second.bytes != bytes || it->second.align != alignment) {
      set_error(B200MLIR_ERR_BAD_ARG,
                "weight_resident: source reused with a different (bytes, alignment) descriptor");
      return nullptr;
    }
    it->second.freed = false;
    return it->second.ptr;  // same address forever; the source is not read again
  }
  void *p = resident_alloc(bytes, alignment);
  if (!p) return nullptr;
  cudaError_t e = cudaMemcpyAsync(p, (const void *)(uintptr_t)src, bytes, cudaMemcpyDefault,
                                  ctx().stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx().stream);
  if (e != cudaSuccess) {
    set_error(B200MLIR_ERR_CUDA, "weight_resident: copy of the image failed: %s",
              cudaGetErrorString(e));
    return nullptr;
  }
  Resident &r = g_res.weights[src];
  r.ptr = p;
  r.bytes = bytes;
  r.align = alignment;
  g_res.by_ptr[p] = &r;
  return p;
}

void *hexagon_runtime_weight_resident_v2(uint64_t src, uint32_t bytes, uint32_t alignment) {
  return weight_resident(src, bytes, alignment);
}
// The reference keeps a DDR mirror for weights too large for VTCM; with one
// HBM pool both entry points name the same resident store.
void *hexagon_runtime_weight_resident_ddr_v2(uint64_t src, uint32_t bytes, uint32_t alignment) {
  return weight_resident(src, bytes, alignment);
}

int32_t hexagon_runtime_resident_free_v2(void *ptr, uint32_t bytes) {
  clear_error();
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_res.by_ptr.find(ptr);
  if (it == g_res.by_ptr.end() || it->second->bytes != bytes) {
    set_error(B200MLIR_ERR_BAD_ARG, "resident_free: pointer/bytes match no registered resident");
    return -1;
  }
  it->second->freed = true;  // recorded; the pinned block is not released
  return 0;
}

void hexagon_runtime_hmx_ensure(void) {}
void hexagon_runtime_hmx_unlock(void) {}

// ---- seam 2: asynchronous copies -----------------------------------------------------------
static uint32_t dma_issue(void *src, void *dst, uint32_t width, uint32_t height,
                          uint32_t srcStride, uint32_t dstStride, int *status) {
  clear_error();
  const uint32_t kNone = 0xFFFFFFFFu;
  auto refuse = [&](const char *why) {
    if (status) *status = -1;
    set_error(B200MLIR_ERR_BAD_ARG, "dma start refused: %s", why);
    return kNone;
  };
  if (ensure_ready()) {
    if (status) *status = -1;
    return kNone;
  }
  if (!src || !dst) return refuse("null address");
  if (width == 0 || height == 0) return refuse("empty transfer");
  if (height > 1 && (srcStride < width || dstStride < width)) return refuse("stride below width");
  std::lock_guard<std::mutex> lk(g_mu);
  CopyRing &r = g_ring;
  if (!r.stream && cudaStreamCreateWithFlags(&r.stream, cudaStreamNonBlocking) != cudaSuccess)
    return refuse("copy stream creation failed");
  // Slot allocation follows the reference ring (bin/runtime/UserDMA/RingBuffer.h:103-116):
  // descriptors no longer in flight are reclaimed whether or not anybody waited on their token,
  // and a full ring blocks on its oldest descriptor instead of refusing the start.
  int slot = -1;
  for (int i = 0; i < CopyRing::kSlots && slot < 0; ++i)
    if (!r.used[i]) slot = i;
  if (slot < 0) {
    int oldest = 0;
    for (int i = 0; i < CopyRing::kSlots; ++i) {
      if (cudaEventQuery(r.ev[i]) == cudaSuccess) {
        r.used[i] = false;
        if (slot < 0) slot = i;
      } else {
        cudaGetLastError();  // cudaErrorNotReady is not an error here
        if ((int32_t)(r.token_of[i] - r.token_of[oldest]) < 0) oldest = i;
      }
    }
    if (slot < 0) {
      if (cudaEventSynchronize(r.ev[oldest]) != cudaSuccess) return refuse("waiting for the oldest descriptor failed");
      r.used[oldest] = false;
      slot = oldest;
    }
  }
  if (!r.ev[slot] &&
      cudaEventCreateWithFlags(&r.ev[slot], cudaEventDisableTiming) != cudaSuccess)
    return refuse("event creation failed");
  cudaError_t e =
      height == 1
          ? cudaMemcpyAsync(dst, src, width, cudaMemcpyDefault, r.stream)
          : cudaMemcpy2DAsync(dst, dstStride, src, srcStride, width, height, cudaMemcpyDefault,
                              r.stream);
  if (e == cudaSuccess) e = cudaEventRecord(r.ev[slot], r.stream);
  if (e != cudaSuccess) return refuse(cudaGetErrorString(e));
  uint32_t token = r.next++;
  if (token == kNone) token = r.next++;
  r.used[slot] = true;
  r.token_of[slot] = token;
  if (status) *status = 0;
  return token;
}

uint32_t hexagon_runtime_dma_start(void *src, int, void *dst, int, uint32_t length, bool, bool,
                                   int *status) {
  return dma_issue(src, dst, length, 1, length, length, status);
}

uint32_t hexagon_runtime_dma2d_start(void *src, int, void *dst, int, uint32_t width,
                                     uint32_t height, uint32_t srcStride, uint32_t dstStride, bool,
                                     bool, bool, uint32_t, int *status) {
  return dma_issue(src, dst, width, height, srcStride, dstStride, status);
}

void hexagon_runtime_dma_wait(uint32_t token) {
  clear_error();
  if (token == 0xFFFFFFFFu) return;
  cudaEvent_t ev = nullptr;
  int slot = -1;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    for (int i = 0; i < CopyRing::kSlots; ++i)
      if (g_ring.used[i] && g_ring.token_of[i] == token) {
        slot = i;
        ev = g_ring.ev[i];
        break;
      }
  }
  if (slot < 0) return;  // unknown or already retired: nothing to wait for
  cudaError_t e = cudaEventSynchronize(ev);
  if (e != cudaSuccess) set_error(B200MLIR_ERR_CUDA, "dma_wait: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_ring.token_of[slot] == token) g_ring.used[slot] = false;  // (a start may have reclaimed and reused the slot meanwhile)
}

int b200mlir_benchmark(b200mlir_thunk fn, void *user, int iterations, double *mean_us) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!fn || iterations < 1 || !mean_us)
    return set_error(B200MLIR_ERR_BAD_ARG, "benchmark: null thunk / iterations < 1");
  cudaStream_t s = ctx().stream;
  cudaEvent_t e0, e1;
  B200_CUDA(cudaEventCreate(&e0));
  B200_CUDA(cudaEventCreate(&e1));
  fn(user);  // discarded warm call (hexagon_launcher_base.py:114-153)
  B200_CUDA(cudaStreamSynchronize(s));
  B200_CUDA(cudaEventRecord(e0, s));
  for (int i = 0; i < iterations; ++i) fn(user);
  B200_CUDA(cudaEventRecord(e1, s));
  B200_CUDA(cudaEventSynchronize(e1));
  float ms = 0;
  B200_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *mean_us = (double)ms * 1000.0 / iterations;
  return t_err_code;
}

}  // extern "C"
