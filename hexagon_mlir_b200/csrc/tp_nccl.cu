// Tensor-parallel plumbing in the C++ host: one NCCL communicator per process (one process per
// GPU), the MLP block whose output is summed over the ranks with ncclAllReduce, and the exchange
// of row slabs for host-buffer GEMMs whose A operand every rank holds.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy already loaded into the process
// when there is one), so the library loads and every single-GPU entry works on a machine without
// NCCL; the tensor-parallel entries then fail with B200MLIR_ERR_UNSUPPORTED.  Only the handful of
// NCCL calls used here are declared, with NCCL's published signatures.
//
// No counterpart in the reference, which drives one device; the partitioning it applies inside a
// device (column blocks of one resident weight per program:
// qcom_hexagon_backend/test/Dialect/Hmx/Transforms/weight-resident-nsplit.mlir:9-27) is the cut
// made across GPUs here.
#include <dlfcn.h>

#include <mutex>

#include "common.h"

namespace b200 {
namespace {

struct NcclUniqueId {
  char internal[128];
};
typedef void *NcclComm;
typedef int (*FnGetUniqueId)(NcclUniqueId *);
typedef int (*FnCommInitRank)(NcclComm *, int, NcclUniqueId, int);
typedef int (*FnCommDestroy)(NcclComm);
typedef int (*FnAllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*FnAllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t);
typedef const char *(*FnGetErrorString)(int);
typedef int (*FnGroup)(void);
constexpr int kNcclInt8 = 0, kNcclFloat16 = 6, kNcclSum = 0;  // ncclDataType_t / ncclRedOp_t values

struct Nccl {
  void *handle = nullptr;
  FnGetUniqueId get_unique_id = nullptr;
  FnCommInitRank comm_init_rank = nullptr;
  FnCommDestroy comm_destroy = nullptr;
  FnAllReduce all_reduce = nullptr;
  FnAllGather all_gather = nullptr;
  FnGetErrorString error_string = nullptr;
  FnGroup group_start = nullptr, group_end = nullptr;
};

// One rank's exchange window: [4 KB of flag words][A buffer], one cudaMalloc, exported through
// CUDA IPC and mapped by every other rank of the group.
constexpr size_t kWindowHeader = 4096;
constexpr long long kExchangeWaitCycles = 2000000000LL;  // about a second: the ranks entered the call together
struct ExchangeWindow {
  char *local = nullptr;
  size_t a_bytes = 0;
  char *peer[kMaxPushRanks] = {};  // peer[rank] == local
  char *d_small = nullptr;         // device scratch of the handle gathers; its first word holds the sequence number
  uint32_t seq = 0;                // collective calls so far (every rank counts the same calls)
  bool refused = false;            // the machine gave no mapping, or the environment asked for NCCL: stay on ncclAllGather
  cudaStream_t push = nullptr;
};

struct TpState {
  Nccl api;
  ExchangeWindow xw;
  NcclComm comm = nullptr;
  int rank = 0, world = 1;
  cudaStream_t comm_stream = nullptr;  // collectives of chunk i run here while chunk i+1 is computed
};

std::mutex g_tp_mu;
TpState g_tp;

int load_nccl(Nccl &n) {
  if (n.handle) return 0;
  void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the host application brought, if any
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return set_error(B200MLIR_ERR_UNSUPPORTED, "tensor parallelism needs NCCL: %s", dlerror());
  n.get_unique_id = (FnGetUniqueId)dlsym(h, "ncclGetUniqueId");
  n.comm_init_rank = (FnCommInitRank)dlsym(h, "ncclCommInitRank");
  n.comm_destroy = (FnCommDestroy)dlsym(h, "ncclCommDestroy");
  n.all_reduce = (FnAllReduce)dlsym(h, "ncclAllReduce");
  n.all_gather = (FnAllGather)dlsym(h, "ncclAllGather");
  n.error_string = (FnGetErrorString)dlsym(h, "ncclGetErrorString");
  n.group_start = (FnGroup)dlsym(h, "ncclGroupStart");
  n.group_end = (FnGroup)dlsym(h, "ncclGroupEnd");
  if (!n.get_unique_id || !n.comm_init_rank || !n.comm_destroy || !n.all_reduce || !n.all_gather || !n.error_string ||
      !n.group_start || !n.group_end)
    return set_error(B200MLIR_ERR_UNSUPPORTED, "libnccl.so.2 lacks a symbol this library binds");
  n.handle = h;
  return 0;
}

#define B200_NCCL(expr)                                                                                   \
  do {                                                                                                    \
    int _r = (expr);                                                                                      \
    if (_r != 0)                                                                                          \
      return set_error(B200MLIR_ERR_CUDA, "%s failed: %s", #expr, g_tp.api.error_string ? g_tp.api.error_string(_r) : "?"); \
  } while (0)

}  // namespace

int tp_rank() { return g_tp.rank; }
int tp_world() { return g_tp.comm ? g_tp.world : 1; }

// rows [r0, r0 + rows) of every rank's slab, gathered in rank order into `dst` (rank r's slab at
// dst + r * bytes_per_rank); `src` is this rank's slab.  In-place when src == dst + rank * bytes.
int tp_all_gather_bytes(const void *src, void *dst, size_t bytes_per_rank, cudaStream_t s) {
  if (!g_tp.comm) return set_error(B200MLIR_ERR_UNSUPPORTED, "tensor-parallel group not initialised (b200mlir_tp_init)");
  B200_NCCL(g_tp.api.all_gather(src, dst, bytes_per_rank, kNcclInt8, g_tp.comm, s));
  return 0;
}

int tp_all_reduce_f16(void *buf, size_t count, cudaStream_t s) {
  if (!g_tp.comm) return set_error(B200MLIR_ERR_UNSUPPORTED, "tensor-parallel group not initialised (b200mlir_tp_init)");
  B200_NCCL(g_tp.api.all_reduce(buf, buf, count, kNcclFloat16, kNcclSum, g_tp.comm, s));
  return 0;
}

static int comm_stream_locked(cudaStream_t *s) {  // g_tp_mu held
  if (!g_tp.comm_stream) B200_CUDA(cudaStreamCreateWithFlags(&g_tp.comm_stream, cudaStreamNonBlocking));
  *s = g_tp.comm_stream;
  return 0;
}
int tp_comm_stream(cudaStream_t *s) {
  std::lock_guard<std::mutex> lk(g_tp_mu);
  return comm_stream_locked(s);
}

namespace {

__global__ void set_word_kernel(uint32_t *p, uint32_t v) { *p = v; }

// One thread per peer rank: spin (bounded) until that rank's flag reaches `seq`.  The flag is
// written by the peer's copy engine after its slab; a wait that runs out records {site 47, rank}
// in the status word, and every later wait of the call returns at once.
__global__ void wait_flags_kernel(const uint32_t *flags, int world, int self, uint32_t seq, int *status,
                                  long long limit_cycles) {
  const int r = threadIdx.x;
  if (r >= world || r == self) return;
  if (*(volatile int *)status != 0) return;
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
    if ((int32_t)(v - seq) >= 0) return;
    if (clock64() - t0 > limit_cycles) {
      if (atomicCAS(status, 0, 47) == 0) status[1] = r;
      return;
    }
    __nanosleep(256);
  }
}

// every rank's `bytes` (at most 120) gathered into host memory, rank order; also a barrier.
// g_tp_mu is held by the caller.
int gather_small(ExchangeWindow &w, const void *mine, size_t bytes, char *all_host /* world * 128 */) {
  cudaStream_t s;
  B200_TRY(comm_stream_locked(&s));
  char *slots = w.d_small + 256;  // after the sequence word
  B200_CUDA(cudaMemcpyAsync(slots + (size_t)g_tp.rank * 128, mine, bytes, cudaMemcpyHostToDevice, s));
  B200_NCCL(g_tp.api.all_gather(slots + (size_t)g_tp.rank * 128, slots, 128, kNcclInt8, g_tp.comm, s));
  B200_CUDA(cudaMemcpyAsync(all_host, slots, (size_t)g_tp.world * 128, cudaMemcpyDeviceToHost, s));
  B200_CUDA(cudaStreamSynchronize(s));
  return 0;
}

void close_peers(ExchangeWindow &w) {
  for (int r = 0; r < kMaxPushRanks; ++r) {
    if (w.peer[r] && w.peer[r] != w.local) cudaIpcCloseMemHandle(w.peer[r]);
    w.peer[r] = nullptr;
  }
  cudaGetLastError();
}

// Collective: every rank frees its window and creates one of `a_bytes`, and the ranks map each
// other's.  Nothing of the old windows is in flight: every call that used them waited for its
// own streams before it returned, and the gather below is passed only when all ranks are here.
int window_grow(ExchangeWindow &w, size_t a_bytes) {
  char all[kMaxPushRanks * 128];
  char mine[128] = {};
  close_peers(w);
  B200_TRY(gather_small(w, mine, 8, all));  // every mapping of the old windows is closed
  if (w.local) B200_CUDA(cudaFree(w.local));
  w.local = nullptr;
  w.a_bytes = 0;
  char *p = nullptr;
  cudaIpcMemHandle_t h;
  int ok = cudaMalloc(&p, kWindowHeader + a_bytes) == cudaSuccess ? 1 : 0;
  if (ok) ok = cudaMemset(p, 0, kWindowHeader) == cudaSuccess;
  if (ok) ok = cudaIpcGetMemHandle(&h, p) == cudaSuccess;
  cudaGetLastError();
  static_assert(sizeof(cudaIpcMemHandle_t) <= 64, "handle slot");
  memcpy(mine, &ok, 4);
  if (ok) memcpy(mine + 8, &h, sizeof(h));
  B200_TRY(gather_small(w, mine, 8 + sizeof(h), all));
  int all_ok = 1;
  for (int r = 0; r < g_tp.world; ++r) {
    int o;
    memcpy(&o, all + r * 128, 4);
    all_ok &= o;
  }
  if (all_ok) {
    for (int r = 0; r < g_tp.world && ok; ++r) {
      if (r == g_tp.rank) { w.peer[r] = p; continue; }
      cudaIpcMemHandle_t hr;
      memcpy(&hr, all + r * 128 + 8, sizeof(hr));
      void *q = nullptr;
      if (cudaIpcOpenMemHandle(&q, hr, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) ok = 0;
      w.peer[r] = (char *)q;
    }
    cudaGetLastError();
  }
  // every rank mapped every window, or none is used
  memcpy(mine, &ok, 4);
  B200_TRY(gather_small(w, mine, 8, all));
  for (int r = 0; r < g_tp.world; ++r) {
    int o;
    memcpy(&o, all + r * 128, 4);
    all_ok &= o;
  }
  if (!all_ok) {
    close_peers(w);
    if (p) cudaFree(p);
    cudaGetLastError();
    w.refused = true;
    B200_TRY(gather_small(w, mine, 8, all));  // closed everywhere before anyone moves on
    return 0;
  }
  w.local = p;
  w.a_bytes = a_bytes;
  return 0;
}

}  // namespace

int tp_slab_exchange_begin(size_t a_bytes, SlabExchange *x) {
  *x = SlabExchange();
  std::lock_guard<std::mutex> lk(g_tp_mu);
  if (!g_tp.comm) return set_error(B200MLIR_ERR_UNSUPPORTED, "tensor-parallel group not initialised (b200mlir_tp_init)");
  ExchangeWindow &w = g_tp.xw;
  if (w.refused) return 0;
  if (!w.d_small) {
    const char *e = getenv("B200MLIR_SLAB_EXCHANGE");  // "nccl": keep the slabs on ncclAllGather
    if (e && strcmp(e, "nccl") == 0) {
      w.refused = true;
      return 0;
    }
    B200_CUDA(cudaMalloc(&w.d_small, 256 + kMaxPushRanks * 128));
    B200_CUDA(cudaMemset(w.d_small, 0, 256 + kMaxPushRanks * 128));
    B200_CUDA(cudaStreamCreateWithFlags(&w.push, cudaStreamNonBlocking));
  }
  const size_t want = (a_bytes + 4095) & ~(size_t)4095;
  if (want > w.a_bytes) {
    B200_TRY(window_grow(w, want));
    if (w.refused) return 0;
  } else {
    // every rank is in this call, so every rank has finished the one before: the single A buffer
    // and the flags can be written again
    char all[kMaxPushRanks * 128], mine[8] = {};
    B200_TRY(gather_small(w, mine, 8, all));
  }
  ++w.seq;
  set_word_kernel<<<1, 1, 0, w.push>>>((uint32_t *)w.d_small, w.seq);
  B200_TRY(check_launch("slab exchange sequence word"));
  x->a = w.local + kWindowHeader;
  x->flags = (uint32_t *)w.local;
  for (int r = 0; r < g_tp.world; ++r) {
    x->peer_a[r] = w.peer[r] + kWindowHeader;
    x->peer_flags[r] = (uint32_t *)w.peer[r];
  }
  x->d_seq = (const uint32_t *)w.d_small;
  x->seq = w.seq;
  x->push = w.push;
  return 0;
}

int tp_slab_exchange_wait(const SlabExchange &x, int panel, cudaStream_t s) {
  wait_flags_kernel<<<1, 32, 0, s>>>(x.flags + (size_t)panel * kMaxPushRanks, g_tp.world, g_tp.rank, x.seq, ctx().d_status,
                                     kExchangeWaitCycles);
  return check_launch("slab exchange wait");
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200mlir_tp_unique_id(void *id128) {
  clear_error();
  if (!id128) return set_error(B200MLIR_ERR_BAD_ARG, "tp_unique_id: null buffer (128 bytes wanted)");
  std::lock_guard<std::mutex> lk(g_tp_mu);
  B200_TRY(load_nccl(g_tp.api));
  B200_NCCL(g_tp.api.get_unique_id((NcclUniqueId *)id128));
  return 0;
}

int b200mlir_tp_init(const void *id128, int rank, int world) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!id128 || world < 1 || world > kMaxPushRanks || rank < 0 || rank >= world)
    return set_error(B200MLIR_ERR_BAD_ARG, "tp_init: id, 0 <= rank < world <= %d", kMaxPushRanks);
  std::lock_guard<std::mutex> lk(g_tp_mu);
  if (g_tp.comm) return set_error(B200MLIR_ERR_BAD_ARG, "tp_init: a group of %d ranks is already initialised", g_tp.world);
  B200_TRY(load_nccl(g_tp.api));
  NcclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  NcclComm comm = nullptr;
  B200_NCCL(g_tp.api.comm_init_rank(&comm, world, id, rank));
  g_tp.comm = comm;
  g_tp.rank = rank;
  g_tp.world = world;
  return 0;
}

int b200mlir_tp_info(int *rank, int *world) {
  if (rank) *rank = g_tp.comm ? g_tp.rank : 0;
  if (world) *world = g_tp.comm ? g_tp.world : 1;
  return g_tp.comm ? 1 : 0;
}

int b200mlir_tp_slab_exchange_mode(void) {
  std::lock_guard<std::mutex> lk(g_tp_mu);
  return g_tp.xw.refused ? 2 : g_tp.xw.local ? 1 : 0;
}

int b200mlir_tp_shutdown(void) {
  clear_error();
  std::lock_guard<std::mutex> lk(g_tp_mu);
  if (!g_tp.comm) return 0;
  cudaStreamSynchronize(ctx().stream);
  if (g_tp.comm_stream) cudaStreamSynchronize(g_tp.comm_stream);
  ExchangeWindow &w = g_tp.xw;
  if (w.push) cudaStreamSynchronize(w.push);
  if (w.d_small) {
    // mappings closed on every rank before any window is freed
    close_peers(w);
    char all[kMaxPushRanks * 128], mine[8] = {};
    gather_small(w, mine, 8, all);
    if (w.local) cudaFree(w.local);
    cudaFree(w.d_small);
    if (w.push) cudaStreamDestroy(w.push);
    cudaGetLastError();
  }
  w = ExchangeWindow();
  int r = g_tp.api.comm_destroy(g_tp.comm);
  g_tp.comm = nullptr;
  g_tp.world = 1;
  g_tp.rank = 0;
  if (r != 0) return set_error(B200MLIR_ERR_CUDA, "ncclCommDestroy failed: %s", g_tp.api.error_string(r));
  return 0;
}

int b200mlir_tp_all_reduce_float16(void *buf, int64_t count) {
  clear_error();
  B200_TRY(ensure_ready());
  if (!buf || count < 0 || !is_device_ptr(buf)) return set_error(B200MLIR_ERR_BAD_ARG, "tp_all_reduce: a device buffer is required");
  if (count == 0) return 0;
  return tp_all_reduce_f16(buf, (size_t)count, ctx().stream);
}

}  // extern "C"
