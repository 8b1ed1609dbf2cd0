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

struct TpState {
  Nccl api;
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

int tp_comm_stream(cudaStream_t *s) {
  std::lock_guard<std::mutex> lk(g_tp_mu);
  if (!g_tp.comm_stream) B200_CUDA(cudaStreamCreateWithFlags(&g_tp.comm_stream, cudaStreamNonBlocking));
  *s = g_tp.comm_stream;
  return 0;
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

int b200mlir_tp_shutdown(void) {
  clear_error();
  std::lock_guard<std::mutex> lk(g_tp_mu);
  if (!g_tp.comm) return 0;
  cudaStreamSynchronize(ctx().stream);
  if (g_tp.comm_stream) cudaStreamSynchronize(g_tp.comm_stream);
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
