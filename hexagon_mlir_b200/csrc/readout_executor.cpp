// The read-out executor of seam 2
// (qcom_hexagon_backend/bin/runtime/include/HmxVectorExecutor.h:86-156, implementation
// bin/runtime/multithreading/HmxVectorExecutor.cpp:725-905): a resident host thread that runs a
// caller-supplied read-out function on groups of accumulator rows while the caller's thread goes
// on issuing matrix work.  Inside this library's GEMM kernels the same split is done by the
// epilogue warps and two TMEM accumulator stages; these four symbols exist for hosts whose
// compiled kernels call them, and keep the reference's contract:
//   * configure: 0, or -1 (null function), -2 (more than one thread asked for: one is used),
//     -3 (the thread would not start); a different function waits for the running read-out first;
//   * publish: single producer, NEVER blocks, returns how many batches it accepted — fewer than
//     `count` only when the 16-slot ring (15 usable) is full, and the caller must read out the
//     rest itself; 0 before configure and after shutdown;
//   * drain: returns once every accepted batch has been read out (two monotone totals, so the
//     barrier cannot be stepped over);
//   * shutdown: drain, then release the thread.
// The consumer spins a bounded number of times before it parks on a condition variable, and so
// does drain: no wait here is unbounded while the other side is alive.
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <mutex>
#include <thread>

#include "b200mlir_capi.h"

namespace {

constexpr uint32_t kRingCapacity = 16;  // HmxVectorExecutor.cpp: kRingCapacity
constexpr uint32_t kRingMask = kRingCapacity - 1;
constexpr uint32_t kUsable = kRingCapacity - 1;
constexpr unsigned kPollCount = 2000;  // bounded spin before parking (same figure as the reference)

struct Executor {
  B200HmxReadoutBatch slots[kRingCapacity];
  std::atomic<uint32_t> idx_write{0};        // producer cursor
  std::atomic<uint32_t> idx_read{0};         // consumer cursor
  std::atomic<uint32_t> published_total{0};  // batches accepted, monotone
  std::atomic<uint32_t> retired_total{0};    // batches read out, monotone
  std::atomic<B200HmxReadoutFn> fn{nullptr};
  std::atomic<bool> stop{false};
  std::atomic<bool> started{false};
  std::atomic<uint64_t> batches_run{0};
  std::mutex mu;
  std::condition_variable work_cv;    // consumer parks here
  std::condition_variable retire_cv;  // drain parks here
  std::thread thread;
};

// Never destroyed: a resident thread may still be parked when the process exits, and a joinable
// std::thread must not meet its destructor.
Executor &g_exec = *new Executor;

void consumer_loop(Executor *e) {
  for (;;) {
    unsigned spins = kPollCount;
    for (;;) {
      const uint32_t ir = e->idx_read.load(std::memory_order_relaxed);
      const uint32_t iw = e->idx_write.load(std::memory_order_acquire);
      if (ir != iw) {
        // one call per batch: the group size travels with the descriptor, groups are never merged or split
        B200HmxReadoutFn fn = e->fn.load(std::memory_order_acquire);
        if (fn) fn(&e->slots[ir], 1);
        e->idx_read.store((ir + 1) & kRingMask, std::memory_order_release);
        e->batches_run.fetch_add(1, std::memory_order_relaxed);
        {
          std::lock_guard<std::mutex> lk(e->mu);
          e->retired_total.fetch_add(1, std::memory_order_release);
        }
        e->retire_cv.notify_all();
        spins = kPollCount;
        continue;
      }
      if (e->stop.load(std::memory_order_acquire)) return;
      if (spins != 0) {
        --spins;
        continue;
      }
      std::unique_lock<std::mutex> lk(e->mu);
      e->work_cv.wait(lk, [&] {
        return e->stop.load(std::memory_order_acquire) ||
               e->idx_read.load(std::memory_order_relaxed) != e->idx_write.load(std::memory_order_acquire);
      });
      spins = kPollCount;
    }
  }
}

void drain_locked(Executor &e) {
  if (!e.started.load(std::memory_order_acquire)) return;
  const uint32_t target = e.published_total.load(std::memory_order_acquire);
  unsigned spins = kPollCount;
  while (e.retired_total.load(std::memory_order_acquire) != target) {
    if (spins != 0) {
      --spins;
      continue;
    }
    std::unique_lock<std::mutex> lk(e.mu);
    e.retire_cv.wait(lk, [&] { return e.retired_total.load(std::memory_order_acquire) == target; });
  }
}

}  // namespace

extern "C" {

int32_t hexagon_runtime_hmx_exec_configure(B200HmxReadoutFn fn, int32_t numThreads) {
  if (fn == nullptr) return B200_HMX_EXEC_ERR_NULL_FN;
  int32_t status = B200_HMX_EXEC_OK;
  if (numThreads < 1) numThreads = 1;
  if (numThreads != 1) status = B200_HMX_EXEC_ERR_THREADS;  // one read-out thread, whatever was asked for
  Executor &e = g_exec;
  drain_locked(e);  // a different function waits for the current read-out first
  e.fn.store(fn, std::memory_order_release);
  if (!e.started.load(std::memory_order_acquire)) {
    e.stop.store(false, std::memory_order_release);
    try {
      e.thread = std::thread(consumer_loop, &e);
    } catch (...) {
      e.fn.store(nullptr, std::memory_order_release);
      return B200_HMX_EXEC_ERR_CREATE;
    }
    e.started.store(true, std::memory_order_release);
  }
  return status;
}

uint32_t hexagon_runtime_hmx_exec_publish(const B200HmxReadoutBatch *batches, uint32_t count) {
  Executor &e = g_exec;
  if (batches == nullptr || count == 0u) return 0;
  if (!e.started.load(std::memory_order_acquire) || e.fn.load(std::memory_order_acquire) == nullptr) return 0;
  if (e.stop.load(std::memory_order_acquire)) return 0;
  const uint32_t iw = e.idx_write.load(std::memory_order_relaxed);
  const uint32_t ir = e.idx_read.load(std::memory_order_acquire);
  const uint32_t occupancy = (iw - ir) & kRingMask;
  if (occupancy >= kUsable) return 0;  // full: the caller reads these out itself
  const uint32_t free_slots = kUsable - occupancy;
  const uint32_t accepted = count < free_slots ? count : free_slots;
  for (uint32_t i = 0; i < accepted; ++i) e.slots[(iw + i) & kRingMask] = batches[i];
  {
    std::lock_guard<std::mutex> lk(e.mu);  // pairs with the consumer's parked predicate: no lost wake-up
    e.published_total.fetch_add(accepted, std::memory_order_release);
    e.idx_write.store((iw + accepted) & kRingMask, std::memory_order_release);
  }
  e.work_cv.notify_one();
  return accepted;
}

void hexagon_runtime_hmx_exec_drain(void) { drain_locked(g_exec); }

void hexagon_runtime_hmx_exec_shutdown(void) {
  Executor &e = g_exec;
  if (!e.started.load(std::memory_order_acquire)) return;
  drain_locked(e);
  {
    std::lock_guard<std::mutex> lk(e.mu);
    e.stop.store(true, std::memory_order_release);
  }
  e.work_cv.notify_all();
  if (e.thread.joinable()) e.thread.join();
  e.started.store(false, std::memory_order_release);
  e.fn.store(nullptr, std::memory_order_release);
}

uint64_t b200mlir_hmx_exec_batches_run(void) { return g_exec.batches_run.load(std::memory_order_relaxed); }

}  // extern "C"
