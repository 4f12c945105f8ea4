// A team of parked workers: one pinned thread per core of every NUMA node, created once through the thread pools and
// then re-used for any number of jobs.  Each worker sleeps on its own futex word (an epoch, the multi-shot form of the
// reference's one-shot MutexGate, threading/linux_threading.mojo:174-198) and reports completion on a second one, so
// handing a job to a worker costs a store and a wake instead of a clone3 + exit, which is what `ThreadPool::launch`
// (threading/linux_threading.mojo:103-121) pays per task.  All waits are bounded.
#pragma once
#include <atomic>
#include <cstdint>
#include <vector>

#include "heap_move_array.hpp"
#include "numa.hpp"
#include "pool.hpp"

namespace hostrt {

struct alignas(64) TeamSlot {
  std::atomic<uint32_t> go;      // epoch of the job to run; the worker sleeps while it equals the last one it ran
  std::atomic<uint32_t> done;    // epoch of the last finished job
  WorkerFn fn;
  uint64_t arg;
  uint32_t quit;
  int node;
  int cpu;                       // the one CPU this worker pins itself to (-1: the node's mask)
};

class WorkerTeam {
 public:
  WorkerTeam(const NumaInfo& info, int max_workers_per_node);
  WorkerTeam(const WorkerTeam&) = delete;
  WorkerTeam& operator=(const WorkerTeam&) = delete;
  ~WorkerTeam();                                  // tells every worker to leave and joins the pools (bounded)
  explicit operator bool() const { return valid_; }
  int size() const { return static_cast<int>(slots_.size()); }
  int node_of(int worker) const { return slots_[worker].node; }
  // fn(args[i]) on worker i for every i < size(); 0, or -ETIMEDOUT if a worker did not finish in time.
  // After a timeout the team is invalid (every later run() returns -EINVAL).  run() then waits up to
  // kTimeoutGraceNs more for the stragglers before it returns; if `stragglers()` is still true afterwards, workers
  // may still be using `args` and what it points to: that storage has to outlive the team (or the process has to
  // end, as ThreadPool::~ThreadPool does for live threads).
  static constexpr long kTimeoutGraceNs = 2'000'000'000l;
  long run(WorkerFn fn, const uint64_t* args, long timeout_ns = 120'000'000'000l);
  bool stragglers() const { return stragglers_; }
  uint64_t jobs_run() const { return epoch_; }

 private:
  std::vector<TeamSlot> slots_;
  HeapMoveArray<ThreadPool> pools_;
  uint32_t epoch_ = 0;
  bool valid_ = false;
  bool stragglers_ = false;
};

}  // namespace hostrt
