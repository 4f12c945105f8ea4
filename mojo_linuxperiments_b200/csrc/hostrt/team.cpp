#include "team.hpp"

#include <climits>

#include "sys.hpp"

namespace hostrt {

namespace {

constexpr uint32_t kFutex = futex2::SIZE_U32 | futex2::PRIVATE;

void team_loop(uint64_t slot_p, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t) {
  auto* s = reinterpret_cast<TeamSlot*>(slot_p);
  if (s->cpu >= 0 && s->cpu < 1024) {
    // one worker per core: a parked thread that wakes on a CPU another worker occupies would halve both
    uint64_t mask[16] = {};
    mask[s->cpu >> 6] = 1ull << (s->cpu & 63);
    sys_sched_setaffinity(0, sizeof(mask), mask);
  }
  uint32_t seen = 0;
  for (;;) {
    // a short spin keeps back-to-back jobs off the futex path, then sleep until the epoch moves
    for (int i = 0; i < 2000 && s->go.load(std::memory_order_acquire) == seen; ++i) asm volatile("pause");
    while (s->go.load(std::memory_order_acquire) == seen) sys_futex_wait(&s->go, seen, kFutex, 1'000'000'000l);
    seen = s->go.load(std::memory_order_acquire);
    if (s->quit) return;
    s->fn(s->arg, 0, 0, 0, 0, 0);
    s->done.store(seen, std::memory_order_release);
    sys_futex_wake(&s->done, INT_MAX, kFutex);
  }
}

}  // namespace

WorkerTeam::WorkerTeam(const NumaInfo& info, int max_workers_per_node) : pools_(info.num_nodes() > 0 ? info.num_nodes() : 1) {
  const int nn = info.num_nodes();
  if (nn == 0) return;
  std::vector<int> per_node(nn);
  int total = 0;
  for (int k = 0; k < nn; ++k) {
    int c = static_cast<int>(info.nodes()[k].cpu_ids.size());
    if (max_workers_per_node > 0 && c > max_workers_per_node) c = max_workers_per_node;
    per_node[k] = c;
    total += c;
  }
  if (total == 0) return;
  slots_ = std::vector<TeamSlot>(total);
  int w = 0;
  for (int k = 0; k < nn; ++k) {
    // A node that is online but has no CPUs (memory-only: CXL or device memory) gets no pool and no workers; the
    // pools of the other nodes are indexed by their own running count, not by the node's position.
    if (per_node[k] == 0) continue;
    const int node = info.nodes()[k].id;
    auto m = info.get_node_mask<128>(node);
    const size_t pi = pools_.size();
    pools_.emplace(per_node[k], m.ptr(), size_t(128), node, stack_size::DEFAULT);
    if (!pools_[pi]) return;
    for (int i = 0; i < per_node[k]; ++i, ++w) {
      TeamSlot& s = slots_[w];
      s.go.store(0); s.done.store(0); s.fn = nullptr; s.arg = 0; s.quit = 0; s.node = node;
      s.cpu = i < static_cast<int>(info.nodes()[k].cpu_ids.size()) ? info.nodes()[k].cpu_ids[i] : -1;
      if (pools_[pi].launch(&team_loop, reinterpret_cast<uint64_t>(&s)) < 0) return;
    }
  }
  valid_ = true;
}

WorkerTeam::~WorkerTeam() {
  ++epoch_;
  for (auto& s : slots_) {
    s.quit = 1;
    s.go.store(epoch_, std::memory_order_release);
    sys_futex_wake(&s.go, INT_MAX, kFutex);
  }
  for (size_t k = 0; k < pools_.size(); ++k)
    if (pools_[k]) pools_[k].wait_all(10'000'000'000l);
}

long WorkerTeam::run(WorkerFn fn, const uint64_t* args, long timeout_ns) {
  if (!valid_) return -err::kINVAL;
  ++epoch_;
  for (size_t i = 0; i < slots_.size(); ++i) {
    TeamSlot& s = slots_[i];
    s.fn = fn;
    s.arg = args[i];
    s.go.store(epoch_, std::memory_order_release);
    sys_futex_wake(&s.go, 1, kFutex);
  }
  const long deadline = sys_clock_monotonic_ns() + timeout_ns;
  for (auto& s : slots_) {
    for (int i = 0; i < 2000 && s.done.load(std::memory_order_acquire) != epoch_; ++i) asm volatile("pause");
    while (s.done.load(std::memory_order_acquire) != epoch_) {
      const long left = deadline - sys_clock_monotonic_ns();
      if (left <= 0) {
        // Stragglers may still be running the job and reading its arguments, which usually live on the caller's
        // stack.  Give them a second bounded grace period; whatever happens the team is dead afterwards (later run()
        // calls fail fast) so that fn / arg are never rewritten under a worker that is still reading them.
        valid_ = false;
        const long grace_end = sys_clock_monotonic_ns() + kTimeoutGraceNs;
        bool all_done = false;
        while (!all_done && sys_clock_monotonic_ns() < grace_end) {
          all_done = true;
          for (auto& t : slots_)
            if (t.done.load(std::memory_order_acquire) != epoch_) { all_done = false; break; }
          if (!all_done) sys_futex_wait(&s.done, s.done.load(std::memory_order_acquire), kFutex, 10'000'000l);
        }
        stragglers_ = !all_done;
        return -err::kTIMEDOUT;
      }
      sys_futex_wait(&s.done, s.done.load(std::memory_order_acquire), kFutex, left < 100'000'000l ? left : 100'000'000l);
    }
  }
  return 0;
}

}  // namespace hostrt
