// Fixed-capacity pool of one-shot kernel threads created with clone3 (no pthread, no libc in the child's
// start-up path), joined through futex2 words, optionally pinned to a CPU set and bound to a NUMA node.
//
// Capability parity: threading/linux_threading.mojo:43-158,202-420 of the reference (ThreadPool, launch,
// wait_all, wait_any, slot arena with guard pages, per-slot FutexNuma32, rseq registration, MutexGate,
// set_thread_affinity, get_cpu_and_node_rseq).
//
// Deliberate differences:
//   * Slot reuse is race free.  The child still clears its tid word and wakes joiners itself (so the wake
//     can use PRIVATE / NUMA futex flags), but the slot also carries a second word that the kernel clears
//     (CLONE_CHILD_CLEARTID) only after the thread has left its stack; launch() reuses a slot only when
//     both words are zero.
//   * Every wait takes a timeout and reports -ETIMEDOUT instead of hanging.
//   * Stack size and mask size are run-time parameters (the C ABI needs that); PoolT<> fixes them at compile
//     time for C++ callers.
//
// Worker contract: a worker is `void f(u64 x 6)` (unused trailing arguments are ignored), runs on a small
// private stack with a private copy of the parent's first 256 bytes of static TLS, and must not call into
// libc facilities that need a real pthread (errno, malloc arenas, stdio, exceptions).
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <vector>

#include "cpumask.hpp"
#include "numa.hpp"
#include "sys.hpp"

namespace hostrt {

namespace stack_size { constexpr size_t DEFAULT = 64 * 1024, MIN = 2048; }

struct SlotLayout {
  static constexpr size_t TLS_COPY = 256;       // [0,256)    copy of the parent's static TLS tail
  static constexpr size_t TCB = 256;            // [256,320)  thread control block; the child's fs base
  static constexpr size_t TCB_SIZE = 64;
  static constexpr size_t TID = 320;            // [320,328)  FutexNuma32 {tid, node}: joiners wait here
  static constexpr size_t EXIT_WORD = 328;      // [328,332)  cleared by the kernel once the stack is dead
  static constexpr size_t MAGIC = 336;          // [336,344)  marks an fs base as belonging to a pool thread
  static constexpr size_t RSEQ = 352;           // [352,384)  struct rseq (fs + 96)
  static constexpr size_t HEADER = 4096;        // guard page follows the header page
  static constexpr size_t STACK = HEADER + 4096;
  static constexpr uint64_t MAGIC_VALUE = 0xB200'5107'7EAD'0001ull;
};

inline size_t slot_total_size(size_t stack_bytes) {
  return align_up(SlotLayout::STACK + stack_bytes, static_cast<size_t>(page_size::STANDARD));
}

using WorkerFn = void (*)(uint64_t, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t);

constexpr long WAIT_FOREVER = -1;
constexpr int WAIT_NOTHING_RUNNING = -1;
constexpr int WAIT_TIMED_OUT = -2;

class ThreadPool {
 public:
  // cpu_mask == nullptr or all-zero: threads are not pinned.  numa_node < 0: slot memory is not bound and
  // futexes carry no NUMA hint.
  ThreadPool(int capacity, const uint8_t* cpu_mask = nullptr, size_t mask_bytes = 0, int numa_node = -1,
             size_t stack_bytes = stack_size::DEFAULT);
  template <size_t B>
  ThreadPool(int capacity, const CpuMask<B>& mask, int numa_node = -1, size_t stack_bytes = stack_size::DEFAULT)
      : ThreadPool(capacity, mask.ptr(), B, numa_node, stack_bytes) {}
  ThreadPool(const ThreadPool&) = delete;
  ThreadPool& operator=(const ThreadPool&) = delete;
  ThreadPool(ThreadPool&& o) noexcept;
  ~ThreadPool();       // waits (bounded) for running threads; aborts the process if one never finishes

  static ThreadPool for_numa_node(const NumaInfo& info, int node, size_t stack_bytes = stack_size::DEFAULT);
  // one slot per CPU of the node except `exclude_cpu` (typically where the orchestrator is parked)
  static ThreadPool for_numa_node_excluding(const NumaInfo& info, int node, int exclude_cpu,
                                            size_t stack_bytes = stack_size::DEFAULT);

  explicit operator bool() const { return valid_; }
  int capacity() const { return capacity_; }
  int numa_node() const { return numa_node_; }
  bool pinned() const { return pinned_; }
  uint32_t futex_flags() const { return futex_flags_; }
  size_t slot_size() const { return slot_size_; }

  // Starts `fn(a0..a5)` on a free slot.  Returns the slot index, or -1 when every slot is busy / clone3 failed.
  int launch(WorkerFn fn, uint64_t a0 = 0, uint64_t a1 = 0, uint64_t a2 = 0, uint64_t a3 = 0, uint64_t a4 = 0,
             uint64_t a5 = 0);
  template <class... A>
  int launch_args(void* fn, A... a) {
    static_assert(sizeof...(A) <= 6, "at most six 8-byte arguments");
    static_assert(((sizeof(A) == 8) && ...), "every argument must be exactly 8 bytes");
    uint64_t v[6] = {0, 0, 0, 0, 0, 0};
    size_t i = 0;
    ((__builtin_memcpy(&v[i++], &a, 8)), ...);
    return launch(reinterpret_cast<WorkerFn>(fn), v[0], v[1], v[2], v[3], v[4], v[5]);
  }
  // 0 when every thread has finished and left its stack, -ETIMEDOUT otherwise.
  long wait_all(long timeout_ns = WAIT_FOREVER);
  // Index of a slot that finished, WAIT_NOTHING_RUNNING, or WAIT_TIMED_OUT.
  int wait_any(long timeout_ns = WAIT_FOREVER);
  bool slot_running(int i) const;
  int running_count() const;

 private:
  uint8_t* slot_base(int i) const { return arena_ + static_cast<size_t>(i) * slot_size_; }
  std::atomic<uint32_t>* tid_word(int i) const { return reinterpret_cast<std::atomic<uint32_t>*>(slot_base(i) + SlotLayout::TID); }
  std::atomic<uint32_t>* exit_word(int i) const { return reinterpret_cast<std::atomic<uint32_t>*>(slot_base(i) + SlotLayout::EXIT_WORD); }
  bool wait_retired(int i, long deadline_ns);
  void release();

  uint8_t* arena_ = nullptr;
  size_t arena_bytes_ = 0, slot_size_ = 0, stack_bytes_ = 0;
  int capacity_ = 0, numa_node_ = -1;
  bool pinned_ = false, valid_ = false;
  uint32_t futex_flags_ = futex2::SIZE_U32 | futex2::PRIVATE;
  std::vector<uint8_t> mask_;
};

template <size_t StackBytes = stack_size::DEFAULT, size_t MaskBytes = 128>
struct PoolT : ThreadPool {
  explicit PoolT(int capacity, const CpuMask<MaskBytes>& m = CpuMask<MaskBytes>(), int node = -1)
      : ThreadPool(capacity, m.ptr(), MaskBytes, node, StackBytes) {}
};

// Pin the calling thread.  Returns the kernel's result.
template <size_t B>
long set_thread_affinity(const CpuMask<B>& m) { return sys_sched_setaffinity(0, B, m.ptr()); }
long set_thread_affinity_raw(const uint8_t* mask, size_t bytes);

// (cpu, node) of the calling thread read from its registered rseq area: no syscall.  Works on pool workers
// (their area sits at a fixed offset from fs) and on libc threads (through libc's own registration);
// returns {-1,-1} when no area can be found.
CpuNode get_cpu_and_node_rseq();

// Single-use binary latch on a caller-supplied 32-bit word: wait() blocks until release() stored 1.
// The word must start at 0 (fresh anonymous memory is).  Passed to workers by value as one 8-byte argument.
struct MutexGate {
  std::atomic<uint32_t>* word;
  static MutexGate from_addr(void* p) { return MutexGate{static_cast<std::atomic<uint32_t>*>(p)}; }
  // 0 once released, -ETIMEDOUT when the bound ran out first
  long wait(long timeout_ns = WAIT_FOREVER) const;
  void release() const;
  void reset() const { word->store(0, std::memory_order_release); }
  uint64_t as_arg() const { return reinterpret_cast<uint64_t>(word); }
};
static_assert(sizeof(MutexGate) == 8);

}  // namespace hostrt
