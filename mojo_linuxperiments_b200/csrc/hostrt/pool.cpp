#include "pool.hpp"
#include "arena.hpp"

#include <climits>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace hostrt {

namespace {

struct StackHead {            // written by the parent at the 16-byte aligned top of the child's stack
  uint64_t entry;             // popped by the `ret` that follows clone3 in the child
  uint64_t slot_base;
  uint64_t user_func;
  uint64_t cpu_mask_ptr;
  uint64_t cpu_mask_size;
  uint64_t futex_flags;
  uint64_t args[6];
  uint64_t pad;
};
static_assert(sizeof(StackHead) == 104);

inline uint64_t read_fs_base() {
  uint64_t v;
  asm volatile("mov %%fs:0, %0" : "=r"(v));    // the TCB's first word points at itself
  return v;
}

// Runs on the new thread, entered by `ret` with rdi = &StackHead and a correctly aligned stack.
extern "C" __attribute__((noreturn, used, noinline)) void hostrt_child_main(StackHead* remote) {
  StackHead h = *remote;      // private copy: from here on nothing reads the parent-written head again
  uint8_t* slot = reinterpret_cast<uint8_t*>(h.slot_base);
  // rseq must be registered before the affinity call so cpu_id/node_id are valid right after migration
  sys_rseq(reinterpret_cast<Rseq*>(slot + SlotLayout::RSEQ), sizeof(Rseq), 0, RSEQ_SIG);
  if (h.cpu_mask_ptr && h.cpu_mask_size)
    sys_sched_setaffinity(sys_gettid(), h.cpu_mask_size, reinterpret_cast<const void*>(h.cpu_mask_ptr));
  reinterpret_cast<WorkerFn>(h.user_func)(h.args[0], h.args[1], h.args[2], h.args[3], h.args[4], h.args[5]);
  auto* tid = reinterpret_cast<std::atomic<uint32_t>*>(slot + SlotLayout::TID);
  const uint32_t flags = static_cast<uint32_t>(h.futex_flags);
  tid->store(0, std::memory_order_release);           // "work done": joiners may proceed
  sys_futex_wake(tid, INT_MAX, flags);
  sys_exit_thread(0);                                  // kernel clears EXIT_WORD after the stack is dead
}

long clone3_with_entry(Clone3Args* args, size_t size) {
  long ret;
  asm volatile(
      "mov $435, %%eax\n\t"
      "syscall\n\t"
      "test %%rax, %%rax\n\t"
      "jnz 1f\n\t"
      "mov %%rsp, %%rdi\n\t"     // child: rsp points at StackHead.entry
      "xor %%ebp, %%ebp\n\t"
      "ret\n\t"
      "1:\n\t"
      : "=a"(ret)
      : "D"(args), "S"(size)
      : "rcx", "r11", "memory");
  return ret;
}

bool mask_any(const uint8_t* m, size_t n) {
  for (size_t i = 0; i < n; ++i) if (m[i]) return true;
  return false;
}

}  // namespace

ThreadPool::ThreadPool(int capacity, const uint8_t* cpu_mask, size_t mask_bytes, int numa_node, size_t stack_bytes)
    : stack_bytes_(stack_bytes < stack_size::MIN ? stack_size::MIN : stack_bytes), capacity_(capacity), numa_node_(numa_node) {
  if (capacity <= 0) return;
  if (cpu_mask && mask_bytes) {
    mask_.assign(cpu_mask, cpu_mask + mask_bytes);
    mask_.resize(align_up(mask_bytes, 8), 0);
    pinned_ = mask_any(mask_.data(), mask_.size());
  }
  slot_size_ = slot_total_size(stack_bytes_);
  arena_bytes_ = slot_size_ * static_cast<size_t>(capacity);
  void* p = mmap_numa(arena_bytes_, numa_node, page_size::STANDARD);
  if (!p) { capacity_ = 0; return; }
  arena_ = static_cast<uint8_t*>(p);
  if (numa_node >= 0) futex_flags_ |= futex2::NUMA;
  for (int i = 0; i < capacity; ++i) {
    uint8_t* s = slot_base(i);
    if (sys_mprotect(s + SlotLayout::HEADER, page_size::GUARD, prot::NONE) < 0) { release(); capacity_ = 0; return; }
    auto* f = reinterpret_cast<FutexNuma32*>(s + SlotLayout::TID);
    f->value = 0;
    f->node = numa_node >= 0 ? numa_node : -1;
    *reinterpret_cast<uint32_t*>(s + SlotLayout::EXIT_WORD) = 0;
    *reinterpret_cast<uint64_t*>(s + SlotLayout::MAGIC) = SlotLayout::MAGIC_VALUE;
  }
  if (futex_flags_ & futex2::NUMA) {
    // kernels without FUTEX2_NUMA reject the flag: fall back to plain private futexes
    if (sys_futex_wake(slot_base(0) + SlotLayout::TID, 1, futex_flags_) == -err::kINVAL) futex_flags_ &= ~futex2::NUMA;
  }
  valid_ = true;
}

ThreadPool::ThreadPool(ThreadPool&& o) noexcept
    : arena_(o.arena_), arena_bytes_(o.arena_bytes_), slot_size_(o.slot_size_), stack_bytes_(o.stack_bytes_),
      capacity_(o.capacity_), numa_node_(o.numa_node_), pinned_(o.pinned_), valid_(o.valid_),
      futex_flags_(o.futex_flags_), mask_(std::move(o.mask_)) {
  // threads already running keep a pointer to the mask bytes: the vector's heap buffer moves with it
  o.arena_ = nullptr; o.valid_ = false; o.capacity_ = 0;
}

void ThreadPool::release() {
  if (arena_) sys_munmap(arena_, arena_bytes_);
  arena_ = nullptr;
  valid_ = false;
}

ThreadPool::~ThreadPool() {
  if (!arena_) return;
  if (wait_all(10'000'000'000l) != 0) {
    std::fprintf(stderr, "hostrt: ThreadPool destroyed while a worker is still running; its stack cannot be unmapped\n");
    std::abort();
  }
  release();
}

ThreadPool ThreadPool::for_numa_node(const NumaInfo& info, int node, size_t stack_bytes) {
  auto m = info.get_node_mask<128>(node);
  return ThreadPool(info.cpus_on_node(node), m.ptr(), 128, node, stack_bytes);
}
ThreadPool ThreadPool::for_numa_node_excluding(const NumaInfo& info, int node, int exclude_cpu, size_t stack_bytes) {
  auto m = info.get_node_mask<128>(node);
  int n = info.cpus_on_node(node);
  if (m.test(exclude_cpu)) { m.clear(exclude_cpu); --n; }
  return ThreadPool(n, m.ptr(), 128, node, stack_bytes);
}

bool ThreadPool::slot_running(int i) const {
  return i >= 0 && i < capacity_ && tid_word(i)->load(std::memory_order_acquire) != 0;
}
int ThreadPool::running_count() const {
  int c = 0;
  for (int i = 0; i < capacity_; ++i) c += slot_running(i) ? 1 : 0;
  return c;
}

bool ThreadPool::wait_retired(int i, long deadline_ns) {
  auto* w = exit_word(i);
  while (true) {
    const uint32_t v = w->load(std::memory_order_acquire);
    if (v == 0) return true;
    long left = -1;
    if (deadline_ns >= 0) {
      left = deadline_ns - sys_clock_monotonic_ns();
      if (left <= 0) return false;
    }
    // the kernel's clear-tid wake is a shared 32-bit futex wake
    sys_futex_wait(w, v, futex2::SIZE_U32, left);
  }
}

int ThreadPool::launch(WorkerFn fn, uint64_t a0, uint64_t a1, uint64_t a2, uint64_t a3, uint64_t a4, uint64_t a5) {
  if (!valid_ || !fn) return -1;
  int slot = -1, finishing = -1;
  for (int i = 0; i < capacity_; ++i) {
    if (tid_word(i)->load(std::memory_order_acquire) != 0) continue;
    if (exit_word(i)->load(std::memory_order_acquire) == 0) { slot = i; break; }
    if (finishing < 0) finishing = i;
  }
  if (slot < 0) {
    // a worker announced completion but is still in its last instructions: give it a moment to leave
    if (finishing < 0) return -1;
    if (!wait_retired(finishing, sys_clock_monotonic_ns() + 100'000'000l)) return -1;
    slot = finishing;
  }
  uint8_t* s = slot_base(slot);
  // thread-local storage for the child: the tail of our own static TLS block and a TCB that points at itself
  const uint64_t parent_fs = read_fs_base();
  std::memcpy(s, reinterpret_cast<const void*>(parent_fs - SlotLayout::TLS_COPY), SlotLayout::TLS_COPY);
  std::memcpy(s + SlotLayout::TCB, reinterpret_cast<const void*>(parent_fs), SlotLayout::TCB_SIZE);
  const uint64_t child_fs = reinterpret_cast<uint64_t>(s + SlotLayout::TCB);
  *reinterpret_cast<uint64_t*>(s + SlotLayout::TCB + 0x00) = child_fs;
  *reinterpret_cast<uint64_t*>(s + SlotLayout::TCB + 0x10) = child_fs;
  std::memset(s + SlotLayout::RSEQ, 0, sizeof(Rseq));
  reinterpret_cast<Rseq*>(s + SlotLayout::RSEQ)->cpu_id = 0xFFFFFFFFu;   // RSEQ_CPU_ID_UNINITIALIZED

  uint8_t* stack_lo = s + SlotLayout::STACK;
  const uint64_t head_addr = (reinterpret_cast<uint64_t>(stack_lo) + stack_bytes_ - sizeof(StackHead)) & ~uint64_t(15);
  auto* head = reinterpret_cast<StackHead*>(head_addr);
  head->entry = reinterpret_cast<uint64_t>(&hostrt_child_main);
  head->slot_base = reinterpret_cast<uint64_t>(s);
  head->user_func = reinterpret_cast<uint64_t>(fn);
  head->cpu_mask_ptr = pinned_ ? reinterpret_cast<uint64_t>(mask_.data()) : 0;
  head->cpu_mask_size = pinned_ ? mask_.size() : 0;
  head->futex_flags = futex_flags_;
  head->args[0] = a0; head->args[1] = a1; head->args[2] = a2; head->args[3] = a3; head->args[4] = a4; head->args[5] = a5;
  head->pad = 0;

  exit_word(slot)->store(1, std::memory_order_release);     // "stack in use" until the kernel clears it
  Clone3Args ca{};
  ca.flags = clone_flag::THREAD_FLAGS;
  ca.child_tid = reinterpret_cast<uint64_t>(exit_word(slot));
  ca.parent_tid = reinterpret_cast<uint64_t>(tid_word(slot));
  ca.stack = reinterpret_cast<uint64_t>(stack_lo);
  ca.stack_size = head_addr - reinterpret_cast<uint64_t>(stack_lo);
  ca.tls = child_fs;
  const long r = clone3_with_entry(&ca, sizeof(ca));
  if (r < 0) {
    exit_word(slot)->store(0, std::memory_order_release);
    tid_word(slot)->store(0, std::memory_order_release);
    return -1;
  }
  return slot;
}

long ThreadPool::wait_all(long timeout_ns) {
  if (!arena_) return 0;
  const long deadline = timeout_ns < 0 ? -1 : sys_clock_monotonic_ns() + timeout_ns;
  for (int i = 0; i < capacity_; ++i) {
    auto* w = tid_word(i);
    while (true) {
      const uint32_t tid = w->load(std::memory_order_acquire);
      if (tid == 0) break;
      long left = -1;
      if (deadline >= 0) {
        left = deadline - sys_clock_monotonic_ns();
        if (left <= 0) return -err::kTIMEDOUT;
      }
      sys_futex_wait(w, tid, futex_flags_, left);
    }
    if (!wait_retired(i, deadline)) return -err::kTIMEDOUT;
  }
  return 0;
}

int ThreadPool::wait_any(long timeout_ns) {
  if (!arena_) return WAIT_NOTHING_RUNNING;
  const long deadline = timeout_ns < 0 ? -1 : sys_clock_monotonic_ns() + timeout_ns;
  FutexWaitv waiters[futex2::WAITV_MAX];
  int slots[futex2::WAITV_MAX];
  // snapshot of what is running now: one of exactly these slots is reported
  int n = 0;
  for (int i = 0; i < capacity_ && n < futex2::WAITV_MAX; ++i) {
    const uint32_t tid = tid_word(i)->load(std::memory_order_acquire);
    if (tid == 0) continue;
    waiters[n] = FutexWaitv{tid, reinterpret_cast<uint64_t>(tid_word(i)), futex_flags_, 0};
    slots[n++] = i;
  }
  if (n == 0) return WAIT_NOTHING_RUNNING;
  while (true) {
    for (int k = 0; k < n; ++k)
      if (tid_word(slots[k])->load(std::memory_order_acquire) == 0) return slots[k];
    long left = -1;
    if (deadline >= 0) {
      left = deadline - sys_clock_monotonic_ns();
      if (left <= 0) return WAIT_TIMED_OUT;
    }
    const long r = sys_futex_waitv(waiters, static_cast<unsigned>(n), left);
    if (r >= 0 && r < n && tid_word(slots[r])->load(std::memory_order_acquire) == 0) return slots[r];
    // -EAGAIN (a word changed before we slept), -EINTR, spurious wake or timeout: rescan
  }
}

long set_thread_affinity_raw(const uint8_t* mask, size_t bytes) { return sys_sched_setaffinity(0, bytes, mask); }

extern "C" {
// exported by glibc >= 2.35: where libc registered this thread's rseq area, relative to the thread pointer
extern const ptrdiff_t __rseq_offset __attribute__((weak));
extern const unsigned int __rseq_size __attribute__((weak));
}

CpuNode get_cpu_and_node_rseq() {
  const uint64_t fs = read_fs_base();
  const uint8_t* tcb = reinterpret_cast<const uint8_t*>(fs);
  // pool worker: fs = slot + TCB, and the slot header carries a magic word
  const uint64_t* magic = reinterpret_cast<const uint64_t*>(tcb - SlotLayout::TCB + SlotLayout::MAGIC);
  const Rseq* area = nullptr;
  // The magic word of a pool slot sits 80 bytes above fs; on a libc thread that address is inside struct
  // pthread and readable, so the probe itself is safe either way.
  if (*magic == SlotLayout::MAGIC_VALUE) area = reinterpret_cast<const Rseq*>(tcb - SlotLayout::TCB + SlotLayout::RSEQ);
  else if (&__rseq_offset && &__rseq_size && __rseq_size >= 20) area = reinterpret_cast<const Rseq*>(tcb + __rseq_offset);
  if (!area) return {-1, -1};
  const uint32_t cpu = reinterpret_cast<const volatile Rseq*>(area)->cpu_id;
  const uint32_t node = reinterpret_cast<const volatile Rseq*>(area)->node_id;
  if (cpu == 0xFFFFFFFFu || cpu == 0xFFFFFFFEu) return {-1, -1};
  return {static_cast<int>(cpu), static_cast<int>(node)};
}

long MutexGate::wait(long timeout_ns) const {
  const long deadline = timeout_ns < 0 ? -1 : sys_clock_monotonic_ns() + timeout_ns;
  while (word->load(std::memory_order_acquire) == 0) {
    long left = -1;
    if (deadline >= 0) {
      left = deadline - sys_clock_monotonic_ns();
      if (left <= 0) return -err::kTIMEDOUT;
    }
    sys_futex_wait(word, 0, futex2::SIZE_U32 | futex2::PRIVATE, left);
  }
  return 0;
}
void MutexGate::release() const {
  word->store(1, std::memory_order_release);
  sys_futex_wake(word, INT_MAX, futex2::SIZE_U32 | futex2::PRIVATE);
}

}  // namespace hostrt
