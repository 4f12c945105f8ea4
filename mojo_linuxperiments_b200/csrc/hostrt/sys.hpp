// Kernel ABI layer of the host runtime: a raw `syscall` instruction shim (no libc wrappers, no errno),
// the constants and structs of the Linux x86-64 ABI that the runtime uses, and one thin function per call.
// Every function returns the kernel's value: >= 0 on success, -errno on failure.
//
// Capability parity: threading/linux.mojo:9-332 of the reference (syscall numbers, clone flags, futex2
// flags, FutexNuma32 / FutexWaitv / Clone3Args / Rseq layouts, mmap / mbind / madvise / move_pages /
// mprotect / futex_wait / futex_waitv / futex_wake / exit / gettid / rseq / sched_setaffinity).
// Differences by design: futex waits take an optional timeout (the reference's are unbounded), and
// getcpu / nanosleep / clock_gettime are routed through the same shim.
#pragma once
#include <cstddef>
#include <cstdint>

#if !defined(__x86_64__) || !defined(__linux__)
#error "hostrt targets x86-64 Linux only"
#endif

namespace hostrt {

// ---------------------------------------------------------------------------------------------
// raw syscall, 0..6 arguments.  rcx and r11 are clobbered by the instruction; arg4 travels in r10.
// ---------------------------------------------------------------------------------------------
inline long raw_syscall(long nr) {
  long ret;
  asm volatile("syscall" : "=a"(ret) : "a"(nr) : "rcx", "r11", "memory");
  return ret;
}
inline long raw_syscall(long nr, long a0) {
  long ret;
  asm volatile("syscall" : "=a"(ret) : "a"(nr), "D"(a0) : "rcx", "r11", "memory");
  return ret;
}
inline long raw_syscall(long nr, long a0, long a1) {
  long ret;
  asm volatile("syscall" : "=a"(ret) : "a"(nr), "D"(a0), "S"(a1) : "rcx", "r11", "memory");
  return ret;
}
inline long raw_syscall(long nr, long a0, long a1, long a2) {
  long ret;
  asm volatile("syscall" : "=a"(ret) : "a"(nr), "D"(a0), "S"(a1), "d"(a2) : "rcx", "r11", "memory");
  return ret;
}
inline long raw_syscall(long nr, long a0, long a1, long a2, long a3) {
  long ret;
  register long r10 asm("r10") = a3;
  asm volatile("syscall" : "=a"(ret) : "a"(nr), "D"(a0), "S"(a1), "d"(a2), "r"(r10) : "rcx", "r11", "memory");
  return ret;
}
inline long raw_syscall(long nr, long a0, long a1, long a2, long a3, long a4) {
  long ret;
  register long r10 asm("r10") = a3;
  register long r8 asm("r8") = a4;
  asm volatile("syscall" : "=a"(ret) : "a"(nr), "D"(a0), "S"(a1), "d"(a2), "r"(r10), "r"(r8) : "rcx", "r11", "memory");
  return ret;
}
inline long raw_syscall(long nr, long a0, long a1, long a2, long a3, long a4, long a5) {
  long ret;
  register long r10 asm("r10") = a3;
  register long r8 asm("r8") = a4;
  register long r9 asm("r9") = a5;
  asm volatile("syscall"
               : "=a"(ret)
               : "a"(nr), "D"(a0), "S"(a1), "d"(a2), "r"(r10), "r"(r8), "r"(r9)
               : "rcx", "r11", "memory");
  return ret;
}

// ---------------------------------------------------------------------------------------------
// constants
// ---------------------------------------------------------------------------------------------
namespace nr {
constexpr long mmap = 9, mprotect = 10, munmap = 11, madvise = 28, nanosleep = 35, exit = 60, gettid = 186,
               sched_setaffinity = 203, sched_getaffinity = 204, clock_gettime = 228, mbind = 237,
               move_pages = 279, getcpu = 309, rseq = 334, clone3 = 435, futex_waitv = 449, futex_wake = 454,
               futex_wait = 455;
}

namespace clone_flag {
constexpr uint64_t VM = 0x00000100, FS = 0x00000200, FILES = 0x00000400, SIGHAND = 0x00000800,
                   PIDFD = 0x00001000, PTRACE = 0x00002000, VFORK = 0x00004000, PARENT = 0x00008000,
                   THREAD = 0x00010000, NEWNS = 0x00020000, SYSVSEM = 0x00040000, SETTLS = 0x00080000,
                   PARENT_SETTID = 0x00100000, CHILD_CLEARTID = 0x00200000, DETACHED = 0x00400000,
                   UNTRACED = 0x00800000, CHILD_SETTID = 0x01000000, NEWCGROUP = 0x02000000,
                   NEWUTS = 0x04000000, NEWIPC = 0x08000000, NEWUSER = 0x10000000, NEWPID = 0x20000000,
                   NEWNET = 0x40000000, IO = 0x80000000ull;
// A kernel thread that shares everything with its parent.  PARENT_SETTID publishes the tid in the slot
// before the parent returns; CHILD_CLEARTID makes the kernel clear a second word once the thread has left
// its stack for good, which is what slot reuse waits for.
constexpr uint64_t THREAD_FLAGS = VM | FS | FILES | SIGHAND | THREAD | SYSVSEM | SETTLS | PARENT_SETTID | CHILD_CLEARTID;
}  // namespace clone_flag

namespace futex2 {
constexpr uint32_t SIZE_U8 = 0x00, SIZE_U16 = 0x01, SIZE_U32 = 0x02, SIZE_U64 = 0x03, NUMA = 0x04, PRIVATE = 0x80;
constexpr int WAITV_MAX = 128;
}

namespace prot { constexpr long NONE = 0, READ = 1, WRITE = 2, EXEC = 4, RW = READ | WRITE; }
namespace map_flag {
constexpr long SHARED = 0x01, PRIVATE = 0x02, FIXED = 0x10, ANONYMOUS = 0x20, NORESERVE = 0x4000, POPULATE = 0x8000,
               HUGETLB = 0x40000, HUGE_2MB = 21l << 26, HUGE_1GB = 30l << 26;
}
namespace mempolicy { constexpr long DEFAULT = 0, PREFERRED = 1, BIND = 2, INTERLEAVE = 3, LOCAL = 4; constexpr long MF_STRICT = 1, MF_MOVE = 2; }
namespace madv { constexpr long NORMAL = 0, RANDOM = 1, SEQUENTIAL = 2, WILLNEED = 3, DONTNEED = 4, HUGEPAGE = 14, NOHUGEPAGE = 15; }
namespace page_size {
constexpr long STANDARD = 4096, THP_2MB = 2l << 20, GUARD = 4096;
constexpr long EXPLICIT_2MB = -2, EXPLICIT_1GB = -1;   // sentinels: ask for MAP_HUGETLB pages
}
namespace err { constexpr long kPERM = 1, kNOENT = 2, kINTR = 4, kAGAIN = 11, kNOMEM = 12, kFAULT = 14, kINVAL = 22, kNOSYS = 38, kTIMEDOUT = 110; }

// ---------------------------------------------------------------------------------------------
// ABI structs
// ---------------------------------------------------------------------------------------------
struct FutexNuma32 {          // a 32-bit futex word followed by the NUMA node hint the kernel reads with FUTEX2_NUMA
  uint32_t value;
  int32_t node;               // -1: let the kernel pick (it writes the node back)
};
static_assert(sizeof(FutexNuma32) == 8);

struct FutexWaitv {
  uint64_t val;
  uint64_t uaddr;
  uint32_t flags;
  uint32_t reserved;
};
static_assert(sizeof(FutexWaitv) == 24);

struct Clone3Args {
  uint64_t flags, pidfd, child_tid, parent_tid, exit_signal, stack, stack_size, tls, set_tid, set_tid_size, cgroup;
};
static_assert(sizeof(Clone3Args) == 88);

struct alignas(32) Rseq {
  uint32_t cpu_id_start;
  uint32_t cpu_id;
  uint64_t rseq_cs;
  uint32_t flags;
  uint32_t node_id;
  uint32_t mm_cid;
  uint32_t pad;
};
static_assert(sizeof(Rseq) == 32);
constexpr uint32_t RSEQ_SIG = 0x53053053u;

struct KTimespec { int64_t sec; int64_t nsec; };
constexpr int CLOCK_MONOTONIC_ID = 1;

// ---------------------------------------------------------------------------------------------
// wrappers
// ---------------------------------------------------------------------------------------------
inline long sys_mmap(void* addr, size_t len, long pr, long flags, long fd = -1, long off = 0) {
  return raw_syscall(nr::mmap, (long)addr, (long)len, pr, flags, fd, off);
}
inline long sys_munmap(void* addr, size_t len) { return raw_syscall(nr::munmap, (long)addr, (long)len); }
inline long sys_mprotect(void* addr, size_t len, long pr) { return raw_syscall(nr::mprotect, (long)addr, (long)len, pr); }
inline long sys_madvise(void* addr, size_t len, long advice) { return raw_syscall(nr::madvise, (long)addr, (long)len, advice); }
// nodemask is a bit array of `maxnode` bits (any number of 64-bit words)
inline long sys_mbind(void* addr, size_t len, long policy, const uint64_t* nodemask, unsigned long maxnode, long flags = 0) {
  return raw_syscall(nr::mbind, (long)addr, (long)len, policy, (long)nodemask, (long)maxnode, flags);
}
// Which NUMA node holds the page at addr?  >= 0 node, -ENOENT if the page was never touched.
inline long sys_move_pages_query(const void* addr) {
  void* pages[1] = {const_cast<void*>(addr)};
  int status[1] = {-1};
  long r = raw_syscall(nr::move_pages, 0, 1, (long)pages, 0 /*nodes = NULL: query*/, (long)status, 0);
  return r < 0 ? r : status[0];
}
inline long sys_clock_monotonic_ns() {
  KTimespec ts{0, 0};
  raw_syscall(nr::clock_gettime, CLOCK_MONOTONIC_ID, (long)&ts);
  return ts.sec * 1000000000l + ts.nsec;
}
// futex2 wait.  timeout_ns < 0 waits forever; otherwise the wait ends with -ETIMEDOUT after that long.
inline long sys_futex_wait(const void* addr, uint64_t expected, uint32_t flags, long timeout_ns = -1) {
  if (timeout_ns < 0) return raw_syscall(nr::futex_wait, (long)addr, (long)expected, 0xFFFFFFFFl, flags, 0, 0);
  const long t = sys_clock_monotonic_ns() + timeout_ns;      // futex2 timeouts are absolute
  KTimespec ts{t / 1000000000l, t % 1000000000l};
  return raw_syscall(nr::futex_wait, (long)addr, (long)expected, 0xFFFFFFFFl, flags, (long)&ts, CLOCK_MONOTONIC_ID);
}
inline long sys_futex_waitv(FutexWaitv* waiters, unsigned n, long timeout_ns = -1) {
  if (timeout_ns < 0) return raw_syscall(nr::futex_waitv, (long)waiters, n, 0, 0, 0);
  const long t = sys_clock_monotonic_ns() + timeout_ns;
  KTimespec ts{t / 1000000000l, t % 1000000000l};
  return raw_syscall(nr::futex_waitv, (long)waiters, n, 0, (long)&ts, CLOCK_MONOTONIC_ID);
}
inline long sys_futex_wake(const void* addr, int count, uint32_t flags) {
  return raw_syscall(nr::futex_wake, (long)addr, 0xFFFFFFFFl, count, flags);
}
[[noreturn]] inline void sys_exit_thread(int code = 0) {
  raw_syscall(nr::exit, code);
  __builtin_unreachable();
}
inline long sys_gettid() { return raw_syscall(nr::gettid); }
inline long sys_rseq(Rseq* area, uint32_t len, int flags, uint32_t sig) { return raw_syscall(nr::rseq, (long)area, len, flags, sig); }
inline long sys_sched_setaffinity(long tid, size_t mask_bytes, const void* mask) {
  return raw_syscall(nr::sched_setaffinity, tid, (long)mask_bytes, (long)mask);
}
inline long sys_sched_getaffinity(long tid, size_t mask_bytes, void* mask) {
  return raw_syscall(nr::sched_getaffinity, tid, (long)mask_bytes, (long)mask);
}
inline long sys_getcpu(unsigned* cpu, unsigned* node) { return raw_syscall(nr::getcpu, (long)cpu, (long)node, 0); }
inline long sys_nanosleep(long ns) {
  KTimespec ts{ns / 1000000000l, ns % 1000000000l};
  return raw_syscall(nr::nanosleep, (long)&ts, 0);
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace hostrt
