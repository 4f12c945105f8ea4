// The reference's twelve integration behaviours (test_linux_threading.mojo:24-553), restated against this
// runtime.  Each scenario returns SC_PASS / SC_FAIL / SC_SKIP and a one-line detail; nothing here mocks the
// kernel.  Unlike the reference, a failure is a failure (callers turn it into an exit code) and a scenario
// that cannot run on this machine reports SKIP, not PASS.
#include "scenarios.hpp"

#include <atomic>
#include <cstdio>
#include <vector>

#include "arena.hpp"
#include "collectives.hpp"
#include "heap_move_array.hpp"
#include "pool.hpp"

namespace hostrt {

namespace {

constexpr long T10S = 10'000'000'000l;

#define DETAIL(...) std::snprintf(detail, n, __VA_ARGS__)

// ---- workers (raw syscalls and plain memory only) ----------------------------------------------------
void w_mul3(uint64_t a, uint64_t b, uint64_t out, uint64_t, uint64_t, uint64_t) {
  *reinterpret_cast<volatile int64_t*>(out) = static_cast<int64_t>(a * b);
}
void w_square2(uint64_t i, uint64_t out, uint64_t, uint64_t, uint64_t, uint64_t) {
  reinterpret_cast<volatile int64_t*>(out)[i] = static_cast<int64_t>(i * i * 2);
}
void w_count(uint64_t counter, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t) {
  reinterpret_cast<std::atomic<int64_t>*>(counter)->fetch_add(1);
}
void w_sleep_ms(uint64_t ms, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t) { sys_nanosleep(static_cast<long>(ms) * 1'000'000l); }
void w_check_node(uint64_t expect_node, uint64_t errors, uint64_t done, uint64_t, uint64_t, uint64_t) {
  if (get_current_cpu_and_node().node != static_cast<int>(expect_node)) reinterpret_cast<std::atomic<int64_t>*>(errors)->fetch_add(1);
  reinterpret_cast<std::atomic<int64_t>*>(done)->fetch_add(1);
}
void w_rseq_vs_getcpu(uint64_t errors, uint64_t done, uint64_t, uint64_t, uint64_t, uint64_t) {
  // the pool pins this worker to exactly one CPU, so both readings must agree
  const CpuNode a = get_cpu_and_node_rseq();
  const CpuNode b = get_current_cpu_and_node();
  if (a.cpu != b.cpu || a.node != b.node) reinterpret_cast<std::atomic<int64_t>*>(errors)->fetch_add(1);
  reinterpret_cast<std::atomic<int64_t>*>(done)->fetch_add(1);
}
// writes slot*1000 + expected_node*10 + node_of_the_memory it wrote to (9 when the query fails)
void w_arena_tag(uint64_t slot, uint64_t expect_node, uint64_t dst, uint64_t, uint64_t, uint64_t) {
  auto* p = reinterpret_cast<volatile int64_t*>(dst);
  *p = -1;                                   // first touch
  const long mem_node = sys_move_pages_query(reinterpret_cast<const void*>(dst));
  *p = static_cast<int64_t>(slot * 1000 + expect_node * 10 + (mem_node >= 0 && mem_node < 9 ? mem_node : 9));
}
// node-local variant: also reports where the thread itself runs: slot*1000 + thread_node*100 + expected*10 + mem_node
void w_arena_local(uint64_t slot, uint64_t expect_node, uint64_t dst, uint64_t, uint64_t, uint64_t) {
  auto* p = reinterpret_cast<volatile int64_t*>(dst);
  *p = -1;
  const long mem_node = sys_move_pages_query(reinterpret_cast<const void*>(dst));
  const int tn = get_current_cpu_and_node().node;
  *p = static_cast<int64_t>(slot * 1000 + (tn >= 0 && tn < 9 ? tn : 9) * 100 + expect_node * 10 + (mem_node >= 0 && mem_node < 9 ? mem_node : 9));
}

int first_cpu(const NumaInfo& info) {
  return info.num_nodes() && !info.nodes()[0].cpu_ids.empty() ? info.nodes()[0].cpu_ids[0] : 0;
}

// ---- scenarios -----------------------------------------------------------------------------------------
int sc_thread_constructor(char* detail, size_t n) {
  const size_t stacks[4] = {4096, 8192, 12288, stack_size::DEFAULT};
  for (int i = 0; i < 4; ++i) {
    ThreadPool pool(1, nullptr, 0, -1, stacks[i]);
    if (!pool) { DETAIL("pool %d invalid", i); return SC_FAIL; }
    volatile int64_t out = 0;
    if (pool.launch(&w_mul3, 6 + i, 7, reinterpret_cast<uint64_t>(&out)) < 0) { DETAIL("launch %d failed", i); return SC_FAIL; }
    if (pool.wait_all(T10S) != 0) { DETAIL("join %d timed out", i); return SC_FAIL; }
    if (out != (6 + i) * 7) { DETAIL("pool %d wrote %ld", i, static_cast<long>(out)); return SC_FAIL; }
  }
  DETAIL("4 single-slot pools, stacks 4K/8K/12K/64K");
  return SC_PASS;
}

int sc_thread_pool(char* detail, size_t n) {
  constexpr int N = 32;
  ThreadPool pool(N, nullptr, 0, -1, 2048);
  if (!pool) { DETAIL("pool invalid"); return SC_FAIL; }
  std::vector<int64_t> out(N, -1);
  for (int batch = 0; batch < 2; ++batch) {
    for (int i = 0; i < N; ++i) out[i] = -1;
    for (int i = 0; i < N; ++i)
      if (pool.launch(&w_square2, i, reinterpret_cast<uint64_t>(out.data())) < 0) { DETAIL("launch %d/%d failed", batch, i); return SC_FAIL; }
    if (pool.wait_all(T10S) != 0) { DETAIL("join timed out"); return SC_FAIL; }
    for (int i = 0; i < N; ++i) if (out[i] != static_cast<int64_t>(i) * i * 2) { DETAIL("batch %d slot %d -> %ld", batch, i, static_cast<long>(out[i])); return SC_FAIL; }
  }
  DETAIL("32 slots x 2 KiB stacks x 2 batches");
  return SC_PASS;
}

int sc_pool_reuse(char* detail, size_t n) {
  ThreadPool pool(2);
  std::atomic<int64_t> counter{0};
  for (int batch = 0; batch < 2; ++batch) {
    for (int i = 0; i < 2; ++i) if (pool.launch(&w_count, reinterpret_cast<uint64_t>(&counter)) < 0) { DETAIL("launch failed"); return SC_FAIL; }
    if (pool.launch(&w_count, reinterpret_cast<uint64_t>(&counter)) >= 0) {      // a third launch must be refused or reuse a retired slot
      // allowed only if a worker had already finished; then the count below is 3 for this batch
      counter.fetch_sub(1);
    }
    if (pool.wait_all(T10S) != 0) { DETAIL("join timed out"); return SC_FAIL; }
  }
  if (counter.load() != 4) { DETAIL("counter %ld != 4", static_cast<long>(counter.load())); return SC_FAIL; }
  DETAIL("2 slots x 2 batches, counter 4");
  return SC_PASS;
}

int wait_any_order(ThreadPool& pool, char* detail, size_t n) {
  const int ms[4] = {200, 150, 100, 50};
  int slot_of[4];
  for (int i = 0; i < 4; ++i) { slot_of[i] = pool.launch(&w_sleep_ms, ms[i]); if (slot_of[i] < 0) { DETAIL("launch failed"); return SC_FAIL; } }
  int order[4];
  for (int k = 0; k < 4; ++k) {
    order[k] = pool.wait_any(T10S);
    if (order[k] < 0) { DETAIL("wait_any returned %d at %d", order[k], k); return SC_FAIL; }
  }
  if (pool.wait_any(T10S) != WAIT_NOTHING_RUNNING) { DETAIL("wait_any on idle pool did not report idle"); return SC_FAIL; }
  for (int k = 0; k < 4; ++k) if (order[k] != slot_of[3 - k]) { DETAIL("order [%d,%d,%d,%d]", order[0], order[1], order[2], order[3]); return SC_FAIL; }
  pool.wait_all(T10S);
  DETAIL("completion order [%d,%d,%d,%d]", order[0], order[1], order[2], order[3]);
  return SC_PASS;
}
int sc_wait_any(char* detail, size_t n) { ThreadPool pool(4); return wait_any_order(pool, detail, n); }
int sc_wait_any_numa(char* detail, size_t n) {
  NumaInfo info;
  if (!info.ok()) { DETAIL("no NUMA sysfs"); return SC_SKIP; }
  const int node = info.nodes()[0].id;
  auto m = info.get_node_mask<128>(node);
  ThreadPool pool(4, m.ptr(), 128, node);
  if (!pool) { DETAIL("pool invalid"); return SC_FAIL; }
  const int r = wait_any_order(pool, detail, n);
  if (r == SC_PASS) { char tmp[160]; std::snprintf(tmp, sizeof tmp, "%s; futex flags 0x%x", detail, pool.futex_flags()); DETAIL("%s", tmp); }
  return r;
}

int sc_wait_any_reuse(char* detail, size_t n) {
  ThreadPool pool(4, nullptr, 0, -1, 8192);
  std::atomic<int64_t> done{0};
  long launched = 0;
  for (int iter = 0; iter < 1000; ++iter) {
    for (int i = 0; i < 4; ++i) {
      if (pool.launch(&w_count, reinterpret_cast<uint64_t>(&done)) < 0) { DETAIL("iteration %d: launch %d refused (slot leak)", iter, i); return SC_FAIL; }
      ++launched;
    }
    const int s = pool.wait_any(T10S);        // -1 is fine: everything may have finished before we looked
    if (s == WAIT_TIMED_OUT) { DETAIL("wait_any timed out"); return SC_FAIL; }
    if (pool.wait_all(T10S) != 0) { DETAIL("wait_all timed out"); return SC_FAIL; }
  }
  if (done.load() != launched) { DETAIL("launched %ld completed %ld", launched, static_cast<long>(done.load())); return SC_FAIL; }
  DETAIL("1000 x 4 spawns, %ld completed, no slot leak", launched);
  return SC_PASS;
}

int sc_numa_pinning(char* detail, size_t n) {
  NumaInfo info;
  if (!info.ok()) { DETAIL("no NUMA sysfs"); return SC_SKIP; }
  const int park = first_cpu(info);
  CpuMask<128> saved;
  sys_sched_getaffinity(0, 128, saved.ptr());
  set_thread_affinity(CpuMask<128>::from_cpu_list({park}));
  std::atomic<int64_t> errors{0}, done{0};
  long expected = 0;
  int rc = SC_PASS;
  {
    HeapMoveArray<ThreadPool> pools(info.num_nodes());
    for (const auto& nd : info.nodes()) {
      pools.push(ThreadPool::for_numa_node_excluding(info, nd.id, park));
      ThreadPool& p = pools[pools.size() - 1];
      if (p.capacity() == 0) continue;
      if (!p) { DETAIL("pool for node %d invalid", nd.id); rc = SC_FAIL; break; }
      for (int i = 0; i < p.capacity(); ++i) {
        if (p.launch(&w_check_node, nd.id, reinterpret_cast<uint64_t>(&errors), reinterpret_cast<uint64_t>(&done)) < 0) { rc = SC_FAIL; break; }
        ++expected;
      }
    }
    for (auto& p : pools) if (p.wait_all(T10S) != 0) rc = SC_FAIL;
  }
  sys_sched_setaffinity(0, 128, saved.ptr());
  if (rc != SC_PASS) { if (!detail[0]) DETAIL("launch or join failed"); return rc; }
  if (errors.load() != 0 || done.load() != expected) { DETAIL("%ld workers, %ld on the wrong node", expected, static_cast<long>(errors.load())); return SC_FAIL; }
  DETAIL("%ld workers on %d node(s), orchestrator parked on cpu %d", expected, info.num_nodes(), park);
  return SC_PASS;
}

int sc_rseq_api(char* detail, size_t n) {
  NumaInfo info;
  if (!info.ok()) { DETAIL("no NUMA sysfs"); return SC_SKIP; }
  std::atomic<int64_t> errors{0}, done{0};
  long expected = 0;
  for (const auto& nd : info.nodes()) {
    for (int cpu : nd.cpu_ids) {
      auto m = CpuMask<128>::from_cpu_list({cpu});
      ThreadPool pool(1, m.ptr(), 128, nd.id);
      if (!pool || pool.launch(&w_rseq_vs_getcpu, reinterpret_cast<uint64_t>(&errors), reinterpret_cast<uint64_t>(&done)) < 0) { DETAIL("cpu %d: launch failed", cpu); return SC_FAIL; }
      if (pool.wait_all(T10S) != 0) { DETAIL("join timed out"); return SC_FAIL; }
      ++expected;
    }
  }
  const CpuNode self = get_cpu_and_node_rseq();      // libc thread path
  if (errors.load() != 0 || done.load() != expected) { DETAIL("%ld mismatches over %ld cpus", static_cast<long>(errors.load()), expected); return SC_FAIL; }
  DETAIL("rseq == getcpu on %ld cpus; caller reads cpu %d node %d", expected, self.cpu, self.node);
  return SC_PASS;
}

int sc_numa_arena_buffer(char* detail, size_t n) {
  NumaInfo info;
  if (!info.ok()) { DETAIL("no NUMA sysfs"); return SC_SKIP; }
  const int home = info.nodes()[0].id;
  NumaArena arena(home, 4096, 8, page_size::STANDARD);
  if (!arena) { DETAIL("arena invalid"); return SC_FAIL; }
  int workers = info.total_cpus() < 32 ? info.total_cpus() : 32;
  auto* buf = arena.alloc<int64_t>(workers);
  if (!buf) { DETAIL("alloc failed"); return SC_FAIL; }
  if (arena.alloc<int64_t>(4096) != nullptr) { DETAIL("over-allocation was not refused"); return SC_FAIL; }
  HeapMoveArray<ThreadPool> pools(info.num_nodes());
  for (const auto& nd : info.nodes()) pools.push(ThreadPool::for_numa_node(info, nd.id));
  std::vector<int> expect(workers);
  for (int i = 0; i < workers; ++i) {
    const int k = i % info.num_nodes();
    expect[i] = home;
    if (pools[k].launch(&w_arena_tag, i, home, reinterpret_cast<uint64_t>(&buf[i])) < 0) { DETAIL("launch %d failed", i); return SC_FAIL; }
  }
  for (auto& p : pools) if (p.wait_all(T10S) != 0) { DETAIL("join timed out"); return SC_FAIL; }
  for (int i = 0; i < workers; ++i) {
    const int64_t v = buf[i];
    if (v / 1000 != i || (v / 10) % 100 != home || v % 10 != home) { DETAIL("slot %d tag %ld", i, static_cast<long>(v)); return SC_FAIL; }
  }
  if (!arena.verify_placement()) { DETAIL("first page is not on node %d", home); return SC_FAIL; }
  DETAIL("%d workers wrote one node-%d arena; placement verified", workers, home);
  return SC_PASS;
}

int sc_numa_arena_scatter(char* detail, size_t n) {
  NumaInfo info;
  if (!info.ok()) { DETAIL("no NUMA sysfs"); return SC_SKIP; }
  const int park = first_cpu(info);
  CpuMask<128> saved;
  sys_sched_getaffinity(0, 128, saved.ptr());
  set_thread_affinity(CpuMask<128>::from_cpu_list({park}));
  int rc = SC_PASS;
  long checked = 0;
  {
    const int nn = info.num_nodes();
    HeapMoveArray<NumaArena> arenas(nn);
    HeapMoveArray<ThreadPool> pools(nn);
    for (const auto& nd : info.nodes()) {
      arenas.emplace(nd.id, size_t(1) << 20, size_t(64), page_size::STANDARD);
      pools.push(ThreadPool::for_numa_node_excluding(info, nd.id, park));
    }
    for (int iter = 0; iter < 2 && rc == SC_PASS; ++iter) {
      std::vector<std::vector<int64_t*>> bufs(nn);
      for (int k = 0; k < nn; ++k) {
        arenas[k].reset();
        const int node = info.nodes()[k].id;
        for (int i = 0; i < pools[k].capacity(); ++i) {
          // one page per worker so move_pages reports this worker's own first touch
          auto* b = static_cast<int64_t*>(arenas[k].alloc_bytes(4096));
          bufs[k].push_back(b);
          if (!b || pools[k].launch(&w_arena_local, i, node, reinterpret_cast<uint64_t>(b)) < 0) { DETAIL("launch failed"); rc = SC_FAIL; }
        }
      }
      for (auto& p : pools) if (p.wait_all(T10S) != 0) rc = SC_FAIL;
      for (int k = 0; k < nn && rc == SC_PASS; ++k) {
        const int node = info.nodes()[k].id;
        for (size_t i = 0; i < bufs[k].size(); ++i) {
          const int64_t v = *bufs[k][i];
          const bool ok = v / 1000 == static_cast<int64_t>(i) && (v / 100) % 10 == node && (v / 10) % 10 == node && v % 10 == node;
          if (!ok) { DETAIL("iter %d node %d slot %zu tag %ld", iter, node, i, static_cast<long>(v)); rc = SC_FAIL; break; }
          ++checked;
        }
        if (rc == SC_PASS && !arenas[k].verify_placement()) { DETAIL("arena of node %d misplaced", node); rc = SC_FAIL; }
      }
    }
  }
  sys_sched_setaffinity(0, 128, saved.ptr());
  if (rc == SC_PASS) DETAIL("%ld node-local writes: thread node == memory node == expected, 2 iterations", checked);
  return rc;
}

int sc_ring_reduce(char* detail, size_t n) {
  NumaInfo info;
  if (!info.ok()) { DETAIL("no NUMA sysfs"); return SC_SKIP; }
  // one rank per node when there are several nodes; otherwise four ranks share the only node
  const int world = info.num_nodes() >= 2 ? info.num_nodes() : 4;
  const CollectiveResult r = chain_reduce(info, world, T10S);
  const int64_t want = static_cast<int64_t>(world) * (world + 1) / 2;
  if (r.status != 0 || r.value != want) { DETAIL("status %ld value %ld want %ld", r.status, static_cast<long>(r.value), static_cast<long>(want)); return SC_FAIL; }
  DETAIL("%d ranks over %d node(s): rank 0 holds %ld", world, info.num_nodes(), static_cast<long>(want));
  return SC_PASS;
}

int sc_all_reduce(char* detail, size_t n) {
  NumaInfo info;
  if (!info.ok()) { DETAIL("no NUMA sysfs"); return SC_SKIP; }
  int world = info.num_nodes() >= 2 ? info.num_nodes() : 4;
  while (world & (world - 1)) world &= world - 1;          // largest power of two not above the node count
  std::vector<int64_t> out(world, 0);
  const long st = butterfly_allreduce(info, world, out.data(), T10S);
  const int64_t want = static_cast<int64_t>(world) * (world + 1) / 2;
  if (st != 0) { DETAIL("status %ld", st); return SC_FAIL; }
  for (int r = 0; r < world; ++r) if (out[r] != want) { DETAIL("rank %d holds %ld want %ld", r, static_cast<long>(out[r]), static_cast<long>(want)); return SC_FAIL; }
  DETAIL("%d ranks, %d rounds: every rank holds %ld", world, __builtin_ctz(world), static_cast<long>(want));
  return SC_PASS;
}

struct Entry { const char* name; int (*fn)(char*, size_t); };
const Entry kScenarios[] = {
    {"thread_constructor", sc_thread_constructor}, {"thread_pool", sc_thread_pool}, {"pool_reuse", sc_pool_reuse},
    {"wait_any", sc_wait_any}, {"wait_any_numa", sc_wait_any_numa}, {"wait_any_reuse", sc_wait_any_reuse},
    {"numa_pinning", sc_numa_pinning}, {"rseq_api", sc_rseq_api}, {"numa_arena_buffer", sc_numa_arena_buffer},
    {"numa_arena_scatter", sc_numa_arena_scatter}, {"ring_reduce", sc_ring_reduce}, {"all_reduce", sc_all_reduce},
};

}  // namespace

int scenario_count() { return static_cast<int>(sizeof(kScenarios) / sizeof(kScenarios[0])); }
const char* scenario_name(int i) { return i >= 0 && i < scenario_count() ? kScenarios[i].name : ""; }
int scenario_run(int i, char* detail, size_t n) {
  if (i < 0 || i >= scenario_count() || !detail || n == 0) return SC_FAIL;
  detail[0] = 0;
  return kScenarios[i].fn(detail, n);
}

int run_all_scenarios(bool print) {
  int failed = 0;
  NumaInfo info;
  if (print) std::printf("NUMA: %d nodes, %d CPUs/node\n", info.num_nodes(), info.cpus_per_node());
  for (int i = 0; i < scenario_count(); ++i) {
    char detail[256];
    const int r = scenario_run(i, detail, sizeof detail);
    if (print) std::printf("[%s] %s - %s\n", r == SC_PASS ? "PASS" : r == SC_SKIP ? "SKIP" : "FAIL", scenario_name(i), detail);
    if (r == SC_FAIL) ++failed;
  }
  return failed;
}

}  // namespace hostrt
