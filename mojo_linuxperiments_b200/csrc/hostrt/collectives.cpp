#include "collectives.hpp"

#include <atomic>
#include <vector>
#ifdef HOSTRT_STD_THREADS
#include <thread>
#endif

#include "arena.hpp"
#include "fabric/philox.h"
#include "fabric/protocol.h"
#include "heap_move_array.hpp"
#include "pool.hpp"

namespace hostrt {

namespace {

int node_for_rank(const NumaInfo& info, int rank) {
  if (info.num_nodes() == 0) return -1;
  return info.nodes()[rank % info.num_nodes()].id;
}

// one single-slot pool per rank, pinned to the rank's node
bool make_rank_pools(const NumaInfo& info, int world, HeapMoveArray<ThreadPool>& pools) {
  for (int r = 0; r < world; ++r) {
    const int node = node_for_rank(info, r);
    if (node >= 0) {
      auto m = info.get_node_mask<128>(node);
      if (!pools.emplace(1, m.ptr(), size_t(128), node, stack_size::DEFAULT)) return false;
    } else {
      if (!pools.emplace(1)) return false;
    }
    if (!pools[r]) return false;
  }
  return true;
}

// Run worker(rank, shared) on `world` ranks and join them.  Normally every rank is a one-shot thread of its own
// single-slot pool, pinned to the rank's node.  With -DHOSTRT_STD_THREADS (the thread-sanitizer build) the ranks are
// std::threads instead: ThreadSanitizer only knows threads that were created through pthreads, and what it is asked to
// judge is the protocol (epochs, flags, buffer parity), not the clone3 plumbing.
#ifdef HOSTRT_STD_THREADS
long run_ranks(const NumaInfo&, int world, WorkerFn worker, void* shared, long) {
  std::vector<std::thread> th;
  th.reserve(world);
  for (int r = 0; r < world; ++r)
    th.emplace_back([=] { worker(static_cast<uint64_t>(r), reinterpret_cast<uint64_t>(shared), 0, 0, 0, 0); });
  for (auto& t : th) t.join();
  return 0;
}
#else
long run_ranks(const NumaInfo& info, int world, WorkerFn worker, void* shared, long join_timeout_ns) {
  HeapMoveArray<ThreadPool> pools(world);
  if (!make_rank_pools(info, world, pools)) return -err::kNOMEM;
  for (int r = 0; r < world; ++r)
    if (pools[r].launch(worker, r, reinterpret_cast<uint64_t>(shared)) < 0) return -err::kAGAIN;
  long st = 0;
  for (int r = 0; r < world; ++r) if (pools[r].wait_all(join_timeout_ns) != 0) st = -err::kTIMEDOUT;
  return st;
}
#endif

// ---- chain reduce ----------------------------------------------------------------------------------
struct ChainShared { long timeout_ns; std::atomic<int> errors; };

void chain_worker(uint64_t rank, uint64_t world, uint64_t values_p, uint64_t gates_p, uint64_t shared_p, uint64_t) {
  auto* values = reinterpret_cast<volatile int64_t*>(values_p);
  auto* gates = reinterpret_cast<std::atomic<uint32_t>*>(gates_p);
  auto* sh = reinterpret_cast<ChainShared*>(shared_p);
  const int r = static_cast<int>(rank), w = static_cast<int>(world);
  values[r] = r + 1;
  if (b200::chain_upstream(r, w) >= 0) {
    if (MutexGate{&gates[r]}.wait(sh->timeout_ns) != 0) { sh->errors.fetch_add(1); return; }
    values[r] = values[r] + values[r + 1];
  }
  const int down = b200::chain_downstream(r);
  MutexGate{&gates[down >= 0 ? down : 0]}.release();     // rank 0 releases its own gate: nobody waits on it
}

// ---- butterfly -------------------------------------------------------------------------------------
void bfly_read(uint64_t value_p, uint64_t partner_value_p, uint64_t scratch_p, uint64_t, uint64_t, uint64_t) {
  (void)value_p;
  *reinterpret_cast<volatile int64_t*>(scratch_p) = *reinterpret_cast<volatile int64_t*>(partner_value_p);
}
void bfly_write(uint64_t value_p, uint64_t, uint64_t scratch_p, uint64_t, uint64_t, uint64_t) {
  auto* v = reinterpret_cast<volatile int64_t*>(value_p);
  *v = *v + *reinterpret_cast<volatile int64_t*>(scratch_p);
}

// ---- epoch fabric ----------------------------------------------------------------------------------
struct FabricShared {
  int world, rounds, drop_rank;
  long timeout_ns;
  double* slots;                       // [world] published contributions (double buffered by round parity: 2*world)
  std::atomic<uint32_t>* flags;        // [world*world] flags[dst*world + src] = last epoch src published to dst
  const double* in;
  double* out;
  std::atomic<int> errors;
};

void fabric_worker(uint64_t rank, uint64_t shared_p, uint64_t, uint64_t, uint64_t, uint64_t) {
  auto* sh = reinterpret_cast<FabricShared*>(shared_p);
  const int r = static_cast<int>(rank), w = sh->world;
  if (r == sh->drop_rank) return;                        // injected fault: this rank never takes part
  double acc = sh->in[r];
  for (int round = 0; round < sh->rounds; ++round) {
    const uint32_t epoch = static_cast<uint32_t>(round + 1);
    double* buf = sh->slots + static_cast<size_t>(round & 1) * w;
    buf[r] = round == 0 ? sh->in[r] : acc;               // publish, then signal every peer
    for (int s = 0; s < w; ++s) {
      const int dst = b200::staggered_peer(r, s, w);
      sh->flags[dst * w + r].store(epoch, std::memory_order_release);
    }
    double sum = 0.0;
    const long deadline = sys_clock_monotonic_ns() + sh->timeout_ns;
    for (int src = 0; src < w; ++src) {                  // fixed order: every rank computes the same bits
      while (!b200::epoch_reached(sh->flags[r * w + src].load(std::memory_order_acquire), epoch)) {
        if (sys_clock_monotonic_ns() > deadline) { sh->errors.fetch_add(1); return; }
        asm volatile("pause");
      }
      sum += buf[src];
    }
    acc = sum;
  }
  sh->out[r] = acc;
}

// ---- token-sharded exchange protocol (threads as ranks) -------------------------------------------------
// The CPU statement of the protocol the GPU kernels of csrc/kernels/tp_link.cuh use: per-rank "heaps" with two
// gather buffers and two receive areas selected by the parity of a per-rank epoch, per-(source, block) epoch flags,
// per-consumer "done" words that gate the reuse of a gather buffer two calls later, and arrival counters that the
// owner resets.  Ranks are skewed against each other on purpose; any hole in the protocol shows up as a payload that
// does not match its closed-form expectation.
struct ExchangeShared {
  int world, rows, blocks, iters;
  int mode;                            // 1 all-gather only, 2 reduce-scatter only, 3 both in turn
  int fault;                           // deliberate holes: 1 skip the wait for the done acknowledgements, 2 one buffer instead of two
  long timeout_ns;
  uint32_t skew_seed;
  uint64_t* gather;                    // [world heaps][2][world * rows] rows as one 64-bit word each
  uint64_t* recv;                      // [world heaps][2][world sources][rows]
  std::atomic<uint32_t>* flags;        // [world heaps][world sources][blocks]
  std::atomic<uint32_t>* done;         // [world heaps][world consumers]
  std::atomic<uint32_t>* ctr;          // [world heaps][2]
  std::atomic<int> errors;
  std::atomic<int> timeouts;
};

inline uint64_t exch_row_value(int src, int row, uint32_t epoch) { return (static_cast<uint64_t>(epoch) << 32) | (static_cast<uint64_t>(src) << 20) | row; }
inline uint64_t exch_part_value(int src, int owner, int row, uint32_t epoch) { return static_cast<uint64_t>(epoch) * 1000003ull + src * 7919ull + owner * 104729ull + row; }

void exchange_worker(uint64_t rank, uint64_t shared_p, uint64_t, uint64_t, uint64_t, uint64_t) {
  auto* sh = reinterpret_cast<ExchangeShared*>(shared_p);
  const int r = static_cast<int>(rank), w = sh->world, R = sh->rows, B = sh->blocks;
  const size_t M = static_cast<size_t>(w) * R;
  uint32_t rng = sh->skew_seed * 2654435761u + r * 40503u + 1u;
  auto skew = [&]() {                                  // a pseudo-random pause of up to ~20 us
    rng = rng * 1664525u + 1013904223u;
    const long until = sys_clock_monotonic_ns() + static_cast<long>((rng >> 8) % 20000u);
    while (sys_clock_monotonic_ns() < until) asm volatile("pause");
  };
  auto wait_ge = [&](std::atomic<uint32_t>& word, uint32_t target) -> bool {
    const long deadline = sys_clock_monotonic_ns() + sh->timeout_ns;
    while (!b200::epoch_reached(word.load(std::memory_order_acquire), target)) {
      if (sys_clock_monotonic_ns() > deadline) { sh->timeouts.fetch_add(1); return false; }
      asm volatile("pause");
    }
    return true;
  };
  auto gather_of = [&](int heap, int par) { return sh->gather + (static_cast<size_t>(heap) * 2 + par) * M; };
  auto recv_of = [&](int heap, int par, int src) { return sh->recv + ((static_cast<size_t>(heap) * 2 + par) * w + src) * R; };
  for (int it = 0; it < sh->iters; ++it) {
    const uint32_t e = static_cast<uint32_t>(it + 1);
    const int par = (sh->fault & 2) ? 0 : static_cast<int>(e & 1u);
    skew();
    if (sh->mode & 1) {
    // ---- all-gather: wait for the acknowledgements of the call before last, push my rows block by block ----
    if (!(sh->fault & 1))
      for (int p = 0; p < w; ++p) if (!wait_ge(sh->done[static_cast<size_t>(r) * w + p], e - 2u)) return;
    for (int blk = 0; blk < B; ++blk) {
      const int r0 = blk * (R / B), r1 = blk + 1 == B ? R : (blk + 1) * (R / B);
      for (int s = 0; s < w; ++s) {
        const int dst = b200::staggered_peer(r, s, w);
        uint64_t* g = gather_of(dst, par);
        for (int row = r0; row < r1; ++row) g[static_cast<size_t>(r) * R + row] = exch_row_value(r, row, e);
      }
      for (int dst = 0; dst < w; ++dst) sh->flags[(static_cast<size_t>(dst) * w + r) * B + blk].store(e, std::memory_order_release);
      if (blk & 1) skew();
    }
    if (r == 0 && sh->fault) { skew(); skew(); skew(); skew(); skew(); }   // a slow consumer makes a hole visible
    // ---- consume: every source, every block, starting with my own rows ----
    for (int s = 0; s < w; ++s) {
      const int src = b200::staggered_peer(r, s, w);
      for (int blk = 0; blk < B; ++blk) {
        if (!wait_ge(sh->flags[(static_cast<size_t>(r) * w + src) * B + blk], e)) return;
        const int r0 = blk * (R / B), r1 = blk + 1 == B ? R : (blk + 1) * (R / B);
        const uint64_t* g = gather_of(r, par);
        for (int row = r0; row < r1; ++row)
          if (g[static_cast<size_t>(src) * R + row] != exch_row_value(src, row, e)) sh->errors.fetch_add(1);
      }
    }
    for (int p = 0; p < w; ++p) sh->done[static_cast<size_t>(p) * w + r].store(e, std::memory_order_release);
    }
    skew();
    if (!(sh->mode & 2)) continue;
    // ---- reduce-scatter: my partial of every owner's rows into its receive area, own rows last ----
    for (int s = 1; s <= w; ++s) {
      const int owner = b200::staggered_peer(r, s, w);
      uint64_t* dst = recv_of(owner, par, r);
      for (int row = 0; row < R; ++row) dst[row] = exch_part_value(r, owner, row, e);
      sh->ctr[static_cast<size_t>(owner) * 2 + par].fetch_add(static_cast<uint32_t>(R), std::memory_order_release);
    }
    if (!wait_ge(sh->ctr[static_cast<size_t>(r) * 2 + par], static_cast<uint32_t>(w) * R)) return;
    for (int row = 0; row < R; ++row) {
      uint64_t got = 0, want = 0;
      for (int src = 0; src < w; ++src) { got += recv_of(r, par, src)[row]; want += exch_part_value(src, r, row, e); }
      if (got != want) sh->errors.fetch_add(1);
    }
    sh->ctr[static_cast<size_t>(r) * 2 + par].store(0, std::memory_order_release);     // the owner resets its own counter
  }
}

// ---- fill + reduce ---------------------------------------------------------------------------------
struct FillJob {
  float* buf;
  uint64_t begin, end, seed;
  double partial;
  int expect_node;
  int seen_node;
  int mem_node;
};

void fill_worker(uint64_t job_p, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t) {
  auto* j = reinterpret_cast<FillJob*>(job_p);
  double s = 0.0;
  float* out = j->buf;
  uint64_t i = j->begin;
  // whole Philox blocks of four where possible
  for (; i < j->end && (i & 3); ++i) { const float v = b200::philox_uniform_pm1(i, j->seed); *out++ = v; s += v; }
  for (; i + 4 <= j->end; i += 4) {
    const b200::Philox4 r = b200::philox4x32_10(i >> 2, j->seed);
    for (int k = 0; k < 4; ++k) { const float v = b200::u32_to_uniform_pm1(r.v[k]); *out++ = v; s += v; }
  }
  for (; i < j->end; ++i) { const float v = b200::philox_uniform_pm1(i, j->seed); *out++ = v; s += v; }
  j->partial = s;
  j->seen_node = get_current_cpu_and_node().node;
  j->mem_node = j->end > j->begin ? static_cast<int>(sys_move_pages_query(j->buf)) : j->expect_node;
}

}  // namespace

CollectiveResult chain_reduce(const NumaInfo& info, int world, long timeout_ns) {
  if (world < 1) return {-err::kINVAL, 0};
  NumaArena arena(node_for_rank(info, 0), 4096 + static_cast<size_t>(world) * 16, 8, page_size::STANDARD);
  if (!arena) return {-err::kNOMEM, 0};
  auto* values = arena.alloc<int64_t>(world);
  auto* gates = arena.alloc<std::atomic<uint32_t>>(world);      // fresh anonymous memory: all gates closed
  auto* shared = arena.alloc<ChainShared>(1);
  if (!values || !gates || !shared) return {-err::kNOMEM, 0};
  shared->timeout_ns = timeout_ns;
  shared->errors.store(0);
  HeapMoveArray<ThreadPool> pools(world);
  if (!make_rank_pools(info, world, pools)) return {-err::kNOMEM, 0};
  for (int r = 0; r < world; ++r)
    if (pools[r].launch(&chain_worker, r, world, reinterpret_cast<uint64_t>(values), reinterpret_cast<uint64_t>(gates),
                        reinterpret_cast<uint64_t>(shared)) < 0)
      return {-err::kAGAIN, 0};
  long st = 0;
  for (int r = 0; r < world; ++r) if (pools[r].wait_all(timeout_ns < 0 ? -1 : timeout_ns * 2) != 0) st = -err::kTIMEDOUT;
  if (st == 0 && shared->errors.load() != 0) st = -err::kTIMEDOUT;
  return {st, values[0]};
}

long butterfly_allreduce(const NumaInfo& info, int world, int64_t* out, long timeout_ns) {
  if (world < 1 || !b200::is_pow2(world)) return -err::kINVAL;
  NumaArena arena(node_for_rank(info, 0), 4096 + static_cast<size_t>(world) * 16, 8, page_size::STANDARD);
  if (!arena) return -err::kNOMEM;
  auto* values = arena.alloc<int64_t>(world);
  auto* scratch = arena.alloc<int64_t>(world);
  if (!values || !scratch) return -err::kNOMEM;
  for (int r = 0; r < world; ++r) values[r] = r + 1;
  HeapMoveArray<ThreadPool> pools(world);
  if (!make_rank_pools(info, world, pools)) return -err::kNOMEM;
  auto phase = [&](WorkerFn fn, int round) -> long {
    for (int r = 0; r < world; ++r) {
      const int p = b200::butterfly_partner(r, round);
      if (pools[r].launch(fn, reinterpret_cast<uint64_t>(&values[r]), reinterpret_cast<uint64_t>(&values[p]),
                          reinterpret_cast<uint64_t>(&scratch[r])) < 0)
        return -err::kAGAIN;
    }
    for (int r = 0; r < world; ++r) if (pools[r].wait_all(timeout_ns) != 0) return -err::kTIMEDOUT;   // global barrier
    return 0;
  };
  for (int round = 0; round < b200::butterfly_rounds(world); ++round) {
    long st = phase(&bfly_read, round);
    if (st == 0) st = phase(&bfly_write, round);
    if (st != 0) return st;
  }
  for (int r = 0; r < world; ++r) out[r] = values[r];
  return 0;
}

long fabric_allreduce(const NumaInfo& info, int world, const double* in, double* out, int rounds, long timeout_ns,
                      int drop_rank) {
  if (world < 1 || rounds < 1) return -err::kINVAL;
  const size_t bytes = 8192 + static_cast<size_t>(world) * world * 4 + static_cast<size_t>(world) * 16;
  NumaArena arena(node_for_rank(info, 0), bytes, 64, page_size::STANDARD);
  if (!arena) return -err::kNOMEM;
  FabricShared sh{};
  sh.world = world; sh.rounds = rounds; sh.drop_rank = drop_rank; sh.timeout_ns = timeout_ns;
  sh.slots = arena.alloc<double>(2 * static_cast<size_t>(world));
  sh.flags = arena.alloc<std::atomic<uint32_t>>(static_cast<size_t>(world) * world);
  sh.in = in; sh.out = out;
  sh.errors.store(0);
  if (!sh.slots || !sh.flags) return -err::kNOMEM;
  long st = run_ranks(info, world, &fabric_worker, &sh, timeout_ns * 4 + 1'000'000'000l);
  if (st == 0 && sh.errors.load() != 0) st = -err::kTIMEDOUT;
  return st;
}

long fabric_token_exchange(const NumaInfo& info, int world, int rows_per_rank, int blocks, int iters, long timeout_ns,
                           uint32_t skew_seed, int mode, int fault, int* mismatches) {
  if (world < 1 || rows_per_rank < 1 || blocks < 1 || blocks > rows_per_rank || iters < 1 || mode < 1 || mode > 3) return -err::kINVAL;
  const size_t M = static_cast<size_t>(world) * rows_per_rank;
  const size_t words = static_cast<size_t>(world) * 2 * M * 2;
  const size_t bytes = words * 8 + static_cast<size_t>(world) * world * (blocks + 1) * 4 + static_cast<size_t>(world) * 8 + 65536;
  NumaArena arena(node_for_rank(info, 0), bytes, 64, page_size::STANDARD);
  if (!arena) return -err::kNOMEM;
  ExchangeShared sh{};
  sh.world = world; sh.rows = rows_per_rank; sh.blocks = blocks; sh.iters = iters; sh.timeout_ns = timeout_ns; sh.skew_seed = skew_seed;
  sh.mode = mode; sh.fault = fault;
  sh.gather = arena.alloc<uint64_t>(static_cast<size_t>(world) * 2 * M);
  sh.recv = arena.alloc<uint64_t>(static_cast<size_t>(world) * 2 * M);
  sh.flags = arena.alloc<std::atomic<uint32_t>>(static_cast<size_t>(world) * world * blocks);
  sh.done = arena.alloc<std::atomic<uint32_t>>(static_cast<size_t>(world) * world);
  sh.ctr = arena.alloc<std::atomic<uint32_t>>(static_cast<size_t>(world) * 2);
  sh.errors.store(0); sh.timeouts.store(0);
  if (!sh.gather || !sh.recv || !sh.flags || !sh.done || !sh.ctr) return -err::kNOMEM;
  long st = run_ranks(info, world, &exchange_worker, &sh, timeout_ns * 4 + 10'000'000'000l);
  if (mismatches) *mismatches = sh.errors.load();
  if (st == 0 && sh.timeouts.load() != 0) st = -err::kTIMEDOUT;
  return st;
}

FillReduceResult fill_reduce(const NumaInfo& info, uint64_t n_elems, uint64_t seed, int max_workers_per_node) {
  FillReduceResult res{};
  const int nn = info.num_nodes();
  if (nn == 0) { res.status = -err::kNOENT; return res; }
  // who works where
  std::vector<int> per_node(nn);
  int total = 0;
  for (int k = 0; k < nn; ++k) {
    int c = static_cast<int>(info.nodes()[k].cpu_ids.size());
    if (max_workers_per_node > 0 && c > max_workers_per_node) c = max_workers_per_node;
    per_node[k] = c;
    total += c;
  }
  if (total == 0) { res.status = -err::kNOENT; return res; }
  std::vector<FillJob> jobs(total);
  HeapMoveArray<NumaArena> arenas(nn);
  HeapMoveArray<ThreadPool> pools(nn);
  int w = 0;
  for (int k = 0; k < nn; ++k) {
    const int node = info.nodes()[k].id;
    const uint64_t nb = n_elems * (w) / total, ne = n_elems * (w + per_node[k]) / total;
    arenas.emplace(node, static_cast<size_t>(ne - nb) * sizeof(float) + 4096, size_t(64), page_size::THP_2MB);
    auto m = info.get_node_mask<128>(node);
    pools.emplace(per_node[k], m.ptr(), size_t(128), node, stack_size::DEFAULT);
    if (!arenas[k] || !pools[k]) { res.status = -err::kNOMEM; return res; }
    for (int i = 0; i < per_node[k]; ++i, ++w) {
      FillJob& j = jobs[w];
      j.begin = n_elems * w / total;
      j.end = n_elems * (w + 1) / total;
      j.seed = seed;
      j.buf = arenas[k].alloc<float>(j.end - j.begin);
      j.expect_node = node;
      j.partial = 0; j.seen_node = -1; j.mem_node = -1;
      if (!j.buf) { res.status = -err::kNOMEM; return res; }
    }
  }
  const long t0 = sys_clock_monotonic_ns();
  w = 0;
  for (int k = 0; k < nn; ++k)
    for (int i = 0; i < per_node[k]; ++i, ++w)
      if (pools[k].launch(&fill_worker, reinterpret_cast<uint64_t>(&jobs[w])) < 0) { res.status = -err::kAGAIN; }
  for (int k = 0; k < nn; ++k) if (pools[k].wait_all(120'000'000'000l) != 0) res.status = -err::kTIMEDOUT;
  if (res.status != 0) return res;
  // tree reduce: workers -> node partials (pairwise), nodes -> global (pairwise)
  std::vector<double> node_sum(nn, 0.0);
  w = 0;
  for (int k = 0; k < nn; ++k) {
    std::vector<double> v(per_node[k]);
    for (int i = 0; i < per_node[k]; ++i, ++w) {
      v[i] = jobs[w].partial;
      if (jobs[w].seen_node != jobs[w].expect_node || (jobs[w].mem_node >= 0 && jobs[w].mem_node != jobs[w].expect_node)) ++res.misplaced;
    }
    for (size_t stride = 1; stride < v.size(); stride *= 2)
      for (size_t i = 0; i + stride < v.size(); i += 2 * stride) v[i] += v[i + stride];
    node_sum[k] = v.empty() ? 0.0 : v[0];
  }
  for (size_t stride = 1; stride < node_sum.size(); stride *= 2)
    for (size_t i = 0; i + stride < node_sum.size(); i += 2 * stride) node_sum[i] += node_sum[i + stride];
  res.sum = node_sum[0];
  res.elapsed_ns = sys_clock_monotonic_ns() - t0;
  res.workers = total;
  res.nodes = nn;
  return res;
}

double fill_reduce_serial(uint64_t n_elems, uint64_t seed) {
  double s = 0.0;
  for (uint64_t i = 0; i < n_elems; ++i) s += b200::philox_uniform_pm1(i, seed);
  return s;
}

}  // namespace hostrt
