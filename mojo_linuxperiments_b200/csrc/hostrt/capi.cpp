// C ABI of the host runtime (loaded from Python with ctypes).  Handles are opaque pointers; functions return
// >= 0 on success and -errno on failure unless stated otherwise.
#include <cstring>
#include <string>

#include "arena.hpp"
#include "collectives.hpp"
#include "w8a8_host.hpp"
#include "numa.hpp"
#include "pool.hpp"
#include "scenarios.hpp"
#include "fabric/philox.h"
#include "fabric/range_check.h"

using namespace hostrt;

extern "C" {

// ---- kernel ABI facts (for tests that compare against the system headers) ------------------------------
long hostrt_syscall_nr(const char* name) {
  const std::string s(name);
  if (s == "mmap") return nr::mmap; if (s == "mprotect") return nr::mprotect; if (s == "munmap") return nr::munmap;
  if (s == "madvise") return nr::madvise; if (s == "exit") return nr::exit; if (s == "gettid") return nr::gettid;
  if (s == "sched_setaffinity") return nr::sched_setaffinity; if (s == "mbind") return nr::mbind;
  if (s == "move_pages") return nr::move_pages; if (s == "rseq") return nr::rseq; if (s == "clone3") return nr::clone3;
  if (s == "futex_waitv") return nr::futex_waitv; if (s == "futex_wake") return nr::futex_wake;
  if (s == "futex_wait") return nr::futex_wait; if (s == "getcpu") return nr::getcpu;
  if (s == "nanosleep") return nr::nanosleep; if (s == "clock_gettime") return nr::clock_gettime;
  if (s == "sched_getaffinity") return nr::sched_getaffinity;
  return -1;
}
unsigned long long hostrt_thread_clone_flags() { return clone_flag::THREAD_FLAGS; }
long hostrt_struct_size(const char* name) {
  const std::string s(name);
  if (s == "FutexNuma32") return sizeof(FutexNuma32); if (s == "FutexWaitv") return sizeof(FutexWaitv);
  if (s == "Clone3Args") return sizeof(Clone3Args); if (s == "Rseq") return sizeof(Rseq);
  return -1;
}
long hostrt_slot_total_size(unsigned long stack_bytes) { return static_cast<long>(slot_total_size(stack_bytes)); }
long hostrt_gettid() { return sys_gettid(); }
// The range check the debug build of the GPU kernels applies to heap offsets, run on the host: returns 1 when the
// access may go ahead; otherwise 0, and report3 = {code, offset low, offset high} if it was still empty.
int hostrt_range_check(unsigned long long off, unsigned long long len, unsigned long long extent, int* report3) {
  b200::RangeReport rep{report3 ? report3[0] : 0, report3 ? static_cast<unsigned>(report3[1]) : 0u, report3 ? static_cast<unsigned>(report3[2]) : 0u};
  const bool ok = b200::range_check_record(off, len, extent, &rep);
  if (report3) { report3[0] = rep.code; report3[1] = static_cast<int>(rep.off_lo); report3[2] = static_cast<int>(rep.off_hi); }
  return ok ? 1 : 0;
}
long hostrt_monotonic_ns() { return sys_clock_monotonic_ns(); }

// ---- raw memory calls -----------------------------------------------------------------------------------
void* hostrt_mmap_numa(unsigned long size, int node, long page_mode) { return mmap_numa(size, node, page_mode); }
long hostrt_munmap(void* p, unsigned long size) { return sys_munmap(p, size); }
long hostrt_move_pages_query(const void* p) { return sys_move_pages_query(p); }
long hostrt_mprotect(void* p, unsigned long size, long pr) { return sys_mprotect(p, size, pr); }
void hostrt_poke(void* p, long long v) { *static_cast<volatile long long*>(p) = v; }
long long hostrt_peek(const void* p) { return *static_cast<const volatile long long*>(p); }

// ---- topology ---------------------------------------------------------------------------------------------
void* hostrt_numa_create(const char* root) { return new NumaInfo(root && root[0] ? root : "/sys/devices/system/node"); }
void hostrt_numa_destroy(void* h) { delete static_cast<NumaInfo*>(h); }
int hostrt_numa_ok(void* h) { return static_cast<NumaInfo*>(h)->ok() ? 1 : 0; }
int hostrt_numa_num_nodes(void* h) { return static_cast<NumaInfo*>(h)->num_nodes(); }
int hostrt_numa_node_id(void* h, int index) {
  auto* n = static_cast<NumaInfo*>(h);
  return index >= 0 && index < n->num_nodes() ? n->nodes()[index].id : -1;
}
int hostrt_numa_node_cpus(void* h, int node, int* out, int cap) {
  const auto& v = static_cast<NumaInfo*>(h)->get_node_cpus(node);
  for (int i = 0; i < static_cast<int>(v.size()) && i < cap; ++i) out[i] = v[i];
  return static_cast<int>(v.size());
}
int hostrt_numa_node_mask(void* h, int node, unsigned char* mask128) {
  auto m = static_cast<NumaInfo*>(h)->get_node_mask<128>(node);
  m.copy_to(mask128);
  return static_cast<int>(m.count());
}
int hostrt_numa_distance(void* h, int a, int b) { return static_cast<NumaInfo*>(h)->distance(a, b); }
int hostrt_numa_cpus_per_node(void* h) { return static_cast<NumaInfo*>(h)->cpus_per_node(); }
int hostrt_numa_cpus_on_node(void* h, int node) { return static_cast<NumaInfo*>(h)->cpus_on_node(node); }
int hostrt_numa_total_cpus(void* h) { return static_cast<NumaInfo*>(h)->total_cpus(); }
long hostrt_numa_mem_kb(void* h, int node, int free_not_total) {
  const NumaNode* n = static_cast<NumaInfo*>(h)->node(node);
  return n ? (free_not_total ? n->mem_free_kb : n->mem_total_kb) : -1;
}
int hostrt_numa_debug(void* h, char* out, int cap) {
  const std::string s = static_cast<NumaInfo*>(h)->debug_string();
  std::strncpy(out, s.c_str(), cap > 0 ? cap - 1 : 0);
  if (cap > 0) out[cap - 1] = 0;
  return static_cast<int>(s.size());
}
int hostrt_parse_cpulist(const char* text, int* out, int cap) {
  const auto v = parse_cpulist(text);
  for (int i = 0; i < static_cast<int>(v.size()) && i < cap; ++i) out[i] = v[i];
  return static_cast<int>(v.size());
}
long hostrt_parse_meminfo(const char* text, const char* field) { return parse_meminfo_field(text, field); }
void hostrt_current_cpu_node(int* cpu, int* node) { const CpuNode c = get_current_cpu_and_node(); *cpu = c.cpu; *node = c.node; }
void hostrt_current_cpu_node_rseq(int* cpu, int* node) { const CpuNode c = get_cpu_and_node_rseq(); *cpu = c.cpu; *node = c.node; }

// ---- CpuMask over a caller-owned 128-byte buffer ------------------------------------------------------------
static CpuMask<128>* M(void* p) { return static_cast<CpuMask<128>*>(p); }
int hostrt_cpumask_bytes() { return 128; }
void hostrt_cpumask_set(void* m, long cpu) { M(m)->set(cpu); }
void hostrt_cpumask_clear(void* m, long cpu) { M(m)->clear(cpu); }
int hostrt_cpumask_test(void* m, long cpu) { return M(m)->test(cpu) ? 1 : 0; }
void hostrt_cpumask_clear_all(void* m) { M(m)->clear_all(); }
void hostrt_cpumask_set_all(void* m) { M(m)->set_all(); }
long hostrt_cpumask_count(void* m) { return static_cast<long>(M(m)->count()); }
long hostrt_set_thread_affinity(const unsigned char* mask, unsigned long bytes) { return set_thread_affinity_raw(mask, bytes); }
long hostrt_get_thread_affinity(unsigned char* mask, unsigned long bytes) { return sys_sched_getaffinity(0, bytes, mask); }

// ---- arena ----------------------------------------------------------------------------------------------------
void* hostrt_arena_create(int node, unsigned long size, unsigned long alignment, long page_mode) {
  return new NumaArena(node, size, alignment, page_mode);
}
void hostrt_arena_destroy(void* a) { delete static_cast<NumaArena*>(a); }
int hostrt_arena_valid(void* a) { return *static_cast<NumaArena*>(a) ? 1 : 0; }
unsigned long hostrt_arena_mapped_bytes(void* a) { return static_cast<NumaArena*>(a)->mapped_bytes(); }
// destroys the arena and reports what its munmap returned (0, or -errno): only tests need the value
long hostrt_arena_unmap_status(void* a) {
  auto* ar = static_cast<NumaArena*>(a);
  const long r = ar->base() ? sys_munmap(ar->base(), ar->mapped_bytes()) : 0;
  ar->forget();
  delete ar;
  return r;
}
void* hostrt_arena_alloc(void* a, unsigned long bytes) { return static_cast<NumaArena*>(a)->alloc_bytes(bytes); }
unsigned long hostrt_arena_mark(void* a) { return static_cast<NumaArena*>(a)->mark(); }
void hostrt_arena_reset_to(void* a, unsigned long w) { static_cast<NumaArena*>(a)->reset_to(w); }
void hostrt_arena_reset(void* a) { static_cast<NumaArena*>(a)->reset(); }
unsigned long hostrt_arena_remaining(void* a) { return static_cast<NumaArena*>(a)->remaining(); }
unsigned long hostrt_arena_used(void* a) { return static_cast<NumaArena*>(a)->used(); }
void* hostrt_arena_base(void* a) { return static_cast<NumaArena*>(a)->base(); }
int hostrt_arena_verify_placement(void* a) { return static_cast<NumaArena*>(a)->verify_placement() ? 1 : 0; }

// ---- pool -------------------------------------------------------------------------------------------------------
void* hostrt_pool_create(int capacity, const unsigned char* mask, unsigned long mask_bytes, int node, unsigned long stack_bytes) {
  return new ThreadPool(capacity, mask, mask_bytes, node, stack_bytes ? stack_bytes : stack_size::DEFAULT);
}
void hostrt_pool_destroy(void* p) { delete static_cast<ThreadPool*>(p); }
int hostrt_pool_valid(void* p) { return *static_cast<ThreadPool*>(p) ? 1 : 0; }
int hostrt_pool_capacity(void* p) { return static_cast<ThreadPool*>(p)->capacity(); }
unsigned hostrt_pool_futex_flags(void* p) { return static_cast<ThreadPool*>(p)->futex_flags(); }
int hostrt_pool_running(void* p) { return static_cast<ThreadPool*>(p)->running_count(); }
int hostrt_pool_launch(void* p, void* fn, unsigned long long a0, unsigned long long a1, unsigned long long a2,
                       unsigned long long a3, unsigned long long a4, unsigned long long a5) {
  return static_cast<ThreadPool*>(p)->launch(reinterpret_cast<WorkerFn>(fn), a0, a1, a2, a3, a4, a5);
}
long hostrt_pool_wait_all(void* p, long timeout_ns) { return static_cast<ThreadPool*>(p)->wait_all(timeout_ns); }
int hostrt_pool_wait_any(void* p, long timeout_ns) { return static_cast<ThreadPool*>(p)->wait_any(timeout_ns); }

// built-in workers a Python caller can launch by address (a Python function cannot run on a raw clone3 thread)
void hostrt_worker_store(unsigned long long dst, unsigned long long value, unsigned long long, unsigned long long,
                         unsigned long long, unsigned long long) {
  *reinterpret_cast<volatile unsigned long long*>(dst) = value;
}
void hostrt_worker_sleep_store(unsigned long long ms, unsigned long long dst, unsigned long long value,
                               unsigned long long, unsigned long long, unsigned long long) {
  sys_nanosleep(static_cast<long>(ms) * 1000000l);
  if (dst) *reinterpret_cast<volatile unsigned long long*>(dst) = value;
}
void hostrt_worker_where(unsigned long long dst_cpu_node, unsigned long long, unsigned long long, unsigned long long,
                         unsigned long long, unsigned long long) {
  auto* out = reinterpret_cast<volatile int*>(dst_cpu_node);
  const CpuNode a = get_current_cpu_and_node();
  const CpuNode b = get_cpu_and_node_rseq();
  out[0] = a.cpu; out[1] = a.node; out[2] = b.cpu; out[3] = b.node;
}
void hostrt_worker_gate_wait_store(unsigned long long gate, unsigned long long timeout_ns, unsigned long long dst,
                                   unsigned long long, unsigned long long, unsigned long long) {
  const long r = MutexGate::from_addr(reinterpret_cast<void*>(gate)).wait(static_cast<long>(timeout_ns));
  *reinterpret_cast<volatile long long*>(dst) = r == 0 ? 1 : r;
}

// ---- gate ---------------------------------------------------------------------------------------------------------
long hostrt_gate_wait(void* word, long timeout_ns) { return MutexGate::from_addr(word).wait(timeout_ns); }
void hostrt_gate_release(void* word) { MutexGate::from_addr(word).release(); }
void hostrt_gate_reset(void* word) { MutexGate::from_addr(word).reset(); }

// ---- collectives and the config-1 workload ---------------------------------------------------------------------------
long hostrt_chain_reduce(void* numa, int world, long timeout_ns, long long* value) {
  const CollectiveResult r = chain_reduce(*static_cast<NumaInfo*>(numa), world, timeout_ns);
  *value = r.value;
  return r.status;
}
long hostrt_butterfly_allreduce(void* numa, int world, long long* out, long timeout_ns) {
  return butterfly_allreduce(*static_cast<NumaInfo*>(numa), world, reinterpret_cast<int64_t*>(out), timeout_ns);
}
long hostrt_fabric_allreduce(void* numa, int world, const double* in, double* out, int rounds, long timeout_ns, int drop_rank) {
  return fabric_allreduce(*static_cast<NumaInfo*>(numa), world, in, out, rounds, timeout_ns, drop_rank);
}
void* hostrt_team_create(void* numa, int max_workers_per_node) {
  auto* t = new WorkerTeam(*static_cast<NumaInfo*>(numa), max_workers_per_node);
  if (!*t) { delete t; return nullptr; }
  return t;
}
void hostrt_team_destroy(void* team) { delete static_cast<WorkerTeam*>(team); }
int hostrt_team_valid(void* team) { return static_cast<bool>(*static_cast<WorkerTeam*>(team)) ? 1 : 0; }
int hostrt_team_stragglers(void* team) { return static_cast<WorkerTeam*>(team)->stragglers() ? 1 : 0; }
int hostrt_team_node_of(void* team, int worker) { return static_cast<WorkerTeam*>(team)->node_of(worker); }
// Test hook for the timeout path: every worker sleeps sleep_ms inside the job, the caller waits timeout_ms at most.
// The job's argument block lives on the heap and is intentionally kept alive until the team is destroyed.
long hostrt_team_run_sleep(void* team, long sleep_ms, long timeout_ms) {
  auto* t = static_cast<WorkerTeam*>(team);
  static std::vector<uint64_t>* keep = new std::vector<uint64_t>();
  keep->assign(static_cast<size_t>(t->size()), static_cast<uint64_t>(sleep_ms));
  return t->run(
      +[](uint64_t ms, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t) {
        const long end = sys_clock_monotonic_ns() + static_cast<long>(ms) * 1'000'000l;
        uint32_t word = 0;
        while (sys_clock_monotonic_ns() < end) sys_futex_wait(&word, 0, futex2::SIZE_U32 | futex2::PRIVATE, 1'000'000l);
      },
      keep->data(), timeout_ms * 1'000'000l);
}
int hostrt_team_size(void* team) { return static_cast<WorkerTeam*>(team)->size(); }
unsigned long long hostrt_team_jobs_run(void* team) { return static_cast<WorkerTeam*>(team)->jobs_run(); }
long hostrt_w8a8_linear_team(void* team, const void* x_bf16, int M, int K, const void* wq, const float* sw, int N, void* y_bf16,
                             int force_scalar, void* q_out, float* sx_out, int* acc_out, long* info5) {
  const W8A8HostResult r = w8a8_linear_team(*static_cast<WorkerTeam*>(team), static_cast<const uint16_t*>(x_bf16), M, K,
                                            static_cast<const int8_t*>(wq), sw, N, static_cast<uint16_t*>(y_bf16), force_scalar,
                                            static_cast<int8_t*>(q_out), sx_out, reinterpret_cast<int32_t*>(acc_out));
  if (info5) { info5[0] = r.quant_ns; info5[1] = r.gemm_ns; info5[2] = r.workers; info5[3] = r.used_vnni; info5[4] = 0; }
  return r.status;
}
void* hostrt_weights_create(void* team, const void* wq, int N, int K) {
  auto* w = new NodeShardedWeights(*static_cast<WorkerTeam*>(team), static_cast<const int8_t*>(wq), N, K);
  if (!*w) { delete w; return nullptr; }
  return w;
}
void hostrt_weights_destroy(void* w) { delete static_cast<NodeShardedWeights*>(w); }
int hostrt_weights_misplaced(void* w) { return static_cast<NodeShardedWeights*>(w)->misplaced(); }
long hostrt_w8a8_linear_sharded(void* team, void* weights, const void* x_bf16, int M, const float* sw, void* y_bf16,
                                int force_scalar, void* q_out, float* sx_out, int* acc_out, long* info5) {
  const W8A8HostResult r = w8a8_linear_team_sharded(*static_cast<WorkerTeam*>(team), *static_cast<NodeShardedWeights*>(weights),
                                                    static_cast<const uint16_t*>(x_bf16), M, sw, static_cast<uint16_t*>(y_bf16),
                                                    force_scalar, static_cast<int8_t*>(q_out), sx_out,
                                                    reinterpret_cast<int32_t*>(acc_out));
  if (info5) { info5[0] = r.quant_ns; info5[1] = r.gemm_ns; info5[2] = r.workers; info5[3] = r.used_vnni; info5[4] = 0; }
  return r.status;
}
long hostrt_fabric_token_exchange(void* numa, int world, int rows_per_rank, int blocks, int iters, long timeout_ns,
                                  unsigned skew_seed, int mode, int fault, int* mismatches) {
  return fabric_token_exchange(*static_cast<NumaInfo*>(numa), world, rows_per_rank, blocks, iters, timeout_ns, skew_seed, mode, fault,
                               mismatches);
}
long hostrt_fill_reduce(void* numa, unsigned long long n, unsigned long long seed, int max_workers_per_node, double* sum,
                        long* elapsed_ns, int* workers, int* misplaced) {
  const FillReduceResult r = fill_reduce(*static_cast<NumaInfo*>(numa), n, seed, max_workers_per_node);
  *sum = r.sum; *elapsed_ns = r.elapsed_ns; *workers = r.workers; *misplaced = r.misplaced;
  return r.status;
}
double hostrt_fill_reduce_serial(unsigned long long n, unsigned long long seed) { return fill_reduce_serial(n, seed); }
// info5: {quant_ns, gemm_ns, workers, used_vnni, -}
long hostrt_w8a8_linear(void* numa, const void* x_bf16, int M, int K, const void* wq, const float* sw, int N, void* y_bf16,
                        int max_workers_per_node, int force_scalar, void* q_out, float* sx_out, int* acc_out, long* info5) {
  const W8A8HostResult r = w8a8_linear_host(*static_cast<NumaInfo*>(numa), static_cast<const uint16_t*>(x_bf16), M, K,
                                            static_cast<const int8_t*>(wq), sw, N, static_cast<uint16_t*>(y_bf16),
                                            max_workers_per_node, force_scalar, static_cast<int8_t*>(q_out), sx_out,
                                            reinterpret_cast<int32_t*>(acc_out));
  if (info5) { info5[0] = r.quant_ns; info5[1] = r.gemm_ns; info5[2] = r.workers; info5[3] = r.used_vnni; info5[4] = 0; }
  return r.status;
}
float hostrt_philox_uniform(unsigned long long i, unsigned long long seed) { return b200::philox_uniform_pm1(i, seed); }
void hostrt_philox_block(unsigned long long counter, unsigned long long seed, unsigned* out4) {
  const b200::Philox4 r = b200::philox4x32_10(counter, seed);
  for (int k = 0; k < 4; ++k) out4[k] = r.v[k];
}

// ---- scenarios ----------------------------------------------------------------------------------------------------------
int hostrt_scenario_count() { return scenario_count(); }
const char* hostrt_scenario_name(int i) { return scenario_name(i); }
int hostrt_scenario_run(int i, char* detail, int cap) { return scenario_run(i, detail, static_cast<size_t>(cap)); }
int hostrt_run_all_scenarios(int print) { return run_all_scenarios(print != 0); }

}  // extern "C"
