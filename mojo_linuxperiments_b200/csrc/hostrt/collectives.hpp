// Shared-memory collectives between pinned worker threads ("ranks"), one single-slot pool per rank, rank r
// placed on NUMA node nodes[r % num_nodes]:
//   chain_reduce        sum towards rank 0 through point-to-point gates      (reference: test:400-476)
//   butterfly_allreduce recursive doubling driven by the host, two fork-join phases per round (test:478-553)
//   fabric_allreduce    persistent workers, epoch-counted signal words, no host involvement between rounds:
//                       the protocol the GPU peer-memory kernels use, runnable under TSan on the host
// and the config-1 workload: per-node pinned workers fill node-local buffers from a counter RNG and the
// partial sums are tree-reduced to one value.
// Unlike the reference these run for any rank count >= 1 on any machine (ranks wrap around the nodes), and
// every wait is bounded.
#pragma once
#include <cstdint>

#include "numa.hpp"

namespace hostrt {

struct CollectiveResult {
  long status;        // 0 ok, negative errno-style failure (e.g. -ETIMEDOUT)
  int64_t value;      // chain: value on rank 0
};

CollectiveResult chain_reduce(const NumaInfo& info, int world, long timeout_ns);
// out[world] receives every rank's final value (all equal to world*(world+1)/2); world must be a power of two
long butterfly_allreduce(const NumaInfo& info, int world, int64_t* out, long timeout_ns);
// each rank contributes in[r]; out[r] = sum for every r; `rounds` repetitions reuse the same signal words
// (epochs keep increasing); drop_rank >= 0 makes that rank stay silent so the others time out (fault injection)
long fabric_allreduce(const NumaInfo& info, int world, const double* in, double* out, int rounds, long timeout_ns,
                      int drop_rank);

struct FillReduceResult {
  long status;
  double sum;
  long elapsed_ns;        // fill + reduce, measured on the orchestrator
  int workers;
  int nodes;
  int misplaced;          // workers that observed themselves or their buffer on the wrong node
};
// n_elems floats of uniform[-1,1) (Philox, keyed by global index) spread over all CPUs of all nodes
// The token-sharded all-gather / reduce-scatter protocol of the GPU kernels (epoch parity, per-block flags, done
// acknowledgements, owner-reset arrival counters) with threads as ranks and deliberate skew; *mismatches counts payload
// words that differ from their closed-form expectation.  0, or -ETIMEDOUT when a wait ran out.  mode: 1 all-gather only,
// 2 reduce-scatter only, 3 both in turn.  fault: 1 removes the wait for the done acknowledgements (harmless while every
// rank consumes every source each call, which is itself a barrier: the acknowledgements protect consumers that do not),
// 2 uses one buffer instead of two, which the harness must catch as mismatches.
long fabric_token_exchange(const NumaInfo& info, int world, int rows_per_rank, int blocks, int iters, long timeout_ns,
                           uint32_t skew_seed, int mode, int fault, int* mismatches);

FillReduceResult fill_reduce(const NumaInfo& info, uint64_t n_elems, uint64_t seed, int max_workers_per_node);
// single-threaded reference of the same sum (Kahan-free double accumulation in index order per chunk)
double fill_reduce_serial(uint64_t n_elems, uint64_t seed);

}  // namespace hostrt
