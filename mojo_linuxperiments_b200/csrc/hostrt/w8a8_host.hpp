// W8A8 Hadamard linear on the host CPUs, parallelised over the pinned worker pools: the CPU point of the
// tensor-parallel linear benchmark and a bit-exact cross-check of the GPU kernels' integer arithmetic.
//
//   y[m,n] = bf16( (sum_k q[m,k] * wq[n,k])_int32 * sx[m] * sw[n] ),  (q, sx) = quantise(rotate(x[m,:]))
//
// rotate = block-128 Sylvester-Hadamard / sqrt(128) (seven butterfly stages, fp32), quantise = per-row symmetric int8
// (scale = max|.| / 127, 1 for an all-zero row; round to nearest even; clamp to [-127, 127]).  The integer dot products
// use AMX int8 tiles (tdpbssd, weights tile-loaded from their row-major layout) when the CPU and the kernel grant them,
// else AVX-512 VNNI (vpdpbusd on activations biased by +128, corrected with 128 * sum_k wq[n,k]), else plain scalar
// code; all three give the exact int32 result.  Work is split by output channel over one pinned
// worker per core of every NUMA node (the pool, arena and topology code of this directory; the reference's pool is
// threading/linux_threading.mojo:43-158).
#pragma once
#include <cstdint>

#include <vector>

#include "arena.hpp"
#include "heap_move_array.hpp"
#include "numa.hpp"
#include "team.hpp"

namespace hostrt {

struct W8A8HostResult {
  long status;          // 0 or -errno
  long quant_ns;        // rotate + quantise (all rows)
  long gemm_ns;         // integer GEMM + scale epilogue
  int workers;
  int used_vnni;        // 0 scalar, 1 AVX-512 VNNI, 2 AMX int8
};

// x: bf16 bits [M][K] (K % 128 == 0), wq: int8 [N][K], sw: fp32 [N], y: bf16 bits [M][N].
// q_out (int8 [M][K]), sx_out (fp32 [M]) and acc_out (int32 [M][N]) are optional.
W8A8HostResult w8a8_linear_host(const NumaInfo& info, const uint16_t* x, int M, int K, const int8_t* wq, const float* sw,
                                int N, uint16_t* y, int max_workers_per_node, int force_scalar, int8_t* q_out,
                                float* sx_out, int32_t* acc_out);

// int8 weights [N][K] placed where they are used: worker w of a team handles output channels
// [N*w/size, N*(w+1)/size), and those rows are copied into a NumaArena bound to that worker's node (one arena per
// node, threading/numa_arena.mojo:6-140 in the reference), so every worker streams node-local memory.
class NodeShardedWeights {
 public:
  NodeShardedWeights(const WorkerTeam& team, const int8_t* wq, int N, int K);
  explicit operator bool() const { return valid_; }
  int N() const { return N_; }
  int K() const { return K_; }
  // pointer p such that p + n*K is row n for every n of worker w's range
  const int8_t* base_for(int worker) const { return bases_[worker]; }
  int workers() const { return static_cast<int>(bases_.size()); }
  // shards whose first page is not on the node of the worker that reads them (-1: the kernel would not say)
  int misplaced() const;

 private:
  HeapMoveArray<NumaArena> arenas_;
  std::vector<const int8_t*> bases_;
  std::vector<const int8_t*> firsts_;
  std::vector<int> nodes_;
  int N_ = 0, K_ = 0;
  bool valid_ = false;
};

// The same over a team of parked workers (team.hpp): no thread is created or destroyed per call.
W8A8HostResult w8a8_linear_team(WorkerTeam& team, const uint16_t* x, int M, int K, const int8_t* wq, const float* sw, int N,
                                uint16_t* y, int force_scalar, int8_t* q_out, float* sx_out, int32_t* acc_out);
// ... with the weights taken from their node-local shards (wq of the other entry points is then unused)
W8A8HostResult w8a8_linear_team_sharded(WorkerTeam& team, const NodeShardedWeights& w, const uint16_t* x, int M, const float* sw,
                                        uint16_t* y, int force_scalar, int8_t* q_out, float* sx_out, int32_t* acc_out);

}  // namespace hostrt
