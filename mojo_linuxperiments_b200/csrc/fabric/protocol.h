// Collective schedules and the signalling convention shared by the host "threads as ranks" fabric and the
// GPU peer-memory kernels.  Everything here is plain arithmetic, usable from C++ and CUDA.
//
// Signals are monotonically increasing epochs, never reset: a waiter for epoch e proceeds when the word is
// >= e (wrap-safe signed comparison).  That keeps a launch replayable (CUDA graphs) without host clean-up.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define B200_HD __host__ __device__ __forceinline__
#else
#ifndef B200_HD
#define B200_HD inline
#endif
#endif

namespace b200 {

B200_HD bool epoch_reached(uint32_t seen, uint32_t target) { return static_cast<int32_t>(seen - target) >= 0; }

B200_HD bool is_pow2(int n) { return n > 0 && (n & (n - 1)) == 0; }
B200_HD int log2_floor(int n) { int l = 0; while ((1 << (l + 1)) <= n) ++l; return l; }

// chain reduce towards rank 0: rank r waits for rank r+1 (if any), adds its value, then signals rank r-1
B200_HD int chain_upstream(int rank, int world) { return rank + 1 < world ? rank + 1 : -1; }
B200_HD int chain_downstream(int rank) { return rank > 0 ? rank - 1 : -1; }

// butterfly (recursive doubling) all-reduce: in round k rank r exchanges with r ^ (1 << k)
B200_HD int butterfly_rounds(int world) { return log2_floor(world); }
B200_HD int butterfly_partner(int rank, int round) { return rank ^ (1 << round); }

// reduce-scatter / all-gather by rows: rank r owns rows [r*rows/world, (r+1)*rows/world)
B200_HD int shard_begin(int rank, int world, int rows) { return static_cast<int>(static_cast<long long>(rows) * rank / world); }
B200_HD int shard_end(int rank, int world, int rows) { return static_cast<int>(static_cast<long long>(rows) * (rank + 1) / world); }

// visiting order that starts at the local rank so local data is consumed while remote data is in flight
B200_HD int staggered_peer(int rank, int step, int world) { return (rank + step) % world; }

}  // namespace b200
