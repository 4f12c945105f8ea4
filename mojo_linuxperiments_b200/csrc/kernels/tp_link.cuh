// Shared descriptions of the two token-sharded ("sequence parallel") exchanges that the tensor-parallel prefill path
// fuses into its kernels.  Between transformer blocks every rank owns rows [rank*R, rank*R + R) of the token
// dimension (R = rows_per_rank); both exchanges move data with stores into the *receiver's* symmetric heap, so the
// bytes cross NVLink while the producing kernel is still computing, and neither contains a barrier.
//
//   all-gather of quantised activations (column-parallel linears; AgLink)
//     the activation prologue (act_quant.cu, PUSH form) rotates + quantises the R rows this rank owns and stores each
//     int8 row and its scale into every rank's gather buffer (one multimem.st per 16 bytes through the NVSwitch, or
//     world plain peer stores); when a 128-row block is complete it publishes flag[src][block] = epoch on every rank.
//     The consuming GEMM (w8a8_gemm_tp.cu, gather form) waits for the flags of the rows a tile needs just before its
//     TMA loads, and walks the token tiles starting with its own rows, so its main loop overlaps the arrival.
//
//   reduce-scatter of row-parallel partial sums (RsLink)
//     the GEMM (w8a8_gemm_tp.cu, scatter form) stores each finished bf16 tile straight into the receive slot
//     [source rank][local row][N] of the rank that owns those token rows and adds the row count to that rank's arrival
//     counter; it walks token tiles starting after its own rows so that all ranks' partials for a given owner are
//     produced at different times.  After its last tile every CTA waits (bounded) until the counter shows that all
//     world sources delivered all rows, then the grid sums the world slots in rank order into out[R, N].
//
// Both use two buffers selected by the parity of a device-resident epoch, so a rank that runs one call ahead never
// overwrites data a slower rank is still reading; the gather additionally waits for every consumer's "done" word of
// the call before last.  Epoch words live in device memory and are advanced by the kernels themselves, so captured
// launches replay without host involvement.
//
// Reference counterpart: none for the exchanges themselves.  The building blocks are the GPU forms of the reference's
// shared arena that every worker can address (test_linux_threading.mojo:426-435) and of its MutexGate latch
// (threading/linux_threading.mojo:174-198): stores into a peer's mapped memory, then an epoch flag the peer polls.
#pragma once
#include "peer.cuh"

namespace b200 {

struct AgLink {
  PeerTable t;
  size_t q_off[2];            // int8 [m_cap][K] rows indexed by global token row, per parity
  size_t s_off[2];            // fp32 [m_cap] per-token scales, per parity
  size_t flag_off;            // uint32 [world][blk_cap]: epoch of the last completed push of (source, 128-row block)
  size_t done_off;            // uint32 [world]: done[p] = last epoch rank p finished reading
  uint32_t* words;            // local: [0] completed epochs, [1] exit counter of the consumer
  uint32_t* row_ctr;          // local: uint32 [blk_cap] rows stored so far per block (zero between launches)
  int blk_cap;
  int rows_per_rank;          // R
  int* status;
  unsigned long long limit_ns;
};

struct RsLink {
  PeerTable t;
  size_t recv_off[2];         // bf16 [world][r_cap][N] per parity
  size_t ctr_off;             // uint32 [2] arrival counters (rows x column tiles), per parity
  uint32_t* words;            // local: [0] completed epochs, [1] exit counter
  int r_cap;
  int rows_per_rank;          // R
  int* status;
  unsigned long long limit_ns;
};

__device__ __forceinline__ void red_relaxed_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
// fence_proxy_async_all (ptx.cuh) orders generic-proxy observations (a flag another GPU wrote) before this thread's
// later TMA loads of global memory

}  // namespace b200
