// Locality query from inside a kernel: the GPU form of the reference's get_current_cpu_and_node / rseq fast path
// (numa/numa.mojo:6-24, threading/linux_threading.mojo:164-170).  Every CTA records which SM it runs on (%smid), how many
// SM ids the device exposes (%nsmid), the rank tag the host passed (the "node" a worker was asked to run on) and its own
// CTA index, so a test can check that work really landed where the launch said.
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace b200 {

__global__ void where_am_i_kernel(int* out, int n_slots, int rank_tag) {
  unsigned smid, nsmid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  asm volatile("mov.u32 %0, %%nsmid;" : "=r"(nsmid));
  if (threadIdx.x == 0 && static_cast<int>(blockIdx.x) < n_slots) {
    int* o = out + 4 * blockIdx.x;
    o[0] = static_cast<int>(smid);
    o[1] = static_cast<int>(nsmid);
    o[2] = rank_tag;
    o[3] = static_cast<int>(blockIdx.x);
  }
}

}  // namespace b200

// out: int32 [ctas][4] = {sm id, number of sm ids, rank_tag, cta index}
extern "C" int b200_where_am_i(int* out, int ctas, int rank_tag, cudaStream_t stream) {
  if (!out || ctas <= 0) return -1;
  b200::where_am_i_kernel<<<ctas, 32, 0, stream>>>(out, ctas, rank_tag);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
