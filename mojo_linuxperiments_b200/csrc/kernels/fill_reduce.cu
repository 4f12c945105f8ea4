// Config-1 workload on the GPU: fill a float32 buffer with uniform[-1,1) values of a counter-based generator keyed on
// the *global* element index (any split of the index space over GPUs produces the same elements), and reduce them.
//   fill_uniform_reduce   grid-stride fill (16-byte stores) with per-thread double accumulation, warp shuffle and
//                         shared-memory block reduction, one double per CTA; the last CTA to finish adds the CTA
//                         partials (exact in double, so any order gives the same bits) into the result
// The op is bound by the 4 bytes per element written to HBM; Philox costs ~25 integer ops per element.
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"
#include "fabric/philox.h"

namespace b200 {

__global__ void __launch_bounds__(256) fill_uniform_reduce_kernel(float* out, unsigned long long begin,
                                                                  unsigned long long end, unsigned long long seed,
                                                                  double* partials, unsigned* counter,
                                                                  double* result) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  __shared__ double red[8];
  __shared__ int last;
  // work in whole Philox blocks of four elements; `begin` is a multiple of 4 (checked on the host)
  const unsigned long long nblk = (end - begin + 3) / 4;
  // Every value is k * 2^-23 - 1 with a 24-bit integer k, so the sum is accumulated exactly in integers (cheap) and
  // converted once: sum = 2^-23 * sum(k) - count.  The result does not depend on how the index space is split.
  unsigned long long ksum = 0, cnt = 0;
  for (unsigned long long b = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; b < nblk;
       b += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
    const unsigned long long i = begin + 4 * b;
    const Philox4 r = philox4x32_10(i >> 2, seed);
    float4 v;
    v.x = u32_to_uniform_pm1(r.v[0]); v.y = u32_to_uniform_pm1(r.v[1]);
    v.z = u32_to_uniform_pm1(r.v[2]); v.w = u32_to_uniform_pm1(r.v[3]);
    if (i + 4 <= end) {
      *reinterpret_cast<float4*>(out + (i - begin)) = v;
      ksum += static_cast<unsigned long long>((r.v[0] >> 8) + (r.v[1] >> 8)) + ((r.v[2] >> 8) + (r.v[3] >> 8));
      cnt += 4;
    } else {
      const float e[4] = {v.x, v.y, v.z, v.w};
      for (int k = 0; k < 4 && i + k < end; ++k) { out[i - begin + k] = e[k]; ksum += r.v[k] >> 8; ++cnt; }
    }
  }
  double s = static_cast<double>(ksum) * (2.0 / 16777216.0) - static_cast<double>(cnt);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < 8; ++w) t += red[w];
    partials[blockIdx.x] = t;
    __threadfence();
    const unsigned old = atomicAdd(counter, 1u);
    last = (old == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (last) {
    // The CTA partials are integer multiples of 2^-23 far below 2^53 in magnitude, so their double sum is exact and
    // does not depend on the order: the whole CTA adds them (one thread walking a thousand L2 loads one by one
    // cost several microseconds of a 40 us kernel).
    __threadfence();
    double t = 0.0;
    for (unsigned c = threadIdx.x; c < gridDim.x; c += blockDim.x) t += *reinterpret_cast<volatile double*>(partials + c);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    __syncthreads();                       // red[] of the first reduction has been read
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = t;
    __syncthreads();
    if (threadIdx.x == 0) {
      double r = 0.0;
      for (int w = 0; w < 8; ++w) r += red[w];
      *result = r;
      *counter = 0;
    }
  }
}

}  // namespace b200

using namespace b200;

// out: float[end - begin]; partials: double[max_ctas]; counter: zeroed unsigned; result: double
extern "C" int b200_fill_uniform_reduce(float* out, unsigned long long begin, unsigned long long end, unsigned long long seed,
                                        double* partials, int max_ctas, unsigned* counter, double* result, cudaStream_t stream) {
  if (end <= begin || (begin & 3) || (reinterpret_cast<uintptr_t>(out) & 15) || max_ctas < 1) return -1;
  const unsigned long long nblk = (end - begin + 3) / 4;
  long long ctas = static_cast<long long>((nblk + 255) / 256);
  if (ctas > max_ctas) ctas = max_ctas;
  launch_ex(fill_uniform_reduce_kernel, dim3(static_cast<int>(ctas)), dim3(256), 0, stream, 0, out, begin, end, seed, partials, counter, result);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
