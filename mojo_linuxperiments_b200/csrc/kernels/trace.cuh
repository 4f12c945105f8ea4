// In-kernel time stamps for overlap timelines (compiled in only with -DB200RT_TRACE: the production library has none).
//
// A stamped kernel calls B200_TRACE_INIT() at its top, B200_TRACE(kernel, phase) from one thread of a CTA at the points
// of interest and B200_TRACE_FLUSH(kernel) where it leaves; each stamp ends up as {%globaltimer, kernel, phase, SM id,
// CTA index, grid size} in a ring in device memory that the host handed over with b200_trace_set().  Read back, the ring shows for every launch when its CTAs started, when their inputs
// arrived, when the tensor core finished, when a peer's data landed: which part of a launch overlaps what.  The
// reference only prints topology (numa/numa.mojo:166-176); it has no timers.
//
// The ring pointer lives in a device variable of each translation unit (no relocatable device code is used), which the
// launch helper refreshes from the host-side state before a launch whenever b200_trace_set() changed it.  Set the ring
// before the warm-up run that precedes a CUDA-graph capture: the refresh is a synchronous copy and cannot be captured.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

enum TraceKernel : unsigned {
  TK_ACT_QUANT = 1, TK_GEMM_DECODE = 2, TK_GEMM_PREFILL = 3, TK_ROPE_KV = 4, TK_ATTN_DECODE = 5, TK_ATTN_PREFILL = 6,
  TK_PEER_ALLREDUCE = 7, TK_GEMM_TP = 8, TK_MOE = 9, TK_ARGMAX = 10,
};
// phases are free-form per kernel; by convention 0 = CTA started, 1 = dependency wait passed, 63 = CTA about to exit
enum TracePhase : unsigned { TP_START = 0, TP_DEPS = 1, TP_EXIT = 63 };

#ifdef B200RT_TRACE
struct TraceHostState { unsigned long long* buf; unsigned cap; unsigned gen; };
TraceHostState& trace_host_state();                        // trace.cu

static __device__ unsigned long long* g_trace_buf = nullptr;    // [0] = records written so far, records from [2]
static __device__ unsigned g_trace_cap = 0;

// Stamps are collected in shared memory while the CTA runs (a shared-memory atomic and two stores: tens of cycles) and
// written to the ring when the CTA leaves, so the round trips to global memory do not sit between the phases that are
// being timed.  Up to TRACE_MAX_LOCAL stamps per CTA; more are dropped.
constexpr unsigned TRACE_MAX_LOCAL = 24;
struct TraceLocal {
  unsigned n;
  unsigned phase[TRACE_MAX_LOCAL];
  unsigned long long t[TRACE_MAX_LOCAL];
};
__device__ __forceinline__ TraceLocal& trace_local() {
  __shared__ TraceLocal tl;
  return tl;
}
// one thread, before the first barrier of the kernel
__device__ __forceinline__ void trace_init() { trace_local().n = 0; }

__device__ __forceinline__ void trace_stamp(unsigned kernel, unsigned phase) {
  (void)kernel;
  if (!g_trace_buf) return;
  TraceLocal& tl = trace_local();
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  const unsigned i = atomicAdd(&tl.n, 1u);
  if (i < TRACE_MAX_LOCAL) { tl.t[i] = t; tl.phase[i] = phase; }
}

// one thread, after a barrier that follows the CTA's last stamp
__device__ __forceinline__ void trace_flush(unsigned kernel) {
  unsigned long long* b = g_trace_buf;
  if (!b) return;
  TraceLocal& tl = trace_local();
  const unsigned n = min(tl.n, TRACE_MAX_LOCAL);
  if (n == 0) return;
  const unsigned base = atomicAdd(reinterpret_cast<unsigned*>(b), n);
  unsigned smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const unsigned grid = gridDim.x * gridDim.y * gridDim.z;
  for (unsigned k = 0; k < n; ++k) {
    const unsigned i = base + k;
    if (i >= g_trace_cap) break;
    b[2 + 2 * static_cast<size_t>(i)] = tl.t[k];
    b[3 + 2 * static_cast<size_t>(i)] = (static_cast<unsigned long long>(kernel & 63u) << 58) | (static_cast<unsigned long long>(tl.phase[k] & 63u) << 52) |
                                        (static_cast<unsigned long long>(smid & 1023u) << 42) | (static_cast<unsigned long long>(cta & 0x1fffffu) << 21) |
                                        static_cast<unsigned long long>(grid & 0x1fffffu);
  }
  tl.n = 0;
}

// host: make this translation unit's device variables follow the ring the host set last
static inline void trace_refresh() {
  static unsigned seen = 0;
  TraceHostState& h = trace_host_state();
  if (seen != h.gen) {
    cudaMemcpyToSymbol(g_trace_buf, &h.buf, sizeof(h.buf));
    cudaMemcpyToSymbol(g_trace_cap, &h.cap, sizeof(h.cap));
    seen = h.gen;
  }
}
#define B200_TRACE(kernel, phase) ::b200::trace_stamp((kernel), (phase))
#define B200_TRACE_INIT() do { if (threadIdx.x == 0) ::b200::trace_init(); } while (0)
// every thread of the CTA calls this (it contains a barrier), at a point all of them reach
#define B200_TRACE_FLUSH(kernel) do { __syncthreads(); if (threadIdx.x == 0) ::b200::trace_flush(kernel); } while (0)
#else
static inline void trace_refresh() {}
#define B200_TRACE(kernel, phase) do { } while (0)
#define B200_TRACE_INIT() do { } while (0)
#define B200_TRACE_FLUSH(kernel) do { } while (0)
#endif

}  // namespace b200
