// Device side of the range-checked ("debug") build of the kernel library (-DB200RT_DEBUG; see fabric/range_check.h).
//
// B200_DBG_RANGE(off, len, status) is true when the access [off, off + len) into the symmetric heap may go ahead.  In
// the production build it is the constant true.  In the debug build it compares against the heap extent the host
// announced with b200_debug_set_heap_extent(); a violation is recorded once in the status block (word 1: code, words
// 2 and 3: the offset) and the caller skips the access - the kernel never traps and never touches the bad address.
// The extent lives in a device variable of each translation unit, refreshed by the launch helper like the trace ring.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "fabric/range_check.h"

namespace b200 {

#ifdef B200RT_DEBUG
struct DebugHostState { size_t heap_bytes; unsigned gen; };
DebugHostState& debug_host_state();                              // trace.cu

static __device__ size_t g_dbg_heap_bytes = 0;

__device__ __forceinline__ bool dbg_range(size_t off, size_t len, int* status) {
  if (range_ok(off, len, g_dbg_heap_bytes)) return true;
  if (status && atomicCAS(status + 1, 0, RC_OUT_OF_RANGE) == 0) {
    status[2] = static_cast<int>(off & 0xffffffffu);
    status[3] = static_cast<int>(static_cast<unsigned long long>(off) >> 32);
  }
  return false;
}

static inline void debug_refresh() {
  static unsigned seen = 0;
  DebugHostState& h = debug_host_state();
  if (seen != h.gen) {
    cudaMemcpyToSymbol(g_dbg_heap_bytes, &h.heap_bytes, sizeof(h.heap_bytes));
    seen = h.gen;
  }
}
#define B200_DBG_RANGE(off, len, status) ::b200::dbg_range((off), (len), (status))
#else
static inline void debug_refresh() {}
#define B200_DBG_RANGE(off, len, status) (true)
#endif

}  // namespace b200
