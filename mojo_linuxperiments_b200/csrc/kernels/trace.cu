// Host side of the in-kernel time stamps (trace.cuh): where the ring lives and whether stamps are compiled in.
#include "trace.cuh"
#include "debug_check.cuh"
#include "api.h"

namespace b200 {
#ifdef B200RT_TRACE
TraceHostState& trace_host_state() {
  static TraceHostState s = {nullptr, 0u, 0u};
  return s;
}
#endif
#ifdef B200RT_DEBUG
DebugHostState& debug_host_state() {
  static DebugHostState s = {0, 0u};
  return s;
}
#endif
}  // namespace b200

// 1 when this library was built with -DB200RT_DEBUG (peer / heap accesses are range-checked), else 0.
extern "C" int b200_debug_compiled() {
#ifdef B200RT_DEBUG
  return 1;
#else
  return 0;
#endif
}

// Extent in bytes of the symmetric heap the peer kernels work on (0: unknown, nothing is checked).  Returns -1 when
// the checks are not compiled into this library.
extern "C" int b200_debug_set_heap_extent(size_t bytes) {
#ifdef B200RT_DEBUG
  b200::DebugHostState& s = b200::debug_host_state();
  s.heap_bytes = bytes;
  ++s.gen;
  return 0;
#else
  (void)bytes;
  return -1;
#endif
}

// 1 when this library was built with -DB200RT_TRACE (its kernels stamp), else 0.
extern "C" int b200_trace_compiled() {
#ifdef B200RT_TRACE
  return 1;
#else
  return 0;
#endif
}

// ring: device memory of (2 + 2 * capacity) uint64, zeroed by the caller; nullptr switches stamping off.
// Returns -1 when stamps are not compiled into this library.
extern "C" int b200_trace_set(void* ring, unsigned capacity) {
#ifdef B200RT_TRACE
  b200::TraceHostState& s = b200::trace_host_state();
  s.buf = static_cast<unsigned long long*>(ring);
  s.cap = ring ? capacity : 0u;
  ++s.gen;
  return 0;
#else
  (void)ring; (void)capacity;
  return -1;
#endif
}
