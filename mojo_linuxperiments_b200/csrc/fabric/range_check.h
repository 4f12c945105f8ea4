// Range checks for accesses into a symmetric heap, shared by the CUDA kernels (debug build, -DB200RT_DEBUG) and plain
// C++ (where they are unit-tested with out-of-range offsets: nothing on a GPU is ever made to fault).
//
// The reference guards its slots with PROT_NONE pages (threading/linux_threading.mojo:148,419-420) and bounds-checks
// its containers in debug builds (notstdcollections/heap_move_array.mojo:21,26).  A peer-mapped HBM heap has no guard
// pages, and a stray store over NVLink lands in another GPU's memory, so the debug build checks every offset it is
// about to use against the extent of the heap; a violation is recorded (code, offset) and the access is skipped.
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define B200_RC_HD __host__ __device__ __forceinline__
#else
#define B200_RC_HD inline
#endif

namespace b200 {

// the access [off, off + len) lies inside a heap of `extent` bytes (extent 0: unknown, nothing is checked)
B200_RC_HD bool range_ok(size_t off, size_t len, size_t extent) {
  return extent == 0 || (len <= extent && off <= extent - len);
}

// What a violation leaves behind: word 0 the code (first violation wins), word 1 and 2 the offending offset.
constexpr int RC_OUT_OF_RANGE = 0x52430001;       // "RC" 1

struct RangeReport {
  int code;
  unsigned off_lo, off_hi;
};

// Host form of the record (the device form does the same with an atomic compare-and-swap on word 0).
B200_RC_HD bool range_check_record(size_t off, size_t len, size_t extent, RangeReport* rep) {
  if (range_ok(off, len, extent)) return true;
  if (rep && rep->code == 0) {
    rep->code = RC_OUT_OF_RANGE;
    rep->off_lo = static_cast<unsigned>(off & 0xffffffffu);
    rep->off_hi = static_cast<unsigned>(static_cast<unsigned long long>(off) >> 32);
  }
  return false;
}

}  // namespace b200
