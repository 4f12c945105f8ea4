// NUMA-bound bump arena: one anonymous NORESERVE mapping bound (MPOL_BIND) to a node, optionally backed by
// transparent or explicit huge pages, carved up by a monotonically increasing offset.  Pages land on the node
// at first touch.  There is no per-object free; mark()/reset_to() give stack discipline.  Not thread safe.
// Capability parity: threading/numa_arena.mojo:6-140 of the reference.
#pragma once
#include <cstddef>
#include <cstdint>

#include "sys.hpp"

namespace hostrt {

// mmap + (madvise | MAP_HUGETLB) + mbind.  node < 0 skips the binding.  Returns nullptr on any failure.
// mapped_len (optional) receives the length actually mapped (size rounded up to the page size of the mode): the
// length munmap wants back.
void* mmap_numa(size_t size, int node, long page_size_mode = page_size::THP_2MB, long pr = prot::RW,
                size_t* mapped_len = nullptr);

class NumaArena {
 public:
  NumaArena(int node, size_t size, size_t alignment = 8, long page_size_mode = page_size::THP_2MB);
  NumaArena(const NumaArena&) = delete;
  NumaArena& operator=(const NumaArena&) = delete;
  NumaArena(NumaArena&& o) noexcept;
  ~NumaArena();

  explicit operator bool() const { return base_ != nullptr && size_ != 0; }
  // count * elem_size bytes aligned to the arena alignment, or nullptr when they do not fit
  void* alloc_bytes(size_t bytes);
  template <class T>
  T* alloc(size_t count) { return static_cast<T*>(alloc_bytes(count * sizeof(T))); }
  size_t mark() const { return offset_; }
  void reset_to(size_t watermark) { if (watermark <= offset_) offset_ = watermark; }   // only ever backwards
  void reset() { offset_ = 0; }
  size_t remaining() const { return size_ - offset_; }
  size_t used() const { return offset_; }
  size_t size() const { return size_; }
  size_t mapped_bytes() const { return mapped_; }
  void forget() { base_ = nullptr; size_ = 0; offset_ = 0; mapped_ = 0; }      // the caller unmapped the range itself
  int node() const { return node_; }
  void* base() const { return base_; }
  // True when nothing was allocated yet, or when the first page (if faulted in) lives on node().
  bool verify_placement() const;

 private:
  void* base_ = nullptr;
  size_t size_ = 0, offset_ = 0, alignment_ = 8;
  size_t mapped_ = 0;            // bytes the kernel mapped for this arena (>= size_)
  int node_ = -1;
};

}  // namespace hostrt
