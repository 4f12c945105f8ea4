#include "arena.hpp"

namespace hostrt {

void* mmap_numa(size_t size, int node, long page_size_mode, long pr, size_t* mapped_len) {
  if (mapped_len) *mapped_len = 0;
  if (size == 0) return nullptr;
  long flags = map_flag::PRIVATE | map_flag::ANONYMOUS | map_flag::NORESERVE;
  size_t len = size;
  if (page_size_mode == page_size::EXPLICIT_2MB) { flags |= map_flag::HUGETLB | map_flag::HUGE_2MB; len = align_up(size, 2u << 20); }
  else if (page_size_mode == page_size::EXPLICIT_1GB) { flags |= map_flag::HUGETLB | map_flag::HUGE_1GB; len = align_up(size, 1u << 30); }
  else len = align_up(size, static_cast<size_t>(page_size::STANDARD));
  const long r = sys_mmap(nullptr, len, pr, flags);
  if (r < 0 && r > -4096) return nullptr;
  void* p = reinterpret_cast<void*>(r);
  if (page_size_mode == page_size::THP_2MB) sys_madvise(p, len, madv::HUGEPAGE);   // advisory: failure is fine
  if (node >= 0) {
    uint64_t mask[16] = {0};                 // up to 1,024 nodes
    if (node >= 1024) { sys_munmap(p, len); return nullptr; }
    mask[node >> 6] = 1ull << (node & 63);
    if (sys_mbind(p, len, mempolicy::BIND, mask, 1025) < 0) { sys_munmap(p, len); return nullptr; }
  }
  if (mapped_len) *mapped_len = len;
  return p;
}

NumaArena::NumaArena(int node, size_t size, size_t alignment, long page_size_mode)
    : alignment_(alignment ? alignment : 1), node_(node) {
  base_ = mmap_numa(size, node, page_size_mode, prot::RW, &mapped_);
  size_ = base_ ? size : 0;
}
NumaArena::NumaArena(NumaArena&& o) noexcept
    : base_(o.base_), size_(o.size_), offset_(o.offset_), alignment_(o.alignment_), mapped_(o.mapped_), node_(o.node_) {
  o.base_ = nullptr; o.size_ = 0; o.offset_ = 0; o.mapped_ = 0;
}
NumaArena::~NumaArena() {
  // exactly the length that was mapped: a hugetlb mapping was rounded up to its page size and munmap of any other
  // length fails with EINVAL, which would leak the reserved huge pages
  if (base_) sys_munmap(base_, mapped_);
}
void* NumaArena::alloc_bytes(size_t bytes) {
  if (!base_) return nullptr;
  const size_t start = align_up(offset_, alignment_);
  if (start > size_ || bytes > size_ - start) return nullptr;
  offset_ = start + bytes;
  return static_cast<uint8_t*>(base_) + start;
}
bool NumaArena::verify_placement() const {
  if (!base_) return false;
  if (offset_ == 0) return true;
  const long n = sys_move_pages_query(base_);
  if (n == -err::kNOENT) return true;          // nothing faulted in yet
  return node_ < 0 ? n >= 0 : n == node_;
}

}  // namespace hostrt
