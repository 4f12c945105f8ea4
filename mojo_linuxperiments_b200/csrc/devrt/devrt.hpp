// Device runtime: the GPU-side counterparts of the host runtime's topology, mask and arena.
//
//   DeviceMask    <= 64 GPUs bitset (peer sets, rank groups)                  <-> CpuMask  (numa/cpumask.mojo)
//   GpuTopology   devices, SMs, HBM total/free, peer-access matrix, NVLink    <-> NumaInfo (numa/numa.mojo)
//                 P2P attributes, multicast (NVLS) support, PCI -> NUMA node
//   HbmArena      bump allocator over one VMM reservation on a GPU, same      <-> NumaArena (threading/numa_arena.mojo)
//                 alloc / mark / reset_to / reset / remaining / used /
//                 verify_placement contract; 2 MiB granularity plays THP
//
// The CUDA driver is loaded at run time (dlopen), so the library builds and loads on a machine without a GPU;
// every call then reports DEVRT_NO_DRIVER.  B200RT_LIBCUDA overrides the library path (tests point it at a
// host-memory stand-in).  Status convention as in the host runtime: >= 0 ok, negative = failure, never throw.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace devrt {

constexpr int DEVRT_NO_DRIVER = -1000;
constexpr int DEVRT_BAD_ARG = -22;
constexpr int DEVRT_NO_MEM = -12;

class DeviceMask {
 public:
  void set(int d) { if (ok(d)) bits_ |= (1ull << d); }
  void clear(int d) { if (ok(d)) bits_ &= ~(1ull << d); }
  bool test(int d) const { return ok(d) && ((bits_ >> d) & 1ull); }
  void clear_all() { bits_ = 0; }
  void set_first(int n) { bits_ = n >= 64 ? ~0ull : ((1ull << (n < 0 ? 0 : n)) - 1); }
  int count() const { return __builtin_popcountll(bits_); }
  uint64_t raw() const { return bits_; }
  static DeviceMask from_raw(uint64_t r) { DeviceMask m; m.bits_ = r; return m; }
 private:
  static bool ok(int d) { return d >= 0 && d < 64; }
  uint64_t bits_ = 0;
};

struct GpuInfo {
  int ordinal = -1;
  std::string name;
  int sm_count = 0, cc_major = 0, cc_minor = 0;
  size_t mem_total = 0, mem_free = 0;
  int multicast_supported = 0;     // NVLS-capable
  int vmm_supported = 0;
  std::string pci_bus_id;
  int numa_node = -1;              // host NUMA node of the PCI function, -1 unknown
};

class GpuTopology {
 public:
  GpuTopology();                   // queries every visible device
  int status() const { return status_; }
  int num_devices() const { return static_cast<int>(gpus_.size()); }
  const GpuInfo* gpu(int d) const { return d >= 0 && d < num_devices() ? &gpus_[d] : nullptr; }
  // 1 when `from` can map `to`'s memory; the diagonal is 1
  int peer_access(int from, int to) const;
  // NVLink "distance": 0 self, 1 peer with native atomics (NVLink / NVSwitch), 2 peer without, -1 no peer access
  int distance(int from, int to) const;
  DeviceMask peers_of(int d) const;
  bool fully_connected() const;
  std::string debug_string() const;
 private:
  int status_ = 0;
  std::vector<GpuInfo> gpus_;
  std::vector<int> access_, atomics_;
};

class HbmArena {
 public:
  // size is rounded up to the allocation granularity (2 MiB on current GPUs)
  HbmArena(int device, size_t size, size_t alignment = 256);
  HbmArena(const HbmArena&) = delete;
  HbmArena& operator=(const HbmArena&) = delete;
  ~HbmArena();
  explicit operator bool() const { return base_ != 0; }
  int status() const { return status_; }
  uint64_t alloc_bytes(size_t bytes);          // device address, 0 when it does not fit
  size_t mark() const { return offset_; }
  void reset_to(size_t w) { if (w <= offset_) offset_ = w; }
  void reset() { offset_ = 0; }
  size_t remaining() const { return size_ - offset_; }
  size_t used() const { return offset_; }
  size_t size() const { return size_; }
  size_t high_water() const { return high_; }
  uint64_t base() const { return base_; }
  int device() const { return device_; }
  bool verify_placement() const;                // the memory reports `device` as its ordinal
 private:
  uint64_t base_ = 0, handle_ = 0;
  size_t size_ = 0, offset_ = 0, alignment_ = 256, high_ = 0;
  int device_ = -1, status_ = 0;
};

// One rank's share of a symmetric heap, built on the virtual-memory API alone: an HBM block that can be handed to other
// processes as a POSIX file descriptor, and one address range of world x stride bytes in which this rank's block and,
// once their descriptors arrived, every peer's block are mapped at rank * stride.  peer_ptr(r) + off then addresses
// byte `off` of rank r's block from this GPU (NVLink peer access), with the same `off` on every rank - the GPU form
// of the reference's one shared arena that every worker addresses (test_linux_threading.mojo:426-435), bound to its
// owner like mbind binds an arena to a node (threading/numa_arena.mojo:93-137).  The descriptors travel between the
// rank processes over a unix socket (parallel/symm_native.py); nothing here talks to another process.
class SymmSegment {
 public:
  SymmSegment(int device, size_t bytes, int world, int rank);
  SymmSegment(const SymmSegment&) = delete;
  SymmSegment& operator=(const SymmSegment&) = delete;
  ~SymmSegment();
  explicit operator bool() const { return base_ != 0 && fd_ >= 0; }
  int status() const { return status_; }
  int export_fd() const { return fd_; }               // descriptor of this rank's block (owned by the caller's process)
  int map_peer(int peer, int fd);                     // 0, or a negative status
  uint64_t base() const { return base_; }
  size_t stride() const { return stride_; }
  uint64_t peer_ptr(int r) const { return base_ + stride_ * static_cast<size_t>(r); }
  bool mapped(int r) const { return r >= 0 && r < world_ && mapped_[r]; }
  // Multicast object (NVSwitch fans a store to mc_ptr() + off out to byte `off` of every rank's block; multimem loads
  // reduce over them).  Order across the ranks: rank 0 mc_create() -> descriptor; others mc_import(fd); all
  // mc_add_device(); barrier; all mc_bind(); barrier.  Each returns 0 (mc_create: the descriptor) or a negative status.
  int mc_create();
  int mc_import(int fd);
  int mc_add_device();
  int mc_bind();
  uint64_t mc_ptr() const { return mc_base_; }
 private:
  bool map_at(int r, uint64_t handle);
  uint64_t base_ = 0;
  size_t stride_ = 0, gran_ = 0;
  std::vector<uint64_t> handles_;
  std::vector<bool> mapped_;
  int device_ = -1, world_ = 0, rank_ = 0, fd_ = -1, status_ = 0;
  uint64_t mc_handle_ = 0, mc_base_ = 0;
  bool mc_bound_ = false;
};

}  // namespace devrt
