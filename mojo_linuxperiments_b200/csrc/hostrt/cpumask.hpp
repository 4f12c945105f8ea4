// Fixed-size CPU bitset with the memory layout of the kernel's cpu_set_t, so ptr() can be handed straight to
// sched_setaffinity.  Bytes = 128 covers 1,024 CPUs.  Out-of-range indices are ignored by set/clear and read
// as false by test.  Capability parity: numa/cpumask.mojo:4-61 of the reference.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <initializer_list>

namespace hostrt {

template <size_t Bytes = 128>
class CpuMask {
 public:
  static_assert(Bytes % 8 == 0, "mask size must be a multiple of 8 bytes (kernel reads unsigned longs)");
  CpuMask() { clear_all(); }
  static CpuMask from_cpu_list(const int* cpus, size_t n) {
    CpuMask m;
    for (size_t i = 0; i < n; ++i) m.set(cpus[i]);
    return m;
  }
  static CpuMask from_cpu_list(std::initializer_list<int> cpus) {
    CpuMask m;
    for (int c : cpus) m.set(c);
    return m;
  }
  static constexpr size_t byte_size() { return Bytes; }
  static constexpr size_t bit_capacity() { return Bytes * 8; }

  void set(long cpu) { if (in_range(cpu)) bits_[cpu >> 3] |= static_cast<uint8_t>(1u << (cpu & 7)); }
  void clear(long cpu) { if (in_range(cpu)) bits_[cpu >> 3] &= static_cast<uint8_t>(~(1u << (cpu & 7))); }
  bool test(long cpu) const { return in_range(cpu) && ((bits_[cpu >> 3] >> (cpu & 7)) & 1u); }
  void clear_all() { std::memset(bits_, 0, Bytes); }
  void set_all() { std::memset(bits_, 0xff, Bytes); }
  size_t count() const {
    size_t c = 0;
    for (size_t i = 0; i < Bytes; i += 8) {
      uint64_t w;
      std::memcpy(&w, bits_ + i, 8);
      c += static_cast<size_t>(__builtin_popcountll(w));
    }
    return c;
  }
  const uint8_t* ptr() const { return bits_; }
  uint8_t* ptr() { return bits_; }
  void copy_to(void* dst) const { std::memcpy(dst, bits_, Bytes); }
  bool operator==(const CpuMask& o) const { return std::memcmp(bits_, o.bits_, Bytes) == 0; }
  // index of the lowest set bit, or -1
  long first() const {
    for (size_t i = 0; i < Bytes * 8; ++i) if (test(static_cast<long>(i))) return static_cast<long>(i);
    return -1;
  }

 private:
  static bool in_range(long cpu) { return cpu >= 0 && static_cast<size_t>(cpu) < Bytes * 8; }
  alignas(8) uint8_t bits_[Bytes];
};

}  // namespace hostrt
