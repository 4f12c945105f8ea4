// Fixed-capacity heap array for move-only element types (pools, arenas): elements are move-constructed into
// raw storage, addressed by reference, destroyed in order, never copied or reallocated.
// Capability parity: notstdcollections/heap_move_array.mojo:5-58 of the reference.
#pragma once
#include <cstddef>
#include <cstdlib>
#include <new>
#include <utility>

namespace hostrt {

template <class T>
class HeapMoveArray {
 public:
  explicit HeapMoveArray(size_t capacity)
      : data_(capacity ? static_cast<T*>(::operator new(sizeof(T) * capacity, std::align_val_t(alignof(T)))) : nullptr),
        capacity_(capacity), len_(0) {}
  HeapMoveArray(const HeapMoveArray&) = delete;
  HeapMoveArray& operator=(const HeapMoveArray&) = delete;
  HeapMoveArray(HeapMoveArray&& o) noexcept : data_(o.data_), capacity_(o.capacity_), len_(o.len_) {
    o.data_ = nullptr; o.capacity_ = 0; o.len_ = 0;
  }
  ~HeapMoveArray() {
    for (size_t i = 0; i < len_; ++i) data_[i].~T();
    if (data_) ::operator delete(data_, std::align_val_t(alignof(T)));
  }
  // false (and the value is dropped) when the array is full
  bool push(T&& v) {
    if (len_ >= capacity_) return false;
    new (data_ + len_) T(std::move(v));
    ++len_;
    return true;
  }
  template <class... A>
  T* emplace(A&&... a) {
    if (len_ >= capacity_) return nullptr;
    T* p = new (data_ + len_) T(std::forward<A>(a)...);
    ++len_;
    return p;
  }
  T& operator[](size_t i) { return data_[i]; }
  const T& operator[](size_t i) const { return data_[i]; }
  T* at(size_t i) { return i < len_ ? data_ + i : nullptr; }
  size_t size() const { return len_; }
  size_t capacity() const { return capacity_; }
  T* begin() { return data_; }
  T* end() { return data_ + len_; }

 private:
  T* data_;
  size_t capacity_, len_;
};

}  // namespace hostrt
