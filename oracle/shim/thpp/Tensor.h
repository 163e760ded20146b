// Minimal stand-in for thpp::Tensor<T>, written for this repository so that the
// reference's CPU convolution (test/ReferenceConvolutions.cpp) can be compiled
// from where it lies without Torch7/thpp.  TEST INFRASTRUCTURE ONLY.
// Only the members that file uses are provided: brace construction from a size
// list, size(), ndims(), fill(), at({i,j,k,l}).
#pragma once
#include <cstddef>
#include <initializer_list>
#include <stdexcept>
#include <vector>

namespace thpp {

template <class T>
class Tensor {
 public:
  Tensor() = default;
  Tensor(std::initializer_list<long> sizes) : sizes_(sizes) { allocate(); }
  explicit Tensor(const std::vector<long>& sizes) : sizes_(sizes) { allocate(); }

  int ndims() const { return static_cast<int>(sizes_.size()); }
  long size(int d) const { return sizes_[d]; }
  long stride(int d) const { return strides_[d]; }
  void fill(T v) { for (auto& x : data_) x = v; }
  T* data() { return data_.data(); }
  const T* data() const { return data_.data(); }
  size_t numel() const { return data_.size(); }

  T& at(std::initializer_list<long> idx) { return data_[offset(idx)]; }
  const T& at(std::initializer_list<long> idx) const { return data_[offset(idx)]; }

 private:
  void allocate() {
    strides_.assign(sizes_.size(), 1);
    size_t n = 1;
    for (int d = static_cast<int>(sizes_.size()) - 1; d >= 0; --d) {
      strides_[d] = static_cast<long>(n);
      n *= static_cast<size_t>(sizes_[d]);
    }
    data_.assign(n, T(0));
  }
  size_t offset(std::initializer_list<long> idx) const {
    size_t off = 0;
    int d = 0;
    for (long i : idx) off += static_cast<size_t>(i) * strides_[d++];
    return off;
  }
  std::vector<long> sizes_, strides_;
  std::vector<T> data_;
};

}  // namespace thpp
