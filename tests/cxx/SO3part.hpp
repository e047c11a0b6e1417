// Stand-in for the two GElib / cnine types that the binding include/SO3part_b200.cpp touches, so that its translation unit
// can be compiled and run without the cnine sources (an un-vendored submodule of GElib).  Only what that binding uses:
// arr, dims, strides (in elements), get_arr(), canonicalize_to_5d() (core/Gpart.hpp:450-469: (b, 2l+1, n) becomes
// (b, 1, 1, 2l+1, n) with zero strides on the inserted grid dimensions) and cnine::CoutLock.
#pragma once
#include <cuda_runtime.h>

#include <complex>
#include <iostream>
#include <stdexcept>
#include <vector>

namespace cnine {

struct CoutLock {};

template <class T>
struct TensorView {
  T* arr = nullptr;
  std::vector<int> dims;
  std::vector<long long> strides;
  T* get_arr() const { return arr; }
  static TensorView dense(T* p, const std::vector<int>& d) {
    TensorView v;
    v.arr = p;
    v.dims = d;
    v.strides.assign(d.size(), 1);
    for (int i = (int)d.size() - 2; i >= 0; i--) v.strides[i] = v.strides[i + 1] * d[i + 1];
    return v;
  }
  void to_5d() {
    while (dims.size() < 5) {
      dims.insert(dims.begin() + 1, 1);
      strides.insert(strides.begin() + 1, 0);
    }
  }
};

}  // namespace cnine

namespace GElib {

using namespace std;

template <class T>
struct SO3part : public cnine::TensorView<std::complex<T>> {
  SO3part() {}
  SO3part(const cnine::TensorView<std::complex<T>>& v) : cnine::TensorView<std::complex<T>>(v) {}
  void canonicalize_to_5d() { this->to_5d(); }
  static void canonicalize_to_5d(cnine::TensorView<T>& x) { x.to_5d(); }
};

}  // namespace GElib
