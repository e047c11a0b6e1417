// cuda/SO3part_b200.cpp  (replaces the four .cu files listed above)
#include "gelib_b200.h"
#include "SO3part.hpp"

namespace GElib {

  static gelib_tensor5 desc(const SO3part<float>& p) {          // complex view: float strides = 2 x complex strides
    gelib_tensor5 t;
    t.base = reinterpret_cast<float*>(p.get_arr());
    for (int i = 0; i < 5; i++) { t.dims[i] = p.dims[i]; t.strides[i] = 2 * (int64_t)p.strides[i]; }
    return t;
  }
  static gelib_tensor5 desc(const cnine::TensorView<float>& p) { // real view (spherical harmonics input)
    gelib_tensor5 t;
    t.base = p.get_arr();
    for (int i = 0; i < 5; i++) { t.dims[i] = p.dims[i]; t.strides[i] = p.strides[i]; }
    return t;
  }
  static void check(int status) {                                // GELIB_SKIP prints and returns; the rest throws
    if (status == GELIB_OK) return;
    if (status == GELIB_SKIPPED) { cnine::CoutLock lk; cerr << gelib_last_error() << endl; return; }
    throw std::runtime_error(gelib_last_error());
  }

  void SO3part_addCGproduct_cu(const SO3part<float>& r, const SO3part<float>& x, const SO3part<float>& y,
                               const int offs, const cudaStream_t& stream) {
    auto R = desc(r), X = desc(x), Y = desc(y);
    check(gelib_SO3part_addCGproduct(&R, &X, &Y, offs, 0, stream));
  }
  void SO3part_addCGproduct_back0_cu(const SO3part<float>& x, const SO3part<float>& r, const SO3part<float>& y,
                                     const int offs, const cudaStream_t& stream) {
    auto XG = desc(x), G = desc(r), Y = desc(y);
    check(gelib_SO3part_addCGproduct_back0(&XG, &G, &Y, offs, 0, stream));
  }
  void SO3part_addCGproduct_back1_cu(const SO3part<float>& y, const SO3part<float>& r, const SO3part<float>& x,
                                     const int offs, const cudaStream_t& stream) {
    auto YG = desc(y), G = desc(r), X = desc(x);
    check(gelib_SO3part_addCGproduct_back1(&YG, &G, &X, offs, 0, stream));
  }
  void addSPharm_cu(SO3part<float> r, cnine::TensorView<float> x, const cudaStream_t& stream) {
    r.canonicalize_to_5d();
    SO3part<float>::canonicalize_to_5d(x);
    auto R = desc(r), X = desc(x);
    check(gelib_SO3part_addSPharm(&R, &X, 0, stream));
  }

  // the three declarations that are commented out at SO3/SO3part.hpp:36-38 (uncomment them and the bodies of the
  // trampolines at SO3/SO3part.hpp:324-334, which are empty today, so Diag products on the GPU return zeros)
  void SO3part_addDiagCGproduct_cu(const SO3part<float>& r, const SO3part<float>& x, const SO3part<float>& y,
                                   const int offs, const cudaStream_t& stream) {
    auto R = desc(r), X = desc(x), Y = desc(y);
    check(gelib_SO3part_addDiagCGproduct(&R, &X, &Y, offs, 0, stream));
  }
  // _back0 / _back1: as above with gelib_SO3part_addDiagCGproduct_back0 / _back1; core/DiagCGproduct.hpp:81,102 pass
  // (r,x,y) for all three, so map (r,x,y) -> (xg = x, g = r, y) and (yg = y, g = r, x).
}
