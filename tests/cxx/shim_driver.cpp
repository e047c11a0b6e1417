// Calls the four reference-signature functions of the binding include/SO3part_b200.cpp (SO3/SO3part.hpp:33-39 of
// GElib) on dense device buffers, so that a test can drive them from Python through ctypes.
#include "SO3part.hpp"

namespace GElib {
void SO3part_addCGproduct_cu(const SO3part<float>& r, const SO3part<float>& x, const SO3part<float>& y, const int offs,
                             const cudaStream_t& stream);
void SO3part_addCGproduct_back0_cu(const SO3part<float>& x, const SO3part<float>& r, const SO3part<float>& y, const int offs,
                                   const cudaStream_t& stream);
void SO3part_addCGproduct_back1_cu(const SO3part<float>& y, const SO3part<float>& r, const SO3part<float>& x, const int offs,
                                   const cudaStream_t& stream);
void addSPharm_cu(SO3part<float> r, cnine::TensorView<float> x, const cudaStream_t& stream);
}  // namespace GElib

static GElib::SO3part<float> part5(void* p, int b, int l, int n) {
  GElib::SO3part<float> v(cnine::TensorView<std::complex<float>>::dense(static_cast<std::complex<float>*>(p), {b, 2 * l + 1, n}));
  v.canonicalize_to_5d();  // the dispatchers hand 5-D views to the device functions (core/CGproduct.hpp:54)
  return v;
}

// which: 0 forward (out r, a x, b y), 1 back0 (out xg, a g, b y), 2 back1 (out yg, a g, b x); returns 0, or 1 when the
// binding threw (message on stderr).
extern "C" int shim_product(int which, void* out, void* a, void* b, int batch, int lo, int no, int la, int na, int lb, int nb,
                            int offs) {
  try {
    auto O = part5(out, batch, lo, no), A = part5(a, batch, la, na), B = part5(b, batch, lb, nb);
    cudaStream_t s = 0;
    if (which == 0) GElib::SO3part_addCGproduct_cu(O, A, B, offs, s);
    else if (which == 1) GElib::SO3part_addCGproduct_back0_cu(O, A, B, offs, s);
    else GElib::SO3part_addCGproduct_back1_cu(O, A, B, offs, s);
    return cudaStreamSynchronize(s) == cudaSuccess ? 0 : 2;
  } catch (const std::exception& e) {
    std::cerr << e.what() << std::endl;
    return 1;
  }
}

// r (batch, 2l+1, n) += Y_l(x), x (batch, 3, n) real; 3-D views, as SO3part::add_spharm passes them (SO3/SO3part.hpp:399-401).
extern "C" int shim_spharm(void* r, void* x, int batch, int l, int n) {
  try {
    GElib::SO3part<float> R(cnine::TensorView<std::complex<float>>::dense(static_cast<std::complex<float>*>(r), {batch, 2 * l + 1, n}));
    auto X = cnine::TensorView<float>::dense(static_cast<float*>(x), {batch, 3, n});
    cudaStream_t s = 0;
    GElib::addSPharm_cu(R, X, s);
    return cudaStreamSynchronize(s) == cudaSuccess ? 0 : 2;
  } catch (const std::exception& e) {
    std::cerr << e.what() << std::endl;
    return 1;
  }
}
