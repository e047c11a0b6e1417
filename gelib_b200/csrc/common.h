// Internal declarations shared by the kernels, the plan cache and the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/gelib_b200.h"

namespace gelib_b200 {

// ---- device-side views ------------------------------------------------------------------------------

// One SO3part in 5-D canonical form as a kernel sees it.  Strides are in floats.  The fast
// kernels need sc == 2 (channels dense); the strided fallbacks take any sc.
struct PartView {
  float* base;
  long long sb, sg0, sg1;  // batch / grid strides, 0 = broadcast
  long long sm;            // stride between m rows
  long long sc;            // stride between channels
  int n;                   // channels
  int l;
};

constexpr int kMaxParts = GELIB_MAX_PARTS;

// The cells of a call: (b, g0, g1) flattened, g1 fastest.
struct CellGrid {
  int B, G0, G1;
  long long ncells;
};

__host__ __device__ inline long long cell_offset(const PartView& p, const CellGrid& cg, long long cell) {
  if (cg.G0 == 1 && cg.G1 == 1) return cell * p.sb;  // plain SO3parts: no grid
  if (cg.ncells < 0x7fffffffLL) {                     // 32-bit division is several times cheaper
    const unsigned c = (unsigned)cell;
    const unsigned g1 = c % (unsigned)cg.G1, t = c / (unsigned)cg.G1;
    const unsigned g0 = t % (unsigned)cg.G0, b = t / (unsigned)cg.G0;
    return (long long)b * p.sb + (long long)g0 * p.sg0 + (long long)g1 * p.sg1;
  }
  const int g1 = (int)(cell % cg.G1);
  const long long t = cell / cg.G1;
  const int g0 = (int)(t % cg.G0);
  const long long b = t / cg.G0;
  return b * p.sb + (long long)g0 * p.sg0 + (long long)g1 * p.sg1;
}

#ifdef __CUDACC__
// Float offsets of the CTA's cells into every part of one vector, computed once so that no inner loop
// divides: dst[c * kMaxParts + part] for the cells cell0 .. cell0 + WC - 1.
__device__ __forceinline__ void fill_cell_offsets(long long* dst, const PartView* parts, int nparts,
                                                  const CellGrid& cg, long long cell0, int WC) {
  for (int e = threadIdx.x; e < WC * nparts; e += blockDim.x) {
    const int c = e / nparts, p = e - c * nparts;
    const long long cell = cell0 + c;
    dst[c * kMaxParts + p] = cell < cg.ncells ? cell_offset(parts[p], cg, cell) : 0;
  }
}
#endif

// One (l1,l2)->l term of a product.  xi/yi/ri index the part arrays of the call, offs is the first
// output channel of the term inside part ri, coff the offset of its band coefficients in the plan's
// coefficient table (band order: m ascending, then m1 ascending).
struct Triple {
  short l1, l2, l;
  short xi, yi, ri;
  int offs;
  int coff;
};

// ---- host-side plan -------------------------------------------------------------------------------------

struct PartSig {
  int l, n;
};

// What a vector-level product needs besides the tensors: built once per signature, cached per device.
struct Schedule {
  std::vector<Triple> triples;
  std::vector<float> coeffs;  // band coefficients of all triples, concatenated
};

// Triple walk of Gvec::add_CGproduct (l1 ascending, l2 ascending, l ascending, running offsets).
// Parts must be given in ascending l.  Fills band coefficients when with_coeffs is set.
void build_schedule(const std::vector<PartSig>& x, const std::vector<PartSig>& y, const std::vector<PartSig>& r,
                    bool diag, bool with_coeffs, Schedule* out);

double cg_coefficient(int l1, int l2, int l, int m1, int m2);
int band_size(int l1, int l2, int l);  // number of (m1,m2) with |m1|<=l1, |m2|<=l2, |m1+m2|<=l

// Device-resident copy of a plan's tables.  Owned by the per-device cache; never freed before exit.
struct DevicePlan {
  Triple* triples = nullptr;
  float* coeffs = nullptr;
  int4* items = nullptr;   // kernel-specific work list
  int* jobs = nullptr;     // job j covers items [jobs[j], jobs[j+1])
  float* floats = nullptr; // kernel-specific float table (16-byte aligned)
  int ntriples = 0, nitems = 0, njobs = 0;
  std::vector<int4> h_items;
  std::vector<int> h_jobs;
  std::vector<float> h_floats;
  Schedule sched;
};

// ---- error plumbing ---------------------------------------------------------------------------------------

void set_error(const std::string& msg);
int fail(int status, const char* fn, const std::string& msg);  // records "<fn> skipped: <msg>." and returns status
int check_cuda(cudaError_t e, const char* fn, const char* what);
void count_launch(int n = 1);

#define GELIB_CUDA_TRY(fn, expr)                                  \
  do {                                                            \
    cudaError_t _e = (expr);                                      \
    if (_e != cudaSuccess) return check_cuda(_e, fn, #expr);      \
  } while (0)

}  // namespace gelib_b200
