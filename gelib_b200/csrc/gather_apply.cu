// Two callers of the Clebsch-Gordan path that move or mix whole SO3parts:
//
//  * gather: r[.., t, ..] += sum over the sources s of target t of x[.., s, ..] along one array dimension of an
//    SO3partArr -- message passing over a gather map.  Replaces Gpart::add_gather / add_gather_back
//    (core/Gpart.hpp:555-561 of GElib), which hand the work to cnine::GatherSlices.  The map arrives as CSR (targets ->
//    sources) in device memory; one CTA sums the sources of one (outer index, target) without atomics.
//  * apply: r[cell] (+)= D x[cell] with D the (2l+1) x (2l+1) Wigner matrix of a rotation, the operation behind
//    SO3part.apply (python/src/gelib/SO3part.py:132-135, SO3/SO3irrep.hpp:65-103: the reference builds D on the host and
//    calls torch.matmul).  D is built on the host here too (it is 2l+1 squared numbers) and applied by one kernel.
#include <cmath>
#include <vector>

#include "plan.h"

namespace gelib_b200 {

namespace {

// r, x: [outer][n_out | n_in][inner] complex, dense
__global__ void __launch_bounds__(256) gather_kernel(float2* __restrict__ r, const float2* __restrict__ x, int n_out, int n_in,
                                                     long long inner, const int* __restrict__ row_ptr,
                                                     const int* __restrict__ col) {
  const int t = blockIdx.x;
  const long long o = blockIdx.y;
  const int s0 = row_ptr[t], s1 = row_ptr[t + 1];
  if (s0 == s1) return;
  float2* dst = r + (o * n_out + t) * inner;
  const float2* src = x + o * n_in * inner;
  for (long long e = (long long)blockIdx.z * blockDim.x + threadIdx.x; e < inner; e += (long long)gridDim.z * blockDim.x) {
    float2 acc = dst[e];
    for (int k = s0; k < s1; k++) {
      const float2 v = src[(long long)col[k] * inner + e];
      acc.x += v.x;
      acc.y += v.y;
    }
    dst[e] = acc;
  }
}

struct ApplyArgs {
  PartView r, x;
  CellGrid cg;
  const float2* D;  // [2l+1][2l+1], row-major
  int overwrite;
};

__global__ void __launch_bounds__(256) apply_kernel(const __grid_constant__ ApplyArgs A) {
  extern __shared__ float2 Ds[];
  const int L = 2 * A.x.l + 1, n = A.x.n;
  for (int e = threadIdx.x; e < L * L; e += blockDim.x) Ds[e] = A.D[e];
  __syncthreads();
  const long long cell = blockIdx.x;
  const float* xb = A.x.base + cell_offset(A.x, A.cg, cell);
  float* rb = A.r.base + cell_offset(A.r, A.cg, cell);
  for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < L * n; e += gridDim.y * blockDim.x) {
    const int m = e / n, ch = e - m * n;
    float sr = 0.f, si = 0.f;
    for (int k = 0; k < L; k++) {
      const float2 d = Ds[m * L + k];
      const float2 v = *reinterpret_cast<const float2*>(xb + (long long)k * A.x.sm + (long long)ch * A.x.sc);
      sr = fmaf(d.x, v.x, sr); sr = fmaf(-d.y, v.y, sr);
      si = fmaf(d.x, v.y, si); si = fmaf(d.y, v.x, si);
    }
    float* p = rb + (long long)m * A.r.sm + (long long)ch * A.r.sc;
    if (A.overwrite) {
      p[0] = sr; p[1] = si;
    } else {
      p[0] += sr; p[1] += si;
    }
  }
}

// Wigner's little d by the factorial sum (SO3/SO3irrep.hpp:80-103), in double.
double little_d(int l, int m1, int m2, double beta) {
  const double c = std::cos(beta / 2), s = std::sin(beta / 2);
  auto lf = [](int k) { return std::lgamma((double)k + 1.0); };
  const double pref = 0.5 * (lf(l + m1) + lf(l - m1) + lf(l + m2) + lf(l - m2));
  double x = 0.0;
  for (int k = std::max(0, m1 - m2); k <= std::min(l + m1, l - m2); k++) {
    const double lg = pref - (lf(l + m1 - k) + lf(k) + lf(m2 - m1 + k) + lf(l - m2 - k));
    const double term = std::exp(lg) * std::pow(c, 2 * l + m1 - m2 - 2 * k) * std::pow(s, m2 - m1 + 2 * k);
    x += ((m2 - m1 + k) & 1) ? -term : term;
  }
  return x;
}

}  // namespace

int launch_gather(float* r, const float* x, long long outer, int n_out, int n_in, long long inner, const int* row_ptr,
                  const int* col, cudaStream_t s) {
  static const char* fn = "add_gather";
  if (outer == 0 || n_out == 0 || inner == 0) return GELIB_OK;
  if (outer > 65535) return fail(GELIB_SKIPPED, fn, "more than 65535 outer slices");
  const unsigned gz = (unsigned)std::min<long long>(64, (inner + 255) / 256);
  gather_kernel<<<dim3((unsigned)n_out, (unsigned)outer, gz), 256, 0, s>>>(reinterpret_cast<float2*>(r),
                                                                         reinterpret_cast<const float2*>(x), n_out, n_in,
                                                                         inner, row_ptr, col);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "gather kernel launch");
  count_launch();
  return GELIB_OK;
}

int launch_apply(const PartView& r, const PartView& x, const CellGrid& cg, const float* D, int flags, cudaStream_t s) {
  static const char* fn = "SO3part_apply";
  if (cg.ncells == 0 || x.n == 0) return GELIB_OK;
  if (cg.ncells > 0x7fffffffLL) return fail(GELIB_SKIPPED, fn, "number of cells exceeds 2^31-1");
  ApplyArgs a;
  a.r = r;
  a.x = x;
  a.cg = cg;
  a.D = reinterpret_cast<const float2*>(D);
  a.overwrite = (flags & GELIB_OVERWRITE) ? 1 : 0;
  const int L = 2 * x.l + 1;
  const size_t smem = (size_t)L * L * sizeof(float2);
  if (smem > 48 * 1024) return fail(GELIB_SKIPPED, fn, "l too large for the shared-memory copy of D");
  const unsigned gy = (unsigned)std::min<long long>(64, ((long long)L * x.n + 255) / 256);
  apply_kernel<<<dim3((unsigned)cg.ncells, gy), 256, smem, s>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "apply kernel launch");
  count_launch();
  return GELIB_OK;
}

// D[m1+l][m2+l] = d^l_{m2 m1}(beta) e^{i m1 alpha} e^{i m2 gamma}  (SO3/SO3irrep.hpp:69-77); out: (2l+1)^2 x (re, im)
void wigner_D(int l, double alpha, double beta, double gamma, float* out) {
  const int L = 2 * l + 1;
  for (int m1 = -l; m1 <= l; m1++)
    for (int m2 = -l; m2 <= l; m2++) {
      const double d = little_d(l, m2, m1, beta), ph = m1 * alpha + m2 * gamma;
      out[2 * ((m1 + l) * L + (m2 + l))] = (float)(d * std::cos(ph));
      out[2 * ((m1 + l) * L + (m2 + l)) + 1] = (float)(d * std::sin(ph));
    }
}

}  // namespace gelib_b200
