// Spherical harmonics Y_L^m of 3-vectors, for one part or for every part of an SO3vec in one pass.
//
// Replaces add_spharm_kernel / addSPharm_cu (cuda/SPharm.cu:30-123 of GElib), which runs one CTA per
// cell with one thread per channel, keeps the Legendre triangle in shared memory and is launched once
// per L (so the recursion is redone for every L).  Here a thread owns one (cell, channel) point, keeps
// two levels of the associated-Legendre triangle in registers (loops fully unrolled up to the template
// cap), and emits every requested L while it walks the levels once.
//
// The arithmetic restates the CPU branch SO3part::add_spharm (SO3/SO3part.hpp:355-394), including its
// float/double mix -- the table entries are float, each recursion step is evaluated in double because
// of the literals 2.0*l-1.0, the factors (l+m-1) and (l-m) are cast to float first -- and its z-axis
// branch (vx = vy = 0 gives only the m = 0 entry, whatever the sign of vz).  This file is compiled
// without FMA contraction so the rounding points stay where the reference has them.
#include "plan.h"

namespace gelib_b200 {

namespace {

struct SphArgs {
  PartView r[kMaxParts];
  PartView x;        // real tensor: rows are the 3 coordinates, sc = channel stride in floats
  int part_of_l[65]; // index into r of level l, or -1
  int lmax;          // highest requested level
  int n;             // channels
  CellGrid cg;
  int accumulate;
};

__device__ __forceinline__ void emit(const SphArgs& A, const PartView& rp, long long cell, int ch, int L,
                                     const float* P, float cr, float ci) {
  // phase_0 = sqrt((2L+1)/4pi); phase_{m+1} = phase_m * cphi / sqrt((L-m)(L+m+1))   (SO3/SO3part.hpp:383-392)
  float* base = rp.base + cell_offset(rp, A.cg, cell) + (long long)ch * rp.sc;
  float pr = (float)sqrt((2.0 * L + 1.0) / (M_PI * 4.0)), pi = 0.f;
  const bool acc = A.accumulate != 0;
#pragma unroll
  for (int m = 0; m <= L; m++) {
    const float ar = pr * P[m], ai = pi * P[m];
    float2* p = reinterpret_cast<float2*>(base + (long long)(L + m) * rp.sm);
    float2 v = acc ? *p : make_float2(0.f, 0.f);
    v.x += ar;
    v.y += ai;
    *p = v;
    if (m > 0) {
      const float sgn = (float)(1 - 2 * (m % 2));
      float2* q = reinterpret_cast<float2*>(base + (long long)(L - m) * rp.sm);
      float2 w = acc ? *q : make_float2(0.f, 0.f);
      w.x += sgn * ar;
      w.y += sgn * (-ai);
      *q = w;
    }
    if (m < L) {
      const float d = sqrtf((float)(L - m) * (L + m + 1));
      const float qr = cr / d, qi = ci / d;
      const float nr = pr * qr - pi * qi, ni = pr * qi + pi * qr;
      pr = nr;
      pi = ni;
    }
  }
}

template <int LCAP>
__global__ void __launch_bounds__(128) spharm_kernel(const __grid_constant__ SphArgs A) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= A.cg.ncells * A.n) return;
  const long long cell = idx / A.n;
  const int ch = (int)(idx - cell * A.n);
  const float* xp = A.x.base + cell_offset(A.x, A.cg, cell) + (long long)ch * A.x.sc;
  const float vx = xp[0], vy = xp[A.x.sm], vz = xp[2 * A.x.sm];
  const float length = sqrtf(vx * vx + vy * vy + vz * vz);
  const float len2 = sqrtf(vx * vx + vy * vy);

  if (len2 == 0 || isnan(vx / len2) || isnan(vy / len2)) {  // SO3/SO3part.hpp:363-365
#pragma unroll
    for (int L = 0; L <= LCAP; L++) {
      if (L <= A.lmax && A.part_of_l[L] >= 0) {
        const PartView& rp = A.r[A.part_of_l[L]];
        float* p = rp.base + cell_offset(rp, A.cg, cell) + (long long)L * rp.sm + (long long)ch * rp.sc;
        const float a = (float)sqrt(((float)(2 * L + 1)) / (M_PI * 4.0));
        if (A.accumulate) {
          p[0] += a;
        } else {
          for (int m = 0; m <= 2 * L; m++) {
            float* q = rp.base + cell_offset(rp, A.cg, cell) + (long long)m * rp.sm + (long long)ch * rp.sc;
            q[0] = (m == L) ? a : 0.f;
            q[1] = 0.f;
          }
        }
      }
    }
    return;
  }

  const float x = vz / length;
  const float xfact = (float)sqrt(1.0 - x * x);
  const float cr = vx / len2, ci = vy / len2;
  float Pa[LCAP + 1], Pb[LCAP + 1];  // levels l-1 and l-2 (roles swap every level)
#pragma unroll
  for (int m = 0; m <= LCAP; m++) Pa[m] = Pb[m] = 0.f;
  Pa[0] = 1.f;
  if (A.part_of_l[0] >= 0) emit(A, A.r[A.part_of_l[0]], cell, ch, 0, Pa, cr, ci);
#pragma unroll
  for (int l = 1; l <= LCAP; l++) {
    if (l <= A.lmax) {
      // current level overwrites the l-2 array: prev = (l odd ? Pa : Pb), cur/prev2 = the other
      float* prev = (l & 1) ? Pa : Pb;
      float* cur = (l & 1) ? Pb : Pa;
      float nw[LCAP + 1];
#pragma unroll
      for (int m = 0; m <= LCAP; m++) nw[m] = 0.f;
      nw[l] = (float)(-(2.0 * l - 1.0) * xfact * prev[l - 1]);
      nw[l - 1] = (float)((2.0 * l - 1.0) * prev[l - 1] * x);
#pragma unroll
      for (int m = 0; m < l - 1; m++)
        nw[m] = (float)(((2.0 * l - 1.0) * prev[m] * x - ((float)(l + m - 1.0)) * (cur[m])) / ((float)(l - m)));
#pragma unroll
      for (int m = 0; m <= l; m++) cur[m] = nw[m];
      if (A.part_of_l[l] >= 0) emit(A, A.r[A.part_of_l[l]], cell, ch, l, cur, cr, ci);
    }
  }
}

// Same arithmetic for any l up to 64 with the two Legendre levels in local memory (runtime loops).
__global__ void __launch_bounds__(128) spharm_generic_kernel(const __grid_constant__ SphArgs A) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= A.cg.ncells * A.n) return;
  const long long cell = idx / A.n;
  const int ch = (int)(idx - cell * A.n);
  const float* xp = A.x.base + cell_offset(A.x, A.cg, cell) + (long long)ch * A.x.sc;
  const float vx = xp[0], vy = xp[A.x.sm], vz = xp[2 * A.x.sm];
  const float length = sqrtf(vx * vx + vy * vy + vz * vz);
  const float len2 = sqrtf(vx * vx + vy * vy);
  const bool degenerate = len2 == 0 || isnan(vx / len2) || isnan(vy / len2);
  float P[2][65];
  for (int m = 0; m < 65; m++) P[0][m] = P[1][m] = 0.f;
  P[0][0] = 1.f;
  const float x = degenerate ? 0.f : vz / length;
  const float xfact = (float)sqrt(1.0 - x * x);
  const float cr = degenerate ? 0.f : vx / len2, ci = degenerate ? 0.f : vy / len2;
  for (int l = 0; l <= A.lmax; l++) {
    float* cur = P[l & 1];
    if (l > 0 && !degenerate) {
      const float* prev = P[(l - 1) & 1];
      const float top = (float)(-(2.0 * l - 1.0) * xfact * prev[l - 1]);
      const float sub = (float)((2.0 * l - 1.0) * prev[l - 1] * x);
      for (int m = 0; m < l - 1; m++)
        cur[m] = (float)(((2.0 * l - 1.0) * prev[m] * x - ((float)(l + m - 1.0)) * (cur[m])) / ((float)(l - m)));
      cur[l] = top;
      cur[l - 1] = sub;
    }
    if (A.part_of_l[l] < 0) continue;
    const PartView& rp = A.r[A.part_of_l[l]];
    float* base = rp.base + cell_offset(rp, A.cg, cell) + (long long)ch * rp.sc;
    const bool acc = A.accumulate != 0;
    if (degenerate) {
      const float a = (float)sqrt(((float)(2 * l + 1)) / (M_PI * 4.0));
      for (int m = 0; m <= 2 * l; m++) {
        float* q = base + (long long)m * rp.sm;
        if (!acc) { q[0] = 0.f; q[1] = 0.f; }
        if (m == l) q[0] += a;
      }
      continue;
    }
    float pr = (float)sqrt((2.0 * l + 1.0) / (M_PI * 4.0)), pi = 0.f;
    for (int m = 0; m <= l; m++) {
      const float ar = pr * cur[m], ai = pi * cur[m];
      float* p = base + (long long)(l + m) * rp.sm;
      if (acc) { p[0] += ar; p[1] += ai; } else { p[0] = ar; p[1] = ai; }
      if (m > 0) {
        const float sgn = (float)(1 - 2 * (m % 2));
        float* q = base + (long long)(l - m) * rp.sm;
        if (acc) { q[0] += sgn * ar; q[1] += sgn * (-ai); } else { q[0] = sgn * ar; q[1] = sgn * (-ai); }
      }
      if (m < l) {
        const float d = sqrtf((float)(l - m) * (l + m + 1));
        const float qr = cr / d, qi = ci / d;
        const float nr = pr * qr - pi * qi, ni = pr * qi + pi * qr;
        pr = nr;
        pi = ni;
      }
    }
  }
}

}  // namespace

int launch_spharm(const std::vector<PartView>& r, const PartView& x, const CellGrid& cg, int flags, cudaStream_t s) {
  static const char* fn = "addSPharm";
  SphArgs a;
  for (int l = 0; l < 65; l++) a.part_of_l[l] = -1;
  a.lmax = 0;
  for (size_t i = 0; i < r.size(); i++) {
    if (r[i].l > 64) return fail(GELIB_SKIPPED, fn, "l exceeds 64");
    a.r[i] = r[i];
    a.part_of_l[r[i].l] = (int)i;
    a.lmax = std::max(a.lmax, r[i].l);
  }
  a.x = x;
  a.n = x.n;
  a.cg = cg;
  a.accumulate = (flags & GELIB_OVERWRITE) ? 0 : 1;
  const long long total = cg.ncells * (long long)x.n;
  if (total == 0 || r.empty()) return GELIB_OK;
  const long long blocks = (total + 127) / 128;
  if (blocks > 0x7fffffffLL) return fail(GELIB_SKIPPED, fn, "number of points exceeds 2^38");
  if (a.lmax <= 4) spharm_kernel<4><<<(unsigned)blocks, 128, 0, s>>>(a);
  else if (a.lmax <= 8) spharm_kernel<8><<<(unsigned)blocks, 128, 0, s>>>(a);
  else if (a.lmax <= 12) spharm_kernel<12><<<(unsigned)blocks, 128, 0, s>>>(a);
  else spharm_generic_kernel<<<(unsigned)blocks, 128, 0, s>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "spherical harmonics kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
