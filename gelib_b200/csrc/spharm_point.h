// Spherical harmonics Y_l^m, l = 0..lmax, of ONE 3-vector, written as rows of complex numbers: the same recursion
// and float/double mix as spharm.cu (SO3part::add_spharm, SO3/SO3part.hpp:355-394 of GElib, z-axis branch included),
// for kernels that generate the harmonics where they use them instead of reading them from memory.
// out[2 * (row0[l] + l + m) * pitch] receives (re, im) of Y_l^m; pitch in complex numbers.
#pragma once
#include <cuda_runtime.h>
#include <math.h>

namespace gelib_b200 {

constexpr int kSphPointMaxL = 16;

__device__ inline void spharm_point(float vx, float vy, float vz, int lmax, float* out, const int* row0, int pitch) {
  const float length = sqrtf(vx * vx + vy * vy + vz * vz);
  const float len2 = sqrtf(vx * vx + vy * vy);
  const bool degenerate = len2 == 0 || isnan(vx / len2) || isnan(vy / len2);
  float P[2][kSphPointMaxL + 1];
  for (int m = 0; m <= kSphPointMaxL; m++) P[0][m] = P[1][m] = 0.f;
  P[0][0] = 1.f;
  const float x = degenerate ? 0.f : vz / length;
  const float xfact = (float)sqrt(1.0 - x * x);
  const float cr = degenerate ? 0.f : vx / len2, ci = degenerate ? 0.f : vy / len2;
  for (int l = 0; l <= lmax; l++) {
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
    float* base = out + 2 * row0[l] * pitch;
    if (degenerate) {
      const float a = (float)sqrt(((float)(2 * l + 1)) / (M_PI * 4.0));
      for (int m = 0; m <= 2 * l; m++) {
        base[2 * m * pitch] = m == l ? a : 0.f;
        base[2 * m * pitch + 1] = 0.f;
      }
      continue;
    }
    float pr = (float)sqrt((2.0 * l + 1.0) / (M_PI * 4.0)), pi = 0.f;
    for (int m = 0; m <= l; m++) {
      const float ar = pr * cur[m], ai = pi * cur[m];
      base[2 * (l + m) * pitch] = ar;
      base[2 * (l + m) * pitch + 1] = ai;
      if (m > 0) {
        const float sgn = (float)(1 - 2 * (m % 2));
        base[2 * (l - m) * pitch] = sgn * ar;
        base[2 * (l - m) * pitch + 1] = sgn * (-ai);
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

}  // namespace gelib_b200
