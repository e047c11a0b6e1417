/*
 * CPU oracle for the Clebsch-Gordan hot path of GElib.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA kernels are
 * compared against and the timed CPU baseline of the benchmark; it is never linked
 * into, imported by or called from the shipped library.
 *
 * It restates, in plain C and without the cnine tensor library, the arithmetic of the
 * reference's CPU path (paths are relative to the GElib source tree):
 *
 *   SO3/SO3CGbank.hpp:58-95     Clebsch-Gordan coefficient (Racah sum in log-gamma form)
 *   SO3/SO3part.hpp:205-257     CG product forward / back0 / back1 per-cell loops
 *   SO3/SO3part.hpp:276-322     diagonal CG product forward / back0 / back1
 *   SO3/SO3part.hpp:340-397     spherical harmonics (incl. the degenerate z-axis branch)
 *   core/Gpart.hpp:168-185      batch broadcasting (batch 1 <-> stride 0)
 *
 * Faithfulness notes.  The reference keeps tensors as complex<float>, the coefficient
 * matrix as float, and accumulates with `inc` (+=) in float in the loop order
 * n1, n2, m1, m2.  The same order and the same float rounding points are kept here and
 * the file is compiled with -ffp-contract=off so no product is fused into an FMA
 * (the reference's default x86-64 build has no FMA either).  The batch loop may be
 * spread over OpenMP threads; cells are independent so results do not depend on the
 * thread count.
 *
 * Parity pins (see tests/): the (1,2,2) coefficient matrix printed in
 * python/docs/source/SO3CG.rst:49-53, sympy's Clebsch-Gordan coefficients, scipy's
 * sph_harm_y, and the Diag-is-the-diagonal-of-Full identity shown in
 * python/docs/source/SO3partB.rst:136-138,177-179.
 *
 * Layout of every complex tensor argument: dense row-major (batch, 2l+1, n) with
 * interleaved (re,im) floats.  A tensor whose batch size is 1 while the call's batch is
 * B > 1 is broadcast (forward) or receives the sum over the batch (backward), as the
 * reference's stride-0 promotion does.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#ifndef M_PI
#define M_PI 3.14159265358979323846
#endif

/* ---- coefficients: SO3/SO3CGbank.hpp:67-95 -------------------------------------- */

static double logfact(double n) { return lgamma(n + 1); }           /* :67-69 */
static double plusminus(int k) { return (k % 2 == 1) ? -1 : +1; }    /* :71    */

/* SO3CGbank::slowCG, SO3/SO3CGbank.hpp:73-95 */
double oracle_cg_coeff(int l1, int l2, int l, int m1, int m2) {
  int m = m1 + m2;
  int m3 = -m;
  int t1 = l2 - m1 - l;
  int t2 = l1 + m2 - l;
  int t3 = l1 + l2 - l;
  int t4 = l1 - m1;
  int t5 = l2 + m2;
  int tmin = t1 > t2 ? t1 : t2; if (tmin < 0) tmin = 0;
  int tmax = t4 < t5 ? t4 : t5; if (t3 < tmax) tmax = t3;

  double logA = (logfact(l1 + l2 - l) + logfact(l1 - l2 + l) + logfact(-l1 + l2 + l) -
                 logfact(l1 + l2 + l + 1)) / 2;
  logA += (logfact(l1 + m1) + logfact(l1 - m1) + logfact(l2 + m2) + logfact(l2 - m2) +
           logfact(l + m3) + logfact(l - m3)) / 2;

  double wigner = 0;
  for (int t = tmin; t <= tmax; t++) {
    double logB = logfact(t) + logfact(t - t1) + logfact(t - t2) + logfact(t3 - t) +
                  logfact(t4 - t) + logfact(t5 - t);
    wigner += plusminus(t) * exp(logA - logB);
  }
  return plusminus(l1 - l2 - m3) * plusminus(l1 - l2 + m) * sqrt((double)(2 * l + 1)) * wigner;
}

/* SO3CGbank::CGmatrix, SO3/SO3CGbank.hpp:58-65: (2l1+1) x (2l2+1) floats, zero off the band. */
void oracle_cg_matrix(int l1, int l2, int l, float* C) {
  int L2 = 2 * l2 + 1;
  memset(C, 0, sizeof(float) * (size_t)(2 * l1 + 1) * L2);
  for (int m1 = -l1; m1 <= l1; m1++) {
    int lo = -l2 > -l - m1 ? -l2 : -l - m1;
    int hi = l2 < l - m1 ? l2 : l - m1;
    for (int m2 = lo; m2 <= hi; m2++)
      C[(m1 + l1) * L2 + (m2 + l2)] = (float)oracle_cg_coeff(l1, l2, l, m1, m2);
  }
}

/* ---- helpers --------------------------------------------------------------------- */

static int imax(int a, int b) { return a > b ? a : b; }
static int imin(int a, int b) { return a < b ? a : b; }

static int set_threads(int nthreads) {
#ifdef _OPENMP
  if (nthreads <= 0) nthreads = omp_get_max_threads();
  return nthreads;
#else
  (void)nthreads;
  return 1;
#endif
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* complex<float> helpers that round exactly where std::complex<float> arithmetic does */
typedef struct { float re, im; } cf;
static inline cf cmulf(cf a, cf b) {
  cf r; r.re = a.re * b.re - a.im * b.im; r.im = a.re * b.im + a.im * b.re; return r;
}
static inline cf cscale(float c, cf a) { cf r; r.re = c * a.re; r.im = c * a.im; return r; }
static inline cf cconj(cf a) { cf r; r.re = a.re; r.im = -a.im; return r; }

/* ---- CG product, one (l1,l2,l) triple -------------------------------------------- */
/*
 * Arguments shared by the six product routines:
 *   B            number of cells (batch elements) of the call
 *   rB,xB,yB     batch sizes of the three tensors: each is B or 1 (1 = broadcast)
 *   NR           channel count of r/g rows;  offs = first output channel of this triple
 * mode 0: r += C x y      (SO3part::add_CGproduct_kernel,       SO3/SO3part.hpp:205-221)
 * mode 1: x += C r conj y (SO3part::add_CGproduct_back0_kernel, SO3/SO3part.hpp:223-239)
 * mode 2: y += C r conj x (SO3part::add_CGproduct_back1_kernel, SO3/SO3part.hpp:241-257)
 * diag != 0 selects the diagonal variants (SO3/SO3part.hpp:276-322): n1 == n2 == n and the
 * output channel is offs+n.
 */
static void cg_cell(int mode, int diag, cf* r, cf* x, cf* y, const float* C, int l1, int l2,
                    int l, int N1, int N2, int NR, int offs) {
  const int L2 = 2 * l2 + 1;
  if (!diag) {
    for (int n1 = 0; n1 < N1; n1++) {
      for (int n2 = 0; n2 < N2; n2++) {
        for (int m1 = -l1; m1 <= l1; m1++) {
          for (int m2 = imax(-l2, -l - m1); m2 <= imin(l2, l - m1); m2++) {
            float c = C[(m1 + l1) * L2 + (m2 + l2)];
            cf* rp = &r[(size_t)(m1 + m2 + l) * NR + offs + n2];
            cf* xp = &x[(size_t)(m1 + l1) * N1 + n1];
            cf* yp = &y[(size_t)(m2 + l2) * N2 + n2];
            cf t;
            if (mode == 0) { t = cmulf(cscale(c, *xp), *yp); rp->re += t.re; rp->im += t.im; }
            else if (mode == 1) { t = cmulf(cscale(c, *rp), cconj(*yp)); xp->re += t.re; xp->im += t.im; }
            else { t = cmulf(cscale(c, *rp), cconj(*xp)); yp->re += t.re; yp->im += t.im; }
          }
        }
      }
      offs += N2;
    }
  } else {
    for (int n = 0; n < N1; n++) {
      for (int m1 = -l1; m1 <= l1; m1++) {
        for (int m2 = imax(-l2, -l - m1); m2 <= imin(l2, l - m1); m2++) {
          float c = C[(m1 + l1) * L2 + (m2 + l2)];
          cf* rp = &r[(size_t)(m1 + m2 + l) * NR + offs + n];
          cf* xp = &x[(size_t)(m1 + l1) * N1 + n];
          cf* yp = &y[(size_t)(m2 + l2) * N2 + n];
          cf t;
          if (mode == 0) { t = cmulf(cscale(c, *xp), *yp); rp->re += t.re; rp->im += t.im; }
          else if (mode == 1) { t = cmulf(cscale(c, *rp), cconj(*yp)); xp->re += t.re; xp->im += t.im; }
          else { t = cmulf(cscale(c, *rp), cconj(*xp)); yp->re += t.re; yp->im += t.im; }
        }
      }
    }
  }
}

/*
 * Batched driver.  Mirrors Gpart_add_CGproduct / _back0 / _back1 (core/CGproduct.hpp:44-104)
 * and the Diag twins (core/DiagCGproduct.hpp:44-105): reconcile batches, then loop over cells.
 * When the tensor being written is broadcast (batch 1 < B) the cells all accumulate into the
 * same rows, exactly as the reference's stride-0 view does; that loop is kept serial.
 * Returns 0, or 1 when the reference would GELIB_SKIP (batches cannot be reconciled,
 * l outside |l1-l2|..l1+l2, or the output row is too short).
 */
int oracle_cg(int mode, int diag, float* r, float* x, float* y, int B, int rB, int xB, int yB,
              int l1, int l2, int l, int N1, int N2, int NR, int offs, int nthreads) {
  if ((rB != 1 && rB != B) || (xB != 1 && xB != B) || (yB != 1 && yB != B)) return 1;
  if (l < abs(l1 - l2) || l > l1 + l2) return 1;
  if (diag && N1 != N2) return 1;
  if ((diag ? N1 : N1 * N2) + offs > NR) return 1;
  float* C = (float*)malloc(sizeof(float) * (size_t)(2 * l1 + 1) * (2 * l2 + 1));
  oracle_cg_matrix(l1, l2, l, C);
  const size_t rs = (rB == 1 && B > 1) ? 0 : (size_t)(2 * l + 1) * NR;
  const size_t xs = (xB == 1 && B > 1) ? 0 : (size_t)(2 * l1 + 1) * N1;
  const size_t ys = (yB == 1 && B > 1) ? 0 : (size_t)(2 * l2 + 1) * N2;
  const size_t ws = mode == 0 ? rs : (mode == 1 ? xs : ys); /* stride of the written tensor */
  int nt = set_threads(nthreads);
  if (ws == 0 && B > 1) nt = 1;
  (void)nt;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int b = 0; b < B; b++)
    cg_cell(mode, diag, (cf*)r + b * rs, (cf*)x + b * xs, (cf*)y + b * ys, C, l1, l2, l, N1, N2, NR,
            offs);
  free(C);
  return 0;
}

/* ---- spherical harmonics: SO3part::add_spharm CPU branch, SO3/SO3part.hpp:340-397 ---- */
/*
 * X: (xB, 3, n) float, R: (B, 2L+1, n) complex float, R += Y_L(X).  xB is B or 1.
 * The float/double mix of the reference is kept: the Legendre table is float, each
 * recursion step is evaluated in double (the literals 2.0*l-1.0 promote it) except the
 * explicitly float-cast factors, and every store rounds to float.
 */
int oracle_spharm(float* R, const float* X, int B, int xB, int L, int n, int nthreads) {
  if (xB != 1 && xB != B) return 1;
  const size_t xs = (xB == 1 && B > 1) ? 0 : (size_t)3 * n;
  int nt = set_threads(nthreads);
  (void)nt;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int b = 0; b < B; b++) {
    cf* r = (cf*)R + (size_t)b * (2 * L + 1) * n;
    const float* x3 = X + b * xs;
    const int W = 2 * L + 1;
    float* P = (float*)malloc(sizeof(float) * (size_t)W * W);
    for (int j = 0; j < n; j++) {
      float vx = x3[0 * n + j];
      float vy = x3[1 * n + j];
      float vz = x3[2 * n + j];
      float length = sqrtf(vx * vx + vy * vy + vz * vz);
      float len2 = sqrtf(vx * vx + vy * vy);
      if (len2 == 0 || isnan(vx / len2) || isnan(vy / len2)) {          /* :363-365 */
        float a = (float)sqrt(((float)(2 * L + 1)) / (M_PI * 4.0));
        r[(size_t)L * n + j].re += a;
      } else {
        float x = vz / length;                                            /* :370 */
        memset(P, 0, sizeof(float) * (size_t)W * W);
        P[0] = 1;
        float xfact = (float)sqrt(1.0 - x * x);
        for (int l = 1; l <= L; l++) {                                    /* :374-379 */
          P[l * W + l] = (float)(-(2.0 * l - 1.0) * xfact * P[(l - 1) * W + (l - 1)]);
          P[l * W + l - 1] = (float)((2.0 * l - 1.0) * P[(l - 1) * W + (l - 1)] * x);
          for (int m = 0; m < l - 1; m++)
            P[l * W + m] = (float)(((2.0 * l - 1.0) * P[(l - 1) * W + m] * x -
                                    ((float)(l + m - 1.0)) * (P[(l - 2) * W + m])) /
                                   ((float)(l - m)));
        }
        cf cphi; cphi.re = vx / len2; cphi.im = vy / len2;                /* :382 */
        cf phase; phase.re = (float)sqrt((2.0 * L + 1.0) / (M_PI * 4.0)); phase.im = 0;
        for (int m = 0; m <= L; m++) {                                    /* :387-393 */
          float p = P[L * W + m];
          cf a; a.re = phase.re * p; a.im = phase.im * p;
          r[(size_t)(L + m) * n + j].re += a.re;
          r[(size_t)(L + m) * n + j].im += a.im;
          if (m > 0) {
            float s = (float)(1 - 2 * (m % 2));
            r[(size_t)(L - m) * n + j].re += s * a.re;
            r[(size_t)(L - m) * n + j].im += s * (-a.im);
          }
          if (m < L) {
            float d = sqrtf((float)(L - m) * (L + m + 1));
            cf q; q.re = cphi.re / d; q.im = cphi.im / d;
            phase = cmulf(phase, q);
          }
        }
      }
    }
    free(P);
  }
  return 0;
}
