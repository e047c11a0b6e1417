// Clebsch-Gordan coefficient bank, triple schedules and error plumbing (host code).
//
// Replaces SO3CGbank (SO3/SO3CGbank.hpp:25-97 of GElib): instead of one dense matrix per
// (l1,l2,l) cached in an unsynchronised unordered_map for "the" GPU, coefficients are laid out
// band-by-band in the order the kernels traverse them, concatenated for all triples of a product,
// and uploaded once per (device, product signature) under a mutex.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>

#include "common.h"

namespace gelib_b200 {

// ---- errors ---------------------------------------------------------------------------------------------

static thread_local std::string g_last_error;
static std::atomic<long long> g_launches{0};

void set_error(const std::string& msg) { g_last_error = msg; }

int fail(int status, const char* fn, const std::string& msg) {
  if (status == GELIB_SKIPPED)
    g_last_error = std::string("Function ") + fn + " skipped: " + msg + ".";
  else
    g_last_error = std::string("GElib error in ") + fn + " : " + msg + ".";
  return status;
}

int check_cuda(cudaError_t e, const char* fn, const char* what) {
  g_last_error = std::string("CUDA error in ") + fn + " (" + what + "): " + cudaGetErrorString(e);
  return GELIB_CUDA_ERROR;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }
const std::string& last_error() { return g_last_error; }

// ---- coefficients ---------------------------------------------------------------------------------------

// <l1 m1 l2 m2 | l m> with m = m1+m2, Condon-Shortley phases, by Racah's single-sum formula.
// All factorials go through lgamma so l up to the hundreds stays finite; the sum is done in double.
double cg_coefficient(int l1, int l2, int l, int m1, int m2) {
  const int m = m1 + m2;
  if (l < std::abs(l1 - l2) || l > l1 + l2) return 0.0;
  if (std::abs(m1) > l1 || std::abs(m2) > l2 || std::abs(m) > l) return 0.0;
  auto lf = [](int k) { return std::lgamma((double)k + 1.0); };
  // triangle factor and the six (j +- m)! terms, as half-logs
  const double half_log = 0.5 * (lf(l1 + l2 - l) + lf(l1 - l2 + l) + lf(l2 - l1 + l) - lf(l1 + l2 + l + 1) +
                                 lf(l1 + m1) + lf(l1 - m1) + lf(l2 + m2) + lf(l2 - m2) + lf(l + m) + lf(l - m));
  // k runs over the values for which all six factorial arguments are non-negative
  const int a = l1 + l2 - l, b = l1 - m1, c = l2 + m2, d = l - l2 + m1, e = l - l1 - m2;
  int kmin = 0;
  if (-d > kmin) kmin = -d;
  if (-e > kmin) kmin = -e;
  int kmax = a;
  if (b < kmax) kmax = b;
  if (c < kmax) kmax = c;
  double sum = 0.0;
  for (int k = kmin; k <= kmax; k++) {
    const double lg = lf(k) + lf(a - k) + lf(b - k) + lf(c - k) + lf(d + k) + lf(e + k);
    const double term = std::exp(half_log - lg);
    sum += (k & 1) ? -term : term;
  }
  return std::sqrt(2.0 * l + 1.0) * sum;
}

int band_size(int l1, int l2, int l) {
  int T = 0;
  for (int m = -l; m <= l; m++) {
    const int lo = std::max(-l1, m - l2), hi = std::min(l1, m + l2);
    if (hi >= lo) T += hi - lo + 1;
  }
  return T;
}

// ---- schedule ---------------------------------------------------------------------------------------------

void build_schedule(const std::vector<PartSig>& x, const std::vector<PartSig>& y, const std::vector<PartSig>& r,
                    bool diag, bool with_coeffs, Schedule* out) {
  out->triples.clear();
  out->coeffs.clear();
  std::vector<int> offset(r.size(), 0);
  for (size_t i = 0; i < x.size(); i++) {
    for (size_t j = 0; j < y.size(); j++) {
      const int l1 = x[i].l, l2 = y[j].l;
      for (int l = std::abs(l1 - l2); l <= l1 + l2; l++) {
        int ri = -1;
        for (size_t k = 0; k < r.size(); k++)
          if (r[k].l == l) ri = (int)k;
        if (ri < 0) continue;
        Triple t;
        t.l1 = (short)l1; t.l2 = (short)l2; t.l = (short)l;
        t.xi = (short)i; t.yi = (short)j; t.ri = (short)ri;
        t.offs = offset[ri];
        t.coff = (int)out->coeffs.size();
        offset[ri] += diag ? x[i].n : x[i].n * y[j].n;
        if (with_coeffs) {
          for (int m = -l; m <= l; m++) {
            const int lo = std::max(-l1, m - l2), hi = std::min(l1, m + l2);
            for (int m1 = lo; m1 <= hi; m1++) out->coeffs.push_back((float)cg_coefficient(l1, l2, l, m1, m - m1));
          }
        }
        out->triples.push_back(t);
      }
    }
  }
}

}  // namespace gelib_b200
