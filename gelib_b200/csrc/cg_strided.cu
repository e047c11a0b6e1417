// Fully strided fallback kernels for the (Diag)CG product and its two gradients.
//
// They accept what the tiled kernels do not: a channel stride other than one complex element, rows
// too long for shared-memory staging, and outputs that are broadcast over cells (several cells add
// into the same memory, core/Gpart.hpp:168-185 of GElib).  One CTA handles one (cell, triple); a
// thread owns one output element and walks the band.  Gradients are combined with atomicAdd because
// several triples (and, for broadcast outputs, several cells) contribute to one element.
#include <cstring>
#include <mutex>

#include "plan.h"

namespace gelib_b200 {

namespace {

struct StridedArgs {
  PartView x[kMaxParts], y[kMaxParts], r[kMaxParts];  // for gradients x or y is the output view
  CellGrid cg;
  const Triple* triples;
  const float* coeffs;
  const double* coeffs64;  // the same table in double (GELIB_FP64), else nullptr
  int offs_extra;
  int diag;
  int atomic_out;  // forward only: output is broadcast, combine with atomics
  int overwrite;   // forward only
};

__device__ __forceinline__ float2 ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }

// mode 0: forward, 1: gradient wrt x, 2: gradient wrt y.  ACC: float, or double for GELIB_FP64 (coefficients and sums).
template <int MODE, typename ACC>
__global__ void __launch_bounds__(256) cg_strided_kernel(const __grid_constant__ StridedArgs A) {
  const long long cell = blockIdx.x;
  const Triple t = A.triples[blockIdx.y];
  const PartView& xp = A.x[t.xi];
  const PartView& yp = A.y[t.yi];
  const PartView& rp = A.r[t.ri];
  const int l1 = t.l1, l2 = t.l2, l = t.l;
  const int n1 = xp.n, n2 = yp.n;
  const ACC* C = (sizeof(ACC) == 8 ? reinterpret_cast<const ACC*>(A.coeffs64) : reinterpret_cast<const ACC*>(A.coeffs)) + t.coff;
  float* xb = xp.base + cell_offset(xp, A.cg, cell);
  float* yb = yp.base + cell_offset(yp, A.cg, cell);
  float* rb = rp.base + cell_offset(rp, A.cg, cell) + (long long)(t.offs + A.offs_extra) * rp.sc;
  const bool diag = A.diag != 0;

  if (MODE == 0) {
    const int per_row = diag ? n1 : n1 * n2;
    const int total = (2 * l + 1) * per_row;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int mi = e / per_row, ch = e - mi * per_row;
      const int m = mi - l;
      const int a = diag ? ch : ch / n2, b = diag ? ch : ch - a * n2;
      const int lo = max(-l1, m - l2), hi = min(l1, m + l2);
      // offset of this row's first coefficient in the band table
      int cpos = 0;
      for (int mm = -l; mm < m; mm++) cpos += max(0, min(l1, mm + l2) - max(-l1, mm - l2) + 1);
      ACC sr = 0, si = 0;
      for (int m1 = lo; m1 <= hi; m1++) {
        const ACC c = C[cpos + (m1 - lo)];
        const float2 xv = ld2(xb + (long long)(m1 + l1) * xp.sm + (long long)a * xp.sc);
        const float2 yv = ld2(yb + (long long)(m - m1 + l2) * yp.sm + (long long)b * yp.sc);
        const ACC cr = c * xv.x, ci = c * xv.y;
        sr = fma(cr, (ACC)yv.x, sr); sr = fma(-ci, (ACC)yv.y, sr);
        si = fma(cr, (ACC)yv.y, si); si = fma(ci, (ACC)yv.x, si);
      }
      float* p = rb + (long long)mi * rp.sm + (long long)ch * rp.sc;
      if (A.atomic_out) {
        atomicAdd(p, (float)sr);
        atomicAdd(p + 1, (float)si);
      } else if (A.overwrite) {
        p[0] = (float)sr; p[1] = (float)si;
      } else {
        p[0] = (float)(p[0] + sr); p[1] = (float)(p[1] + si);
      }
    }
  } else {
    // output element (mo, ch) of x (MODE 1) or y (MODE 2)
    const int lo_l = MODE == 1 ? l1 : l2, ot_l = MODE == 1 ? l2 : l1;
    const int no = MODE == 1 ? n1 : n2, nt = MODE == 1 ? n2 : n1;
    const PartView& op = MODE == 1 ? xp : yp;
    const PartView& tp = MODE == 1 ? yp : xp;
    float* ob = MODE == 1 ? xb : yb;
    const float* tb = MODE == 1 ? yb : xb;
    const int total = (2 * lo_l + 1) * no;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int mi = e / no, ch = e - mi * no;
      const int mo = mi - lo_l;
      ACC sr = 0, si = 0;
      for (int mt = -ot_l; mt <= ot_l; mt++) {
        const int m = mo + mt;
        if (m < -l || m > l) continue;
        const int m1 = MODE == 1 ? mo : mt;
        int cpos = 0;
        for (int mm = -l; mm < m; mm++) cpos += max(0, min(l1, mm + l2) - max(-l1, mm - l2) + 1);
        const ACC c = C[cpos + (m1 - max(-l1, m - l2))];
        const float* grow = rb + (long long)(m + l) * rp.sm;
        const float* trow = tb + (long long)(mt + ot_l) * tp.sm;
        if (diag) {
          const float2 g = ld2(grow + (long long)ch * rp.sc);
          const float2 tv = ld2(trow + (long long)ch * tp.sc);
          const ACC gr = c * g.x, gi = c * g.y;
          sr = fma(gr, (ACC)tv.x, sr); sr = fma(gi, (ACC)tv.y, sr);
          si = fma(gi, (ACC)tv.x, si); si = fma(-gr, (ACC)tv.y, si);
        } else {
          for (int k = 0; k < nt; k++) {
            const int gch = MODE == 1 ? ch * n2 + k : k * n2 + ch;
            const float2 g = ld2(grow + (long long)gch * rp.sc);
            const float2 tv = ld2(trow + (long long)k * tp.sc);
            const ACC gr = c * g.x, gi = c * g.y;
            sr = fma(gr, (ACC)tv.x, sr); sr = fma(gi, (ACC)tv.y, sr);
            si = fma(gi, (ACC)tv.x, si); si = fma(-gr, (ACC)tv.y, si);
          }
        }
      }
      float* p = ob + (long long)mi * op.sm + (long long)ch * op.sc;
      atomicAdd(p, (float)sr);
      atomicAdd(p + 1, (float)si);
    }
  }
}

}  // namespace

int launch_cg_strided(const VecCall& c, int mode, cudaStream_t s) {
  static const char* fn = "SO3vec_addCGproduct(strided)";
  const std::vector<PartView>& xv = mode == 1 ? c.xg : c.x;
  const std::vector<PartView>& yv = mode == 2 ? c.yg : c.y;
  const bool fp64 = (c.flags & GELIB_FP64) != 0;
  std::vector<int> key = {2 /*family*/, (c.diag ? 1 : 0) | (fp64 ? 2 : 0), (int)xv.size(), (int)yv.size(), (int)c.r.size()};
  for (const auto& p : xv) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : yv) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.r) key.push_back(p.l);
  const auto xs = sig_of(xv), ys = sig_of(yv), rs = sig_of(c.r);
  const bool diag = c.diag;
  DevicePlan* plan = get_plan(key, [&](DevicePlan& p) {
    build_schedule(xs, ys, rs, diag, true, &p.sched);
    if (fp64) {  // the same band tables in double, stored behind the plan's float table slot
      std::vector<double> c64;
      for (const Triple& t : p.sched.triples)
        for (int m = -t.l; m <= t.l; m++)
          for (int m1 = std::max<int>(-t.l1, m - t.l2); m1 <= std::min<int>(t.l1, m + t.l2); m1++)
            c64.push_back(cg_coefficient(t.l1, t.l2, t.l, m1, m - m1));
      p.h_floats.resize(2 * c64.size());
      memcpy(p.h_floats.data(), c64.data(), c64.size() * sizeof(double));
    }
  });
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->ntriples == 0 || c.cg.ncells == 0) return GELIB_OK;
  if (plan->ntriples > 65535) return fail(GELIB_SKIPPED, fn, "more than 65535 triples");
  if (c.cg.ncells > 0x7fffffffLL) return fail(GELIB_SKIPPED, fn, "number of cells exceeds 2^31-1");

  StridedArgs a;
  for (size_t i = 0; i < xv.size(); i++) a.x[i] = xv[i];
  for (size_t i = 0; i < yv.size(); i++) a.y[i] = yv[i];
  for (size_t i = 0; i < c.r.size(); i++) a.r[i] = c.r[i];
  a.cg = c.cg;
  a.triples = plan->triples;
  a.coeffs = plan->coeffs;
  a.coeffs64 = fp64 ? reinterpret_cast<const double*>(plan->floats) : nullptr;
  a.offs_extra = c.offs_extra;
  a.diag = c.diag ? 1 : 0;
  a.atomic_out = c.r_bcast ? 1 : 0;
  a.overwrite = (c.flags & GELIB_OVERWRITE) && !c.r_bcast ? 1 : 0;
  const dim3 grid((unsigned)c.cg.ncells, (unsigned)plan->ntriples);
  if (fp64) {
    if (mode == 0) cg_strided_kernel<0, double><<<grid, 256, 0, s>>>(a);
    else if (mode == 1) cg_strided_kernel<1, double><<<grid, 256, 0, s>>>(a);
    else cg_strided_kernel<2, double><<<grid, 256, 0, s>>>(a);
  } else {
    if (mode == 0) cg_strided_kernel<0, float><<<grid, 256, 0, s>>>(a);
    else if (mode == 1) cg_strided_kernel<1, float><<<grid, 256, 0, s>>>(a);
    else cg_strided_kernel<2, float><<<grid, 256, 0, s>>>(a);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "strided kernel launch");
  count_launch();
  return GELIB_OK;
}

// ---- the forward product without any allocation ---------------------------------------------------------------
//
// Every other launcher keeps its tables (triple list, band coefficients) in device memory that the plan cache gets
// from cudaMalloc on the first call of a product signature.  A caller that must not allocate -- one that runs inside
// a memory pool it may not leave, under a real-time budget where cudaMalloc's implicit synchronisation is not
// acceptable, or after it has handed all device memory to somebody else -- uses this variant instead: the same
// kernel, with the tables in a fixed array that is part of the library's image on every device that loads it.
//
// The array is shared by all calls on a device and keeps the tables of the last call: each call uploads its own
// tables on the caller's stream before its kernel, so calls on ONE stream are ordered, and calls that can overlap on
// the GPU (different streams, different threads) race on the array and must be serialised by the caller.
namespace {

constexpr size_t kStaticTableBytes = 64 * 1024;  // 175 triples + 7651 coefficients (maxl 6) take 34 KB
__device__ __align__(256) unsigned char g_static_tables[kStaticTableBytes];

// Device address of g_static_tables on the current device.  In host code the array's name is only a handle; the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
unsigned char* static_tables_address() {
  static std::mutex mu;
  static unsigned char* addr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_tables) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    addr[dev] = static_cast<unsigned char*>(p);
  }
  return addr[dev];
}

}  // namespace

int launch_cg_strided_static(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addCGproduct_static";
  Schedule sched;  // host memory only
  build_schedule(sig_of(c.x), sig_of(c.y), sig_of(c.r), c.diag, true, &sched);
  const size_t ntr = sched.triples.size();
  if (ntr == 0 || c.cg.ncells == 0) return GELIB_OK;
  if (ntr > 65535) return fail(GELIB_SKIPPED, fn, "more than 65535 triples");
  if (c.cg.ncells > 0x7fffffffLL) return fail(GELIB_SKIPPED, fn, "number of cells exceeds 2^31-1");
  const size_t tbytes = (ntr * sizeof(Triple) + 15) / 16 * 16, cbytes = sched.coeffs.size() * sizeof(float);
  if (tbytes + cbytes > kStaticTableBytes)
    return fail(GELIB_INVALID, fn, "the tables of this product need " + std::to_string(tbytes + cbytes) +
                                       " bytes, the static array holds " + std::to_string(kStaticTableBytes));
  unsigned char* dev = static_tables_address();
  if (!dev) return fail(GELIB_CUDA_ERROR, fn, "cudaGetSymbolAddress failed for the static table array");
  // one upload: [triples | coefficients]; pageable source, so the copy has left this buffer when the call returns
  std::vector<unsigned char> host(tbytes + cbytes);
  memcpy(host.data(), sched.triples.data(), ntr * sizeof(Triple));
  memcpy(host.data() + tbytes, sched.coeffs.data(), cbytes);
  GELIB_CUDA_TRY(fn, cudaMemcpyAsync(dev, host.data(), host.size(), cudaMemcpyHostToDevice, s));

  StridedArgs a;
  for (size_t i = 0; i < c.x.size(); i++) a.x[i] = c.x[i];
  for (size_t i = 0; i < c.y.size(); i++) a.y[i] = c.y[i];
  for (size_t i = 0; i < c.r.size(); i++) a.r[i] = c.r[i];
  a.cg = c.cg;
  a.triples = reinterpret_cast<const Triple*>(dev);
  a.coeffs = reinterpret_cast<const float*>(dev + tbytes);
  a.coeffs64 = nullptr;
  a.offs_extra = c.offs_extra;
  a.diag = c.diag ? 1 : 0;
  a.atomic_out = c.r_bcast ? 1 : 0;
  a.overwrite = (c.flags & GELIB_OVERWRITE) && !c.r_bcast ? 1 : 0;
  cg_strided_kernel<0, float><<<dim3((unsigned)c.cg.ncells, (unsigned)ntr), 256, 0, s>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "strided kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
