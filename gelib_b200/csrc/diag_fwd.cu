// Diagonal Clebsch-Gordan product, forward, one cell per CTA: the variant used for 17 or more channels.
//
// Same arithmetic and item structure as diag_fwd_kernel (diag.cu): an item is one (l1,l2) pair and one output
// row index m; every product p = x[m1] y[m-m1] feeds the accumulators of all output l through a dense
// [m1][l] coefficient table.  What differs is how the bookkeeping reaches the inner loop:
//   * a lane owns one channel, or two adjacent channels when the channel count is even (16-byte loads and
//     stores, 512 contiguous bytes per warp and output row);
//   * items are grouped into chunks; the coefficient tables and item records of a chunk are contiguous in the
//     plan and are copied to shared memory with cp.async one chunk ahead, so the inner loop reads its
//     coefficients with broadcast shared-memory loads and never waits on global memory for them;
//   * a record carries, per output l, the output part and the float offset of (row, first channel) in it
//     (dense output rows are required), so an output address is one shared-memory load and one add.
// The semantics are those of GElib's CPU loop SO3part::add_DiagCGproduct_kernel (SO3/SO3part.hpp:276-290) and of
// Gvec::add_DiagCGproduct (core/Gvec.hpp:358-367); the reference has no GPU version (SO3/SO3part.hpp:324-326).
#include <cuda_pipeline.h>

#include <algorithm>

#include "plan.h"

namespace gelib_b200 {

namespace {

constexpr int kCoefCap = 2048;  // floats of coefficient tables per chunk
constexpr int kRecCap = 256;    // int4 records per chunk
constexpr int kBufFloats = kCoefCap + 4 * kRecCap;

struct DiagFwdArgs {
  PartView x[kMaxParts], y[kMaxParts], r[kMaxParts];
  int xrow0[kMaxParts], yrow0[kMaxParts];
  int nx, ny, nr, xrows, yrows, n;
  CellGrid cg;
  const float* coeffs;
  const int4* recs;
  // 8 ints per chunk: number of items, -, coef_begin, coef_floats, rec_begin, rec_count, -, -.  The record block of a
  // chunk starts with one int per item (padded to int4s): the int4 index of the item's record inside the block.
  const int* chunks;
  int nchunks, chunks_per_z;
  int offs_extra;
  int accumulate;
};

template <int CPL>
__device__ __forceinline__ void stage_rows(float* dst, const PartView* parts, const int* row0, int nparts, int n, int ch0,
                                           const CellGrid& cg, long long cell) {
  constexpr int W = 32 * CPL;  // channels per staged row
  for (int i = 0; i < nparts; i++) {
    const PartView& p = parts[i];
    const float* src = p.base + cell_offset(p, cg, cell) + 2 * ch0;
    const int total = (2 * p.l + 1) * W;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int m = e / W, ch = e % W;
      float2 v = make_float2(0.f, 0.f);
      if (ch0 + ch < n) v = __ldg(reinterpret_cast<const float2*>(src + (long long)m * p.sm + 2 * ch));
      *reinterpret_cast<float2*>(dst + 2 * ((row0[i] + m) * W + ch)) = v;
    }
  }
}

// One band entry: p = x y for the lane's CPL channels, then acc[j] += c[j] p for 4*NG output l.
template <int CPL, int NG>
__device__ __forceinline__ void band_step(const float* smem, int xi, int yi, const float4 (&c)[NG],
                                          float (&acc)[4 * NG][2 * CPL]) {
  float pr[CPL], pi[CPL];
  if constexpr (CPL == 2) {
    const float4 xv = *reinterpret_cast<const float4*>(&smem[xi]);
    const float4 yv = *reinterpret_cast<const float4*>(&smem[yi]);
    pr[0] = xv.x * yv.x - xv.y * yv.y; pi[0] = xv.x * yv.y + xv.y * yv.x;
    pr[1] = xv.z * yv.z - xv.w * yv.w; pi[1] = xv.z * yv.w + xv.w * yv.z;
  } else {
    const float2 xv = *reinterpret_cast<const float2*>(&smem[xi]);
    const float2 yv = *reinterpret_cast<const float2*>(&smem[yi]);
    pr[0] = xv.x * yv.x - xv.y * yv.y; pi[0] = xv.x * yv.y + xv.y * yv.x;
  }
#pragma unroll
  for (int k = 0; k < NG; k++) {
    const float cj[4] = {c[k].x, c[k].y, c[k].z, c[k].w};
#pragma unroll
    for (int q = 0; q < 4; q++)
#pragma unroll
      for (int e = 0; e < CPL; e++) {
        acc[4 * k + q][2 * e] = fmaf(cj[q], pr[e], acc[4 * k + q][2 * e]);
        acc[4 * k + q][2 * e + 1] = fmaf(cj[q], pi[e], acc[4 * k + q][2 * e + 1]);
      }
  }
}

template <int CPL, int NG>
__device__ __forceinline__ void run_item(const float* smem, const long long* rbase, int rec, int nl, int band, int nlp,
                                         int xi, int yi, int ci, int j0, int lane_off, bool ok, bool acc_mode) {
  constexpr int ROW = 64 * CPL;  // floats per staged row
  float acc[4 * NG][2 * CPL];
#pragma unroll
  for (int j = 0; j < 4 * NG; j++)
#pragma unroll
    for (int e = 0; e < 2 * CPL; e++) acc[j][e] = 0.f;
  // two coefficient register sets: entry b+1 is loaded while entry b is used
  float4 ca[NG], cb[NG];
  int cidx = ci + j0;
#pragma unroll
  for (int k = 0; k < NG; k++) ca[k] = *reinterpret_cast<const float4*>(&smem[cidx + 4 * k]);
  for (int b = 0; b < band; b += 2) {
    const bool two = b + 1 < band;
    if (two) {
#pragma unroll
      for (int k = 0; k < NG; k++) cb[k] = *reinterpret_cast<const float4*>(&smem[cidx + nlp + 4 * k]);
    }
    band_step<CPL, NG>(smem, xi, yi, ca, acc);
    if (two) {
      if (b + 2 < band) {
#pragma unroll
        for (int k = 0; k < NG; k++) ca[k] = *reinterpret_cast<const float4*>(&smem[cidx + 2 * nlp + 4 * k]);
      }
      band_step<CPL, NG>(smem, xi + ROW, yi - ROW, cb, acc);
    }
    cidx += 2 * nlp;
    xi += 2 * ROW;
    yi -= 2 * ROW;
  }
#pragma unroll
  for (int j = 0; j < 4 * NG; j++) {
    if (j0 + j < nl) {
      const int4 q = *reinterpret_cast<const int4*>(&smem[rec + 4 * (1 + j0 + j)]);
      const long long off = ((long long)q.z << 32) | (unsigned)q.y;
      float* p = reinterpret_cast<float*>(rbase[q.x]) + off + lane_off;
      if (ok) {
        if constexpr (CPL == 2) {
          float4 v = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
          if (acc_mode) {
            const float4 o = *reinterpret_cast<const float4*>(p);
            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            *reinterpret_cast<float4*>(p) = v;
          } else {
            __stcs(reinterpret_cast<float4*>(p), v);
          }
        } else {
          float2 v = make_float2(acc[j][0], acc[j][1]);
          if (acc_mode) {
            const float2 o = *reinterpret_cast<const float2*>(p);
            v.x += o.x; v.y += o.y;
            *reinterpret_cast<float2*>(p) = v;
          } else {
            __stcs(reinterpret_cast<float2*>(p), v);
          }
        }
      }
    }
  }
}

template <int CPL>
__global__ void __launch_bounds__(256) diag_fwd_cell_kernel(const __grid_constant__ DiagFwdArgs A) {
  extern __shared__ __align__(16) float smem[];
  constexpr int W = 32 * CPL;
  // [0, 2*kMaxParts): address of the cell's first row of every output part; staged x rows; staged y rows; 2 buffers
  long long* rbase = reinterpret_cast<long long*>(smem);
  const long long cell = blockIdx.x;
  const int ch0 = blockIdx.y * W;
  const int XS = 2 * kMaxParts, YS = XS + 2 * A.xrows * W, BUF = YS + 2 * A.yrows * W;
  if ((int)threadIdx.x < A.nr) {
    const PartView& rp = A.r[threadIdx.x];
    rbase[threadIdx.x] = reinterpret_cast<long long>(rp.base + cell_offset(rp, A.cg, cell) + 2LL * A.offs_extra + 2 * ch0);
  }
  const int c_begin = blockIdx.z * A.chunks_per_z, c_end = min(c_begin + A.chunks_per_z, A.nchunks);

  auto fetch = [&](int c, int buf) {
    const int* ck = A.chunks + 8 * c;
    const int coef_begin = __ldg(ck + 2), coef_floats = __ldg(ck + 3), rec_begin = __ldg(ck + 4), rec_count = __ldg(ck + 5);
    float* dst = smem + BUF + buf * kBufFloats;
    for (int e = threadIdx.x; e < coef_floats / 4; e += blockDim.x)
      __pipeline_memcpy_async(dst + 4 * e, A.coeffs + coef_begin + 4 * e, 16);
    for (int e = threadIdx.x; e < rec_count; e += blockDim.x)
      __pipeline_memcpy_async(dst + kCoefCap + 4 * e, A.recs + rec_begin + e, 16);
    __pipeline_commit();
  };

  if (c_begin < c_end) fetch(c_begin, 0);
  stage_rows<CPL>(smem + XS, A.x, A.xrow0, A.nx, A.n, ch0, A.cg, cell);
  stage_rows<CPL>(smem + YS, A.y, A.yrow0, A.ny, A.n, ch0, A.cg, cell);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const bool ok = ch0 + lane * CPL < A.n;
  const bool acc_mode = A.accumulate != 0;
  const int lane_off = 2 * CPL * lane;
  for (int c = c_begin; c < c_end; c++) {
    const int buf = (c - c_begin) & 1;
    if (c + 1 < c_end) {
      fetch(c + 1, buf ^ 1);
      __pipeline_wait_prior(1);
    } else {
      __pipeline_wait_prior(0);
    }
    __syncthreads();
    const int* ck = A.chunks + 8 * c;
    const int nit = __ldg(ck);
    const int CB = BUF + buf * kBufFloats, RB = CB + kCoefCap;
    for (int it = warp; it < nit; it += nwarps) {
      const int rec = RB + 4 * __float_as_int(smem[RB + it]);
      const int4 h = *reinterpret_cast<const int4*>(&smem[rec]);
      const int nl = h.x & 255, band = (h.x >> 8) & 255, nlp = h.x >> 16;
      const int xi = XS + 2 * W * (h.y & 0xffff) + lane_off, yi = YS + 2 * W * (h.y >> 16) + lane_off;
      for (int j0 = 0; j0 < nl; j0 += 12) {
        const int ng = min(3, (nlp - j0) >> 2);
        if (ng == 1) run_item<CPL, 1>(smem, rbase, rec, nl, band, nlp, xi, yi, CB + h.z, j0, lane_off, ok, acc_mode);
        else if (ng == 2) run_item<CPL, 2>(smem, rbase, rec, nl, band, nlp, xi, yi, CB + h.z, j0, lane_off, ok, acc_mode);
        else run_item<CPL, 3>(smem, rbase, rec, nl, band, nlp, xi, yi, CB + h.z, j0, lane_off, ok, acc_mode);
      }
    }
    __syncthreads();  // everyone is done with this buffer before the copy two chunks ahead overwrites it
  }
}

// Plan: items sorted by cost, coefficient tables re-laid in that order, greedy chunks within the buffer caps.
void build_plan(DevicePlan& p, const std::vector<PartSig>& xs, const std::vector<PartSig>& ys,
                const std::vector<PartSig>& rs, const std::vector<int>& xrow0, const std::vector<int>& yrow0) {
  int mx = 0;
  build_diag_items(p, xs, ys, rs, &mx);
  const auto& tr = p.sched.triples;
  struct Rec { std::vector<int4> v; std::vector<float> coef; int cost; };
  std::vector<Rec> all;
  for (const int4& it : p.h_items) {
    const int tf = it.x & 0xffff, nl = it.x >> 16, m = it.y, nlp = it.w;
    const Triple& t0 = tr[tf];
    const int lo = std::max<int>(-t0.l1, m - t0.l2), hi = std::min<int>(t0.l1, m + t0.l2);
    const int band = hi - lo + 1;
    Rec r;
    r.cost = band * (nl + 6) + 4 * nl;
    r.v.push_back(make_int4(nl | (band << 8) | (nlp << 16),
                            (xrow0[t0.xi] + lo + t0.l1) | ((yrow0[t0.yi] + m - lo + t0.l2) << 16), 0, 0));
    for (int j = 0; j < nl; j++) {
      const Triple& t = tr[tf + j];
      const long long off = (long long)(m + t.l) * 2 * rs[t.ri].n + 2LL * t.offs;
      r.v.push_back(make_int4(t.ri, (int)(unsigned)(off & 0xffffffffLL), (int)(off >> 32), 0));
    }
    r.coef.assign(p.sched.coeffs.begin() + it.z, p.sched.coeffs.begin() + it.z + band * nlp);
    all.push_back(std::move(r));
  }
  std::stable_sort(all.begin(), all.end(), [](const Rec& u, const Rec& v) { return u.cost > v.cost; });
  p.h_items.clear();
  p.h_jobs.clear();
  p.sched.coeffs.clear();
  std::vector<int> chunks;
  size_t i = 0;
  while (i < all.size()) {
    // greedy fill within the caps; then keep a multiple of 8 items (one round per warp) when possible
    size_t j = i;
    int nc = 0, nr = 0;
    while (j < all.size()) {
      const int tab = (int)(j + 1 - i + 3) / 4;  // int4s of the item-offset table if item j is taken
      if (j > i && (nc + (int)all[j].coef.size() > kCoefCap || tab + nr + (int)all[j].v.size() > kRecCap)) break;
      nc += (int)all[j].coef.size();
      nr += (int)all[j].v.size();
      j++;
    }
    if (j - i > 8 && j < all.size()) j = i + (j - i) / 8 * 8;
    const int nit = (int)(j - i), tab = (nit + 3) / 4;
    const int coef_begin = (int)p.sched.coeffs.size(), rec_begin = (int)p.h_items.size();
    std::vector<int> offs(4 * tab, 0);
    nc = 0;
    nr = tab;
    for (size_t q = i; q < j; q++) {
      offs[q - i] = nr;
      all[q].v[0].z = nc;  // coefficient index inside the chunk
      nc += (int)all[q].coef.size();
      nr += (int)all[q].v.size();
    }
    for (int t = 0; t < tab; t++) p.h_items.push_back(make_int4(offs[4 * t], offs[4 * t + 1], offs[4 * t + 2], offs[4 * t + 3]));
    for (size_t q = i; q < j; q++) {
      for (const int4& v : all[q].v) p.h_items.push_back(v);
      p.sched.coeffs.insert(p.sched.coeffs.end(), all[q].coef.begin(), all[q].coef.end());
    }
    const int v[8] = {nit, 0, coef_begin, nc, rec_begin, nr, 0, 0};
    chunks.insert(chunks.end(), v, v + 8);
    i = j;
  }
  // jobs = [number of chunks, chunk table]
  p.h_jobs.push_back((int)chunks.size() / 8);
  p.h_jobs.insert(p.h_jobs.end(), chunks.begin(), chunks.end());
}

}  // namespace

// The plan of the one-cell-per-CTA diagonal kernels (forward and backward share it).
DevicePlan* diag_cell_plan(const VecCall& c, const std::vector<int>& xrow0, const std::vector<int>& yrow0) {
  std::vector<int> key = {5 /*family*/, (int)c.x.size(), (int)c.y.size(), (int)c.r.size(), c.x[0].n};
  for (const auto& p : c.x) key.push_back(p.l);
  for (const auto& p : c.y) key.push_back(p.l);
  for (const auto& p : c.r) { key.push_back(p.l); key.push_back(p.n); }
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  return get_plan(key, [&](DevicePlan& p) { build_plan(p, xs, ys, rs, xrow0, yrow0); });
}

int launch_diag_fwd_fast(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addDiagCGproduct";
  if (c.x.empty() || c.y.empty() || c.r.empty()) return -1;
  const int n = c.x[0].n;
  for (const auto& p : c.x) if (p.n != n || p.l > 60) return -1;
  for (const auto& p : c.y) if (p.n != n || p.l > 60) return -1;
  if (n <= 16) return -1;  // small channel counts: several cells per warp (diag_fwd_kernel)
  DiagFwdArgs a;
  std::vector<int> xrow0, yrow0;
  int row = 0;
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    a.xrow0[i] = row;
    xrow0.push_back(row);
    row += 2 * c.x[i].l + 1;
  }
  a.xrows = row;
  row = 0;
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    a.yrow0[i] = row;
    yrow0.push_back(row);
    row += 2 * c.y[i].l + 1;
  }
  a.yrows = row;
  bool two = (n % 2 == 0) && c.vec_ok && (c.offs_extra % 2 == 0) && n > 32;
  for (size_t i = 0; i < c.r.size(); i++) {
    a.r[i] = c.r[i];
    if (c.r[i].sm != 2LL * c.r[i].n) return -1;  // the records assume dense output rows
    if (c.r[i].n % 2) two = false;
  }
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.nr = (int)c.r.size();
  a.n = n;
  const int W = two ? 64 : 32;
  const size_t smem = ((size_t)2 * (a.xrows + a.yrows) * W + 2 * kMaxParts + 2 * kBufFloats) * sizeof(float);
  if (smem > 200 * 1024) return -1;
  DevicePlan* plan = diag_cell_plan(c, xrow0, yrow0);
  if (!plan) return GELIB_CUDA_ERROR;
  const int nchunks = plan->h_jobs.empty() ? 0 : plan->h_jobs[0];
  if (nchunks == 0 || c.cg.ncells == 0) return GELIB_OK;
  a.cg = c.cg;
  a.coeffs = plan->coeffs;
  a.recs = plan->items;
  a.chunks = plan->jobs + 1;
  a.nchunks = nchunks;
  a.offs_extra = c.offs_extra;
  a.accumulate = (c.flags & GELIB_OVERWRITE) ? 0 : 1;
  const int slices = (n + W - 1) / W;
  const long long ctas = c.cg.ncells * slices;
  int nz = 1;
  if (ctas < 1024) nz = (int)std::min<long long>(nchunks, std::max<long long>(1, 1024 / std::max<long long>(ctas, 1)));
  a.chunks_per_z = (nchunks + nz - 1) / nz;
  nz = (nchunks + a.chunks_per_z - 1) / a.chunks_per_z;
  if (c.cg.ncells > 0x7fffffffLL || slices > 65535 || nz > 65535) return -1;
  const dim3 grid((unsigned)c.cg.ncells, (unsigned)slices, (unsigned)nz);
  cudaError_t e;
  if (two) {
    e = cudaFuncSetAttribute(diag_fwd_cell_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) diag_fwd_cell_kernel<2><<<grid, 256, smem, s>>>(a);
  } else {
    e = cudaFuncSetAttribute(diag_fwd_cell_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) diag_fwd_cell_kernel<1><<<grid, 256, smem, s>>>(a);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "diag forward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
