// Diagonal Clebsch-Gordan product, both gradients from one read of g, one cell per CTA (17 or more channels).
//
//   G[m1,m2]   = sum_l C_l[m1,m2] g_l[cell, m1+m2, offs_l + n]
//   xg[m1, n] += G[m1,m2] conj(y[m2, n]),   yg[m2, n] += G[m1,m2] conj(x[m1, n])
//
// Items, records and the chunked cp.async staging of coefficient tables are those of the forward kernel
// (diag_fwd.cu); a record's per-l entries now say where the rows of g are.  A lane owns one channel: it loads
// the g rows of all l of an item into registers (8-byte streaming loads, 256 contiguous bytes per warp and row),
// forms G once per band entry (2 FMAs per l) and adds the two products into gradient rows of the cell kept in
// shared memory, in a structure-of-arrays layout (real and imaginary planes of 32 lanes) so that the
// shared-memory atomics of a warp never collide.  Warps of a CTA split the items of a chunk, hence the
// atomics; there is no per-pair phase, barrier or private copy.  Rows go to global memory once at the end
// (the CTA owns its cell and channel slice; atomicAdd only for an output broadcast over cells).
// Semantics: SO3part::add_DiagCGproduct_back0/_back1_kernel (SO3/SO3part.hpp:292-322 of GElib) and
// Gvec::add_DiagCGproduct_back0/_back1 (core/Gvec.hpp:369-389); the reference has no GPU version.
#include <cuda_pipeline.h>

#include <algorithm>

#include "plan.h"

namespace gelib_b200 {

namespace {

constexpr int kCoefCap = 2048;
constexpr int kRecCap = 256;
constexpr int kBufFloats = kCoefCap + 4 * kRecCap;

struct DiagBwdArgs {
  PartView x[kMaxParts], y[kMaxParts], g[kMaxParts], xg[kMaxParts], yg[kMaxParts];
  int xrow0[kMaxParts], yrow0[kMaxParts];
  int nx, ny, ng, xrows, yrows, n;
  CellGrid cg;
  const float* coeffs;
  const int4* recs;
  const int* chunks;
  int nchunks;
  int offs_extra;
  int do_x, do_y, x_atomic, y_atomic;
};

__device__ __forceinline__ void stage_rows32(float* dst, const PartView* parts, const int* row0, int nparts, int n,
                                             int ch0, const CellGrid& cg, long long cell) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = parts[i];
    const float* src = p.base + cell_offset(p, cg, cell) + 2 * ch0;
    const int total = (2 * p.l + 1) * 32;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int m = e >> 5, ch = e & 31;
      float2 v = make_float2(0.f, 0.f);
      if (ch0 + ch < n) v = __ldg(reinterpret_cast<const float2*>(src + (long long)m * p.sm + 2 * ch));
      *reinterpret_cast<float2*>(dst + 2 * ((row0[i] + m) * 32 + ch)) = v;
    }
  }
}

// acc: planes [row][re|im][32 lanes]
__device__ __forceinline__ void flush_rows32(const float* acc, const PartView* out, const int* row0, int nparts, int n,
                                             int ch0, const CellGrid& cg, long long cell, bool atomic) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = out[i];
    float* dst = p.base + cell_offset(p, cg, cell) + 2 * ch0;
    const int total = (2 * p.l + 1) * 32;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int m = e >> 5, ch = e & 31;
      if (ch0 + ch >= n) continue;
      const float re = acc[(row0[i] + m) * 64 + ch], im = acc[(row0[i] + m) * 64 + 32 + ch];
      float* q = dst + (long long)m * p.sm + 2 * ch;
      if (atomic) {
        atomicAdd(q, re);
        atomicAdd(q + 1, im);
      } else {
        float2 o = *reinterpret_cast<float2*>(q);
        o.x += re;
        o.y += im;
        *reinterpret_cast<float2*>(q) = o;
      }
    }
  }
}

template <int NG>
__device__ __forceinline__ void run_item(float* smem, const long long* gbase, int rec, int nl, int band, int nlp, int xi,
                                         int yi, int axi, int ayi, int ci, int j0, int lane, bool ok, bool do_x,
                                         bool do_y) {
  float gv[4 * NG][2];
#pragma unroll
  for (int j = 0; j < 4 * NG; j++) {
    gv[j][0] = gv[j][1] = 0.f;
    if (ok && j0 + j < nl) {
      const int4 q = *reinterpret_cast<const int4*>(&smem[rec + 4 * (1 + j0 + j)]);
      const long long off = ((long long)q.z << 32) | (unsigned)q.y;
      const float2 v = __ldcs(reinterpret_cast<const float2*>(reinterpret_cast<const float*>(gbase[q.x]) + off + 2 * lane));
      gv[j][0] = v.x;
      gv[j][1] = v.y;
    }
  }
  int cidx = ci + j0;
  for (int b = 0; b < band; b++) {
    float Gr = 0.f, Gi = 0.f;
#pragma unroll
    for (int k = 0; k < NG; k++) {
      const float4 c = *reinterpret_cast<const float4*>(&smem[cidx + 4 * k]);
      Gr = fmaf(c.x, gv[4 * k][0], Gr); Gi = fmaf(c.x, gv[4 * k][1], Gi);
      Gr = fmaf(c.y, gv[4 * k + 1][0], Gr); Gi = fmaf(c.y, gv[4 * k + 1][1], Gi);
      Gr = fmaf(c.z, gv[4 * k + 2][0], Gr); Gi = fmaf(c.z, gv[4 * k + 2][1], Gi);
      Gr = fmaf(c.w, gv[4 * k + 3][0], Gr); Gi = fmaf(c.w, gv[4 * k + 3][1], Gi);
    }
    const float2 xv = *reinterpret_cast<const float2*>(&smem[xi]);
    const float2 yv = *reinterpret_cast<const float2*>(&smem[yi]);
    if (do_x) {  // G conj(y)
      atomicAdd(&smem[axi], fmaf(Gr, yv.x, Gi * yv.y));
      atomicAdd(&smem[axi + 32], fmaf(Gi, yv.x, -Gr * yv.y));
    }
    if (do_y) {  // G conj(x)
      atomicAdd(&smem[ayi], fmaf(Gr, xv.x, Gi * xv.y));
      atomicAdd(&smem[ayi + 32], fmaf(Gi, xv.x, -Gr * xv.y));
    }
    cidx += nlp;
    xi += 64; axi += 64;
    yi -= 64; ayi -= 64;
  }
}

__global__ void __launch_bounds__(256, 2) diag_bwd_cell_kernel(const __grid_constant__ DiagBwdArgs A) {
  extern __shared__ __align__(16) float smem[];
  long long* gbase = reinterpret_cast<long long*>(smem);
  const long long cell = blockIdx.x;
  const int ch0 = blockIdx.y * 32;
  // staged x rows, staged y rows, xg accumulator planes, yg accumulator planes, two chunk buffers
  const int XS = 2 * kMaxParts, YS = XS + 64 * A.xrows, AX = YS + 64 * A.yrows, AY = AX + 64 * A.xrows;
  const int BUF = AY + 64 * A.yrows;
  if ((int)threadIdx.x < A.ng) {
    const PartView& gp = A.g[threadIdx.x];
    gbase[threadIdx.x] = reinterpret_cast<long long>(gp.base + cell_offset(gp, A.cg, cell) + 2LL * A.offs_extra + 2 * ch0);
  }
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
  if (A.nchunks > 0) fetch(0, 0);
  stage_rows32(smem + XS, A.x, A.xrow0, A.nx, A.n, ch0, A.cg, cell);
  stage_rows32(smem + YS, A.y, A.yrow0, A.ny, A.n, ch0, A.cg, cell);
  for (int e = threadIdx.x; e < 64 * (A.xrows + A.yrows); e += blockDim.x) smem[AX + e] = 0.f;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const bool ok = ch0 + lane < A.n;
  const bool do_x = A.do_x != 0, do_y = A.do_y != 0;
  for (int c = 0; c < A.nchunks; c++) {
    const int buf = c & 1;
    if (c + 1 < A.nchunks) {
      fetch(c + 1, buf ^ 1);
      __pipeline_wait_prior(1);
    } else {
      __pipeline_wait_prior(0);
    }
    __syncthreads();
    const int nit = __ldg(A.chunks + 8 * c);
    const int CB = BUF + buf * kBufFloats, RB = CB + kCoefCap;
    for (int it = warp; it < nit; it += nwarps) {
      const int rec = RB + 4 * __float_as_int(smem[RB + it]);
      const int4 h = *reinterpret_cast<const int4*>(&smem[rec]);
      const int nl = h.x & 255, band = (h.x >> 8) & 255, nlp = h.x >> 16;
      const int xr = h.y & 0xffff, yr = h.y >> 16;
      const int xi = XS + 64 * xr + 2 * lane, yi = YS + 64 * yr + 2 * lane;
      const int axi = AX + 64 * xr + lane, ayi = AY + 64 * yr + lane;
      for (int j0 = 0; j0 < nl; j0 += 12) {
        const int ng = min(3, (nlp - j0) >> 2);
        if (ng == 1) run_item<1>(smem, gbase, rec, nl, band, nlp, xi, yi, axi, ayi, CB + h.z, j0, lane, ok, do_x, do_y);
        else if (ng == 2) run_item<2>(smem, gbase, rec, nl, band, nlp, xi, yi, axi, ayi, CB + h.z, j0, lane, ok, do_x, do_y);
        else run_item<3>(smem, gbase, rec, nl, band, nlp, xi, yi, axi, ayi, CB + h.z, j0, lane, ok, do_x, do_y);
      }
    }
    __syncthreads();
  }
  if (do_x) flush_rows32(smem + AX, A.xg, A.xrow0, A.nx, A.n, ch0, A.cg, cell, A.x_atomic != 0);
  if (do_y) flush_rows32(smem + AY, A.yg, A.yrow0, A.ny, A.n, ch0, A.cg, cell, A.y_atomic != 0);
}

}  // namespace

// Shares the plan (records, chunks) with the forward kernel: same key family and builder.
DevicePlan* diag_cell_plan(const VecCall& c, const std::vector<int>& xrow0, const std::vector<int>& yrow0);

int launch_diag_bwd_fast(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addDiagCGproduct_back";
  if (c.x.empty() || c.y.empty() || c.r.empty()) return -1;
  const int n = c.x[0].n;
  for (const auto& p : c.x) if (p.n != n || p.l > 60) return -1;
  for (const auto& p : c.y) if (p.n != n || p.l > 60) return -1;
  if (n <= 16) return -1;
  DiagBwdArgs a;
  std::vector<int> xrow0, yrow0;
  int row = 0;
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    if (!c.xg.empty()) a.xg[i] = c.xg[i];
    a.xrow0[i] = row;
    xrow0.push_back(row);
    row += 2 * c.x[i].l + 1;
  }
  a.xrows = row;
  row = 0;
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    if (!c.yg.empty()) a.yg[i] = c.yg[i];
    a.yrow0[i] = row;
    yrow0.push_back(row);
    row += 2 * c.y[i].l + 1;
  }
  a.yrows = row;
  for (size_t i = 0; i < c.r.size(); i++) {
    a.g[i] = c.r[i];
    if (c.r[i].sm != 2LL * c.r[i].n) return -1;  // the records assume dense rows
  }
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.ng = (int)c.r.size();
  a.n = n;
  const size_t smem = ((size_t)2 * kMaxParts + 128 * (a.xrows + a.yrows) + 2 * kBufFloats) * sizeof(float);
  if (smem > 220 * 1024) return -1;
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
  a.do_x = c.xg.empty() ? 0 : 1;
  a.do_y = c.yg.empty() ? 0 : 1;
  a.x_atomic = c.xg_bcast ? 1 : 0;
  a.y_atomic = c.yg_bcast ? 1 : 0;
  const int slices = (n + 31) / 32;
  if (c.cg.ncells > 0x7fffffffLL || slices > 65535) return -1;
  const dim3 grid((unsigned)c.cg.ncells, (unsigned)slices);
  cudaError_t e = cudaFuncSetAttribute(diag_bwd_cell_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) diag_bwd_cell_kernel<<<grid, 256, smem, s>>>(a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "diag backward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
