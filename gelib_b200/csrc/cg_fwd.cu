// Forward Clebsch-Gordan product, all (l1,l2)->l triples of a call in one launch (sm_100a).
//
//   r_l[cell, m, offs + n1*N2 + n2] (+)= sum_{m1} C[m1, m-m1] x_l1[cell, m1, n1] y_l2[cell, m-m1, n2]
//
// Replaces SO3part_addCGproduct_kernel / _tiled_kernel (cuda/SO3part_addCGproduct.cu:59-178 of GElib)
// and the launch-per-triple loop of Gvec::add_CGproduct (core/Gvec.hpp:311-321).
//
// Data movement.  The output is the only large stream (x and y are a few KB per cell), so the kernel
// is organised around writing r exactly once with full-width stores:
//   * a CTA owns WC cells; it stages every x and y part of those cells in shared memory once;
//   * each warp then takes work items (triple, n1-tile, n2-tile) from the CTA's job, round robin.  For
//     an item a lane owns TA consecutive n1 and two pairs of adjacent n2 (2*lb, 2*lb+1 and the same
//     shifted by 2*NBL) of one cell, so that eight lanes write 128 contiguous bytes per store;
//   * per output row m the lane accumulates the band sum over m1 in registers (TA x 4 complex), with
//     the coefficient folded into x once per (m1, n1) and reused over the four n2;
//   * the row is then stored with streaming 16-byte stores (or read-modify-written when accumulating).
// No thread ever needs another thread's partial result: there are no shuffles, atomics or barriers
// after the staging barrier.
#include <algorithm>
#include <cstdlib>
#include <string>

#include "plan.h"

namespace gelib_b200 {

namespace {

struct FwdArgs {
  PartView x[kMaxParts], y[kMaxParts], r[kMaxParts];
  int xoff[kMaxParts], yoff[kMaxParts];  // float offset of each part inside a cell's shared-memory block
  int xnp[kMaxParts], ynp[kMaxParts];    // padded channel counts (complex) of the staged rows
  int nx, ny, nr;
  int cell_floats;                       // shared-memory floats per cell (x block then y block)
  CellGrid cg;
  const Triple* triples;
  const float* coeffs;
  const int4* items;
  const int* jobs;
  int offs_extra;
  int accumulate;
};

__device__ __forceinline__ void store2(float* p, float a, float b, bool acc) {
  float2 v = make_float2(a, b);
  if (acc) {
    const float2 o = *reinterpret_cast<const float2*>(p);
    v.x += o.x;
    v.y += o.y;
    *reinterpret_cast<float2*>(p) = v;
  } else {
    __stcs(reinterpret_cast<float2*>(p), v);
  }
}

__device__ __forceinline__ void store4(float* p, const float* a, bool acc) {
  float4 v = make_float4(a[0], a[1], a[2], a[3]);
  if (acc) {
    const float4 o = *reinterpret_cast<const float4*>(p);
    v.x += o.x;
    v.y += o.y;
    v.z += o.z;
    v.w += o.w;
    *reinterpret_cast<float4*>(p) = v;
  } else {
    __stcs(reinterpret_cast<float4*>(p), v);
  }
}

// Copies the parts of `n` vectors' cells into shared memory: rows of np complex, channel-dense.
__device__ __forceinline__ void stage_parts(float* dst_cell, const PartView* parts, const int* off, const int* np,
                                            int nparts, const CellGrid& cg, long long cell) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = parts[i];
    const float* src = p.base + cell_offset(p, cg, cell);
    float* dst = dst_cell + off[i];
    const int n = p.n, rows = 2 * p.l + 1, npad = np[i];
    const int total = rows * n;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int m = e / n, ch = e - m * n;
      const float2 v = __ldg(reinterpret_cast<const float2*>(src + (long long)m * p.sm + 2 * ch));
      *reinterpret_cast<float2*>(dst + 2 * (m * npad + ch)) = v;
    }
  }
}

template <int TA, int WA, int NBL, bool VEC>
__global__ void __launch_bounds__(128) cg_fwd_kernel(const __grid_constant__ FwdArgs A) {
  constexpr int WC = 32 / (WA * NBL);
  static_assert(WC * WA * NBL == 32, "lane layout must fill a warp");
  extern __shared__ __align__(16) float smem_raw[];
  long long* roff = reinterpret_cast<long long*>(smem_raw);  // [WC][kMaxParts] output offsets of the CTA's cells
  float* smem = smem_raw + 2 * WC * kMaxParts;

  const long long cell0 = (long long)blockIdx.x * WC;
  fill_cell_offsets(roff, A.r, A.nr, A.cg, cell0, WC);
  for (int c = 0; c < WC; c++) {
    const long long cell = cell0 + c;
    if (cell >= A.cg.ncells) break;
    float* blk = smem + (size_t)c * A.cell_floats;
    stage_parts(blk, A.x, A.xoff, A.xnp, A.nx, A.cg, cell);
    stage_parts(blk, A.y, A.yoff, A.ynp, A.ny, A.cg, cell);
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int lb = lane % NBL, la = (lane / NBL) % WA, lc = lane / (NBL * WA);
  const long long cell = cell0 + lc;
  const bool cell_ok = cell < A.cg.ncells;
  const float* blk = smem + (size_t)lc * A.cell_floats;
  const bool acc_mode = A.accumulate != 0;

  const int it1 = A.jobs[blockIdx.y + 1];
  for (int it = A.jobs[blockIdx.y] + warp; it < it1; it += nwarps) {
    const int4 item = __ldg(&A.items[it]);
    const Triple t = A.triples[item.x];
    const int l1 = t.l1, l2 = t.l2, l = t.l;
    const PartView& rp = A.r[t.ri];
    const int n1 = A.x[t.xi].n, n2 = A.y[t.yi].n;
    const int n1p = A.xnp[t.xi], n2p = A.ynp[t.yi];
    const int i0 = item.y + la * TA;
    const int j0 = item.z + 2 * lb, j1 = j0 + 2 * NBL;
    const float* xs = blk + A.xoff[t.xi] + 2 * i0;
    const float* ys = blk + A.yoff[t.yi];
    const float* cp = A.coeffs + t.coff;
    float* rbase = rp.base + roff[lc * kMaxParts + t.ri] + 2LL * (t.offs + A.offs_extra);

    for (int m = -l; m <= l; m++) {
      const int lo = max(-l1, m - l2), hi = min(l1, m + l2);
      float acc[TA][8];
#pragma unroll
      for (int a = 0; a < TA; a++)
#pragma unroll
        for (int k = 0; k < 8; k++) acc[a][k] = 0.f;

      const float* xq = xs + 2 * (lo + l1) * n1p;
      const float* yq = ys + 2 * (m - lo + l2) * n2p;
#pragma unroll 2
      for (int m1 = lo; m1 <= hi; m1++) {
        const float c = __ldg(cp++);
        float xv[2 * TA];
        if constexpr (TA == 1) {
          const float2 v = *reinterpret_cast<const float2*>(xq);
          xv[0] = v.x; xv[1] = v.y;
        } else {
#pragma unroll
          for (int a = 0; a < TA; a += 2) {
            const float4 v = *reinterpret_cast<const float4*>(xq + 2 * a);
            xv[2 * a] = v.x; xv[2 * a + 1] = v.y; xv[2 * a + 2] = v.z; xv[2 * a + 3] = v.w;
          }
        }
        const float4 y0 = *reinterpret_cast<const float4*>(yq + 2 * j0);
        const float4 y1 = *reinterpret_cast<const float4*>(yq + 2 * j1);
#pragma unroll
        for (int a = 0; a < TA; a++) {
          const float xr = c * xv[2 * a], xi = c * xv[2 * a + 1];
          acc[a][0] = fmaf(xr, y0.x, acc[a][0]); acc[a][0] = fmaf(-xi, y0.y, acc[a][0]);
          acc[a][1] = fmaf(xr, y0.y, acc[a][1]); acc[a][1] = fmaf(xi, y0.x, acc[a][1]);
          acc[a][2] = fmaf(xr, y0.z, acc[a][2]); acc[a][2] = fmaf(-xi, y0.w, acc[a][2]);
          acc[a][3] = fmaf(xr, y0.w, acc[a][3]); acc[a][3] = fmaf(xi, y0.z, acc[a][3]);
          acc[a][4] = fmaf(xr, y1.x, acc[a][4]); acc[a][4] = fmaf(-xi, y1.y, acc[a][4]);
          acc[a][5] = fmaf(xr, y1.y, acc[a][5]); acc[a][5] = fmaf(xi, y1.x, acc[a][5]);
          acc[a][6] = fmaf(xr, y1.z, acc[a][6]); acc[a][6] = fmaf(-xi, y1.w, acc[a][6]);
          acc[a][7] = fmaf(xr, y1.w, acc[a][7]); acc[a][7] = fmaf(xi, y1.z, acc[a][7]);
        }
        xq += 2 * n1p;
        yq -= 2 * n2p;
      }

      if (cell_ok) {
        float* rrow = rbase + (long long)(m + l) * rp.sm;
#pragma unroll
        for (int a = 0; a < TA; a++) {
          const int n1i = i0 + a;
          if (n1i < n1) {
            float* p = rrow + 2LL * n1i * n2;
            if constexpr (VEC) {
              if (j0 < n2) store4(p + 2 * j0, &acc[a][0], acc_mode);
              if (j1 < n2) store4(p + 2 * j1, &acc[a][4], acc_mode);
            } else {
              if (j0 < n2) store2(p + 2 * j0, acc[a][0], acc[a][1], acc_mode);
              if (j0 + 1 < n2) store2(p + 2 * j0 + 2, acc[a][2], acc[a][3], acc_mode);
              if (j1 < n2) store2(p + 2 * j1, acc[a][4], acc[a][5], acc_mode);
              if (j1 + 1 < n2) store2(p + 2 * j1 + 2, acc[a][6], acc[a][7], acc_mode);
            }
          }
        }
      }
    }
  }
}

struct TileCfg {
  int TA, WA, NBL;
};
constexpr TileCfg kCfgs[] = {
    {4, 4, 8},  // 16 x 32 channels, 1 cell per warp
    {2, 4, 8},  //  8 x 32, 1 cell
    {1, 1, 4},  //  1 x 16, 8 cells
    {2, 2, 2},  //  4 x  8, 8 cells
    {1, 1, 1},  //  1 x  4, 32 cells
    {4, 4, 1},  // 16 x  4, 8 cells
};
constexpr int kNumCfgs = sizeof(kCfgs) / sizeof(kCfgs[0]);

template <int TA, int WA, int NBL>
cudaError_t launch_cfg(const FwdArgs& a, dim3 grid, size_t smem, bool vec, cudaStream_t s) {
  auto k = vec ? cg_fwd_kernel<TA, WA, NBL, true> : cg_fwd_kernel<TA, WA, NBL, false>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  k<<<grid, 128, smem, s>>>(a);
  return cudaGetLastError();
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace

int launch_cg_fwd(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addCGproduct";
  // Calls that qualify (channel counts that are multiples of 32, output overwritten) and have at least 512 slabs
  // (rows of 32 x 32 channel tiles) per cell -- 240 when it can use tensor stores -- go to the tensor-core kernel of
  // cg_fwd_tc.cu: with fewer its fixed
  // cost per cell (staging the y tables, tensor-memory allocation) outweighs its cheaper slabs.
  // Option "fwd" (initially GELIB_B200_FWD): "simt" keeps everything on this file's kernel, "tcgen05" sends
  // everything that qualifies there, "tcgen05!" also refuses calls that do not qualify (tests use it to be sure which
  // kernel ran).
  const int mode = fwd_mode();
  if (mode != kFwdSimt) {
    // with tensor stores (every y part the same channel count) the crossover measured is lower: 252 slabs per cell
    // (l1 = 3 x l2 = 4, 64 channels) 1.36 against 1.59 ms, 375 (maxl 4 x 32) a tie, 204 (maxl 2 x 64) 2.35 against 2.14
    bool uniform = pair_tma() && c.offs_extra == 0 && !c.y.empty();
    for (const auto& p : c.y) uniform = uniform && p.n == c.y[0].n;
    const int rc = launch_cg_fwd_tc(c, s, mode == kFwdAuto ? (uniform ? 240 : 512) : 0);
    if (rc != -1) return rc;
    if (mode == kFwdTcStrict) return fail(GELIB_INVALID, fn, "the call does not qualify for the tcgen05 kernel");
  }
  // ---- choose the lane layout: least padded work on the dominant channel counts, then the widest tile
  int n1 = 1, n2 = 1;
  for (const auto& p : c.x) n1 = std::max(n1, p.n);
  for (const auto& p : c.y) n2 = std::max(n2, p.n);
  int best = 0;
  double best_cost = 1e300;
  for (int i = 0; i < kNumCfgs; i++) {
    const int ta = kCfgs[i].TA * kCfgs[i].WA, tb = 4 * kCfgs[i].NBL;
    const double cost = (double)ceil_div(n1, ta) * ta * ceil_div(n2, tb) * tb;
    if (cost < best_cost * 0.999) {
      best_cost = cost;
      best = i;
    }
  }
  const TileCfg cfg = kCfgs[best];
  const int WC = 32 / (cfg.WA * cfg.NBL);
  const int tile_a = cfg.TA * cfg.WA, tile_b = 4 * cfg.NBL;

  // ---- shared-memory layout of one cell
  FwdArgs a;
  int off = 0;
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    a.xnp[i] = ceil_div(c.x[i].n, 4) * 4;
    a.xoff[i] = off;
    off += 2 * (2 * c.x[i].l + 1) * a.xnp[i];
  }
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    a.ynp[i] = ceil_div(c.y[i].n, 4) * 4;
    a.yoff[i] = off;
    off += 2 * (2 * c.y[i].l + 1) * a.ynp[i];
  }
  for (size_t i = 0; i < c.r.size(); i++) a.r[i] = c.r[i];
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.nr = (int)c.r.size();
  a.cell_floats = off;
  const size_t smem = ((size_t)off * WC + 128 + 2 * WC * kMaxParts) * sizeof(float);  // +128 floats: tiles may read past the last row
  if (smem > 200 * 1024) return -1;                             // caller falls back to the strided kernel

  // ---- jobs: enough CTAs to fill the machine several times over
  const long long groups = (c.cg.ncells + WC - 1) / WC;
  int njobs = 1;
  if (groups < 16384) njobs = (int)std::min<long long>(16, (16384 + groups - 1) / groups);

  std::vector<int> key = {1 /*family*/, best, njobs, (int)c.x.size(), (int)c.y.size(), (int)c.r.size()};
  for (const auto& p : c.x) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.y) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.r) key.push_back(p.l);
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  DevicePlan* plan = get_plan(key, [&](DevicePlan& p) {
    build_schedule(xs, ys, rs, false, true, &p.sched);
    std::vector<long long> cost;
    for (size_t ti = 0; ti < p.sched.triples.size(); ti++) {
      const Triple& t = p.sched.triples[ti];
      const int T = band_size(t.l1, t.l2, t.l);
      for (int a0 = 0; a0 < xs[t.xi].n; a0 += tile_a)
        for (int b0 = 0; b0 < ys[t.yi].n; b0 += tile_b) {
          p.h_items.push_back(make_int4((int)ti, a0, b0, 0));
          cost.push_back(T + 2 * (2 * t.l + 1));
        }
    }
    long long total = 0;
    for (long long v : cost) total += v;
    const int nj = std::max(1, std::min<int>(njobs, (int)p.h_items.size() / 4));
    p.h_jobs.push_back(0);
    long long run = 0;
    for (size_t i = 0; i < cost.size(); i++) {
      run += cost[i];
      if ((int)p.h_jobs.size() < nj && run * nj >= total * (long long)p.h_jobs.size()) p.h_jobs.push_back((int)i + 1);
    }
    while ((int)p.h_jobs.size() < nj + 1) p.h_jobs.push_back((int)cost.size());
    p.h_jobs.back() = (int)cost.size();
  });
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->nitems == 0 || c.cg.ncells == 0) return GELIB_OK;

  a.cg = c.cg;
  a.triples = plan->triples;
  a.coeffs = plan->coeffs;
  a.items = plan->items;
  a.jobs = plan->jobs;
  a.offs_extra = c.offs_extra;
  a.accumulate = (c.flags & GELIB_OVERWRITE) ? 0 : 1;

  if (groups > 0x7fffffffLL) return fail(GELIB_SKIPPED, fn, "number of cells exceeds 2^31-1");
  const dim3 grid((unsigned)groups, (unsigned)plan->njobs);
  cudaError_t e = cudaSuccess;
  switch (best) {
    case 0: e = launch_cfg<4, 4, 8>(a, grid, smem, c.vec_ok, s); break;
    case 1: e = launch_cfg<2, 4, 8>(a, grid, smem, c.vec_ok, s); break;
    case 2: e = launch_cfg<1, 1, 4>(a, grid, smem, c.vec_ok, s); break;
    case 3: e = launch_cfg<2, 2, 2>(a, grid, smem, c.vec_ok, s); break;
    case 4: e = launch_cfg<1, 1, 1>(a, grid, smem, c.vec_ok, s); break;
    default: e = launch_cfg<4, 4, 1>(a, grid, smem, c.vec_ok, s); break;
  }
  if (e != cudaSuccess) return check_cuda(e, fn, "forward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
