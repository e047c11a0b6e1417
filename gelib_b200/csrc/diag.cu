// Diagonal Clebsch-Gordan product (channels paired n <-> n) and its gradients, fused over all triples.
//
//   r_l[cell, m, offs_l + n] (+)= sum_{m1} C_l[m1, m-m1] x_l1[cell, m1, n] y_l2[cell, m-m1, n]
//
// GElib has no GPU version of these (the declarations are commented out, SO3/SO3part.hpp:36-38, and the
// device trampolines are empty, SO3/SO3part.hpp:324-334); the semantics are those of its CPU loops
// SO3/SO3part.hpp:276-322 and of Gvec::add_DiagCGproduct / _back0 / _back1 (core/Gvec.hpp:358-389).
//
// The product is elementwise in the channel, so there is no channel tile to reuse operands over.  The
// reuse comes from l instead: the products p[m1,m2] = x[m1] y[m2] do not depend on the output l, and for
// a fixed (l1,l2,m) the band of m1 is the same for every l.  A work item is therefore one (l1,l2) pair
// and one output row index m; a lane owns one channel of one cell, forms each p once and feeds it to the
// accumulators of all output l at once (2 FMAs per term instead of 4).  The coefficients of an item are
// stored as a dense [m1][l] table (padded to a multiple of 4 in l) and read with 16-byte uniform loads.
// A CTA stages one slice of CW channels of every x and y part of WC cells in shared memory; rows of the
// outputs are written as contiguous runs of CW complex numbers.
//
// Backward: G[m1,m2] = sum_l C_l[m1,m2] g_l[m1+m2] is formed from registers holding the g rows of all l,
// then xg[m1] += G conj(y[m2]) and yg[m2] += G conj(x[m1]) go to per-warp shared-memory accumulators that
// are combined in warp order at the end of each (l1,l2) pair (deterministic, no atomics unless an
// output is broadcast over cells).
#include <algorithm>

#include "plan.h"

namespace gelib_b200 {

namespace {

struct DiagArgs {
  PartView x[kMaxParts], y[kMaxParts], r[kMaxParts], xg[kMaxParts], yg[kMaxParts];
  int xrow0[kMaxParts], yrow0[kMaxParts];  // first staged row of each part
  int nx, ny;
  int xrows, yrows;   // staged rows per cell
  int n;              // channels (same for every part)
  int CW, WC;         // channels per warp row (power of two <= 32), cells per warp = 32 / CW
  CellGrid cg;
  const Triple* triples;
  const float* coeffs;
  const int4* items;  // x: first triple | nl << 16, y: m, z: coefficient offset, w: nlp (padded nl)
  const int* jobs;    // forward: job ranges; backward: phases (one per (l1,l2) pair)
  int njobs;
  int job_stride;     // forward: CTA z walks pairs [z*job_stride, (z+1)*job_stride)
  int offs_extra;
  int accumulate;
  int do_x, do_y, x_atomic, y_atomic;
  int priv_floats;    // floats of one warp's private accumulator for one side
};

__device__ __forceinline__ void stage_slice(float* dst, const PartView* parts, const int* row0, int nparts, int rows,
                                            int CW, int WC, int n, int ch0, const CellGrid& cg, long long cell0) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = parts[i];
    const int prow = 2 * p.l + 1;
    const int total = WC * prow * CW;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int ch = e % CW, q = e / CW;
      const int m = q % prow, c = q / prow;
      const long long cell = cell0 + c;
      float2 v = make_float2(0.f, 0.f);
      if (cell < cg.ncells && ch0 + ch < n)
        v = __ldg(reinterpret_cast<const float2*>(p.base + cell_offset(p, cg, cell) + (long long)m * p.sm +
                                                   2LL * (ch0 + ch)));
      *reinterpret_cast<float2*>(dst + 2 * ((size_t)(c * rows + row0[i] + m) * CW + ch)) = v;
    }
  }
}

template <int NLC>
__global__ void __launch_bounds__(128) diag_fwd_kernel(const __grid_constant__ DiagArgs A) {
  extern __shared__ __align__(16) float smem[];
  const int CW = A.CW, WC = A.WC;
  const long long cell0 = (long long)blockIdx.x * WC;
  const int ch0 = blockIdx.y * CW;
  float* xs_all = smem;
  float* ys_all = smem + (size_t)2 * WC * A.xrows * CW;
  stage_slice(xs_all, A.x, A.xrow0, A.nx, A.xrows, CW, WC, A.n, ch0, A.cg, cell0);
  stage_slice(ys_all, A.y, A.yrow0, A.ny, A.yrows, CW, WC, A.n, ch0, A.cg, cell0);
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int lc = lane / CW, ch = lane % CW;
  const long long cell = cell0 + lc;
  const int chan = ch0 + ch;
  const bool ok = cell < A.cg.ncells && chan < A.n;
  const float* xs = xs_all + 2 * ((size_t)lc * A.xrows * CW + ch);
  const float* ys = ys_all + 2 * ((size_t)lc * A.yrows * CW + ch);
  const bool acc_mode = A.accumulate != 0;

  const int it1 = A.jobs[min((int)(blockIdx.z + 1) * A.job_stride, A.njobs)];
  for (int it = A.jobs[blockIdx.z * A.job_stride] + warp; it < it1; it += nwarps) {
    const int4 item = __ldg(&A.items[it]);
    const int tfirst = item.x & 0xffff, nl = item.x >> 16, m = item.y, nlp = item.w;
    const Triple t0 = A.triples[tfirst];
    const int l1 = t0.l1, l2 = t0.l2;
    const int lo = max(-l1, m - l2), hi = min(l1, m + l2);
    const float* xrow = xs + 2 * (size_t)(A.xrow0[t0.xi] + lo + l1) * CW;
    const float* yrow = ys + 2 * (size_t)(A.yrow0[t0.yi] + m - lo + l2) * CW;
    for (int j0 = 0; j0 < nl; j0 += NLC) {
      float acc[NLC][2];
#pragma unroll
      for (int j = 0; j < NLC; j++) acc[j][0] = acc[j][1] = 0.f;
      const float* cptr = A.coeffs + item.z + j0;
      const float* xq = xrow;
      const float* yq = yrow;
      for (int m1 = lo; m1 <= hi; m1++) {
        const float2 xv = *reinterpret_cast<const float2*>(xq);
        const float2 yv = *reinterpret_cast<const float2*>(yq);
        const float pr = xv.x * yv.x - xv.y * yv.y, pi = xv.x * yv.y + xv.y * yv.x;
#pragma unroll
        for (int k = 0; k < NLC / 4; k++) {
          if (j0 + 4 * k < nlp) {
            const float4 c = __ldg(reinterpret_cast<const float4*>(cptr) + k);
            acc[4 * k + 0][0] = fmaf(c.x, pr, acc[4 * k + 0][0]); acc[4 * k + 0][1] = fmaf(c.x, pi, acc[4 * k + 0][1]);
            acc[4 * k + 1][0] = fmaf(c.y, pr, acc[4 * k + 1][0]); acc[4 * k + 1][1] = fmaf(c.y, pi, acc[4 * k + 1][1]);
            acc[4 * k + 2][0] = fmaf(c.z, pr, acc[4 * k + 2][0]); acc[4 * k + 2][1] = fmaf(c.z, pi, acc[4 * k + 2][1]);
            acc[4 * k + 3][0] = fmaf(c.w, pr, acc[4 * k + 3][0]); acc[4 * k + 3][1] = fmaf(c.w, pi, acc[4 * k + 3][1]);
          }
        }
        cptr += nlp;
        xq += 2 * CW;
        yq -= 2 * CW;
      }
      if (ok) {
#pragma unroll
        for (int j = 0; j < NLC; j++) {
          if (j0 + j < nl) {
            const Triple t = A.triples[tfirst + j0 + j];
            const PartView& rp = A.r[t.ri];
            float* p = rp.base + cell_offset(rp, A.cg, cell) + (long long)(m + t.l) * rp.sm +
                       2LL * (t.offs + A.offs_extra + chan);
            float2 v = make_float2(acc[j][0], acc[j][1]);
            if (acc_mode) {
              const float2 o = *reinterpret_cast<const float2*>(p);
              v.x += o.x;
              v.y += o.y;
              *reinterpret_cast<float2*>(p) = v;
            } else {
              __stcs(reinterpret_cast<float2*>(p), v);
            }
          }
        }
      }
    }
  }
}

__device__ __forceinline__ void diag_flush(const float* priv, int priv_stride, int nwarps, const PartView& out, int CW,
                                           int WC, int n, int ch0, long long cell0, const CellGrid& cg, bool atomic) {
  const int rows = 2 * out.l + 1;
  const int total = WC * rows * CW;
  for (int e = threadIdx.x; e < total; e += blockDim.x) {
    const int ch = e % CW, q = e / CW;
    const int row = q % rows, c = q / rows;
    const long long cell = cell0 + c;
    if (cell >= cg.ncells || ch0 + ch >= n) continue;
    float sr = 0.f, si = 0.f;
    for (int w = 0; w < nwarps; w++) {
      const float2 v = *reinterpret_cast<const float2*>(priv + (size_t)w * priv_stride + 2 * e);
      sr += v.x;
      si += v.y;
    }
    float* p = out.base + cell_offset(out, cg, cell) + (long long)row * out.sm + 2LL * (ch0 + ch);
    if (atomic) {
      atomicAdd(p, sr);
      atomicAdd(p + 1, si);
    } else {
      float2 o = *reinterpret_cast<float2*>(p);
      o.x += sr;
      o.y += si;
      *reinterpret_cast<float2*>(p) = o;
    }
  }
}

template <int NLC>
__global__ void __launch_bounds__(256) diag_bwd_kernel(const __grid_constant__ DiagArgs A) {
  extern __shared__ __align__(16) float smem[];
  const int CW = A.CW, WC = A.WC;
  const long long cell0 = (long long)blockIdx.x * WC;
  const int ch0 = blockIdx.y * CW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float* xs_all = smem;
  float* ys_all = xs_all + (size_t)2 * WC * A.xrows * CW;
  float* privx = ys_all + (size_t)2 * WC * A.yrows * CW;
  float* privy = privx + (size_t)nwarps * A.priv_floats;
  stage_slice(xs_all, A.x, A.xrow0, A.nx, A.xrows, CW, WC, A.n, ch0, A.cg, cell0);
  stage_slice(ys_all, A.y, A.yrow0, A.ny, A.yrows, CW, WC, A.n, ch0, A.cg, cell0);

  const int lc = lane / CW, ch = lane % CW;
  const long long cell = cell0 + lc;
  const int chan = ch0 + ch;
  const bool ok = cell < A.cg.ncells && chan < A.n;
  const float* xs = xs_all + 2 * ((size_t)lc * A.xrows * CW + ch);
  const float* ys = ys_all + 2 * ((size_t)lc * A.yrows * CW + ch);
  float* mypx = privx + (size_t)warp * A.priv_floats;
  float* mypy = privy + (size_t)warp * A.priv_floats;

  int cur_xi = -1;
  for (int ph = 0; ph < A.njobs; ph++) {
    const int ib = A.jobs[ph], ie = A.jobs[ph + 1];
    const Triple t0 = A.triples[A.items[ib].x & 0xffff];
    const int xi = t0.xi, yi = t0.yi, l1 = t0.l1, l2 = t0.l2;
    if (xi != cur_xi) {
      for (int e = lane; e < 2 * WC * (2 * l1 + 1) * CW; e += 32) mypx[e] = 0.f;
      cur_xi = xi;
    }
    for (int e = lane; e < 2 * WC * (2 * l2 + 1) * CW; e += 32) mypy[e] = 0.f;
    if (ph == 0) __syncthreads();
    else __syncwarp();
    // lane-private slots: [cell lc][row][ch]
    float* pxl = mypx + 2 * ((size_t)lc * (2 * l1 + 1) * CW + ch);
    float* pyl = mypy + 2 * ((size_t)lc * (2 * l2 + 1) * CW + ch);

    for (int it = ib + warp; it < ie; it += nwarps) {
      const int4 item = __ldg(&A.items[it]);
      const int tfirst = item.x & 0xffff, nl = item.x >> 16, m = item.y, nlp = item.w;
      const int lo = max(-l1, m - l2), hi = min(l1, m + l2);
      const float* xrow = xs + 2 * (size_t)(A.xrow0[xi] + lo + l1) * CW;
      const float* yrow = ys + 2 * (size_t)(A.yrow0[yi] + m - lo + l2) * CW;
      for (int j0 = 0; j0 < nl; j0 += NLC) {
        float gv[NLC][2];
#pragma unroll
        for (int j = 0; j < NLC; j++) {
          gv[j][0] = gv[j][1] = 0.f;
          if (ok && j0 + j < nl) {
            const Triple t = A.triples[tfirst + j0 + j];
            const PartView& gp = A.r[t.ri];
            const float2 v = __ldcs(reinterpret_cast<const float2*>(gp.base + cell_offset(gp, A.cg, cell) +
                                                                    (long long)(m + t.l) * gp.sm +
                                                                    2LL * (t.offs + A.offs_extra + chan)));
            gv[j][0] = v.x;
            gv[j][1] = v.y;
          }
        }
        const float* cptr = A.coeffs + item.z + j0;
        const float* xq = xrow;
        const float* yq = yrow;
        for (int m1 = lo; m1 <= hi; m1++) {
          float Gr = 0.f, Gi = 0.f;
#pragma unroll
          for (int k = 0; k < NLC / 4; k++) {
            if (j0 + 4 * k < nlp) {
              const float4 c = __ldg(reinterpret_cast<const float4*>(cptr) + k);
              Gr = fmaf(c.x, gv[4 * k][0], Gr); Gi = fmaf(c.x, gv[4 * k][1], Gi);
              Gr = fmaf(c.y, gv[4 * k + 1][0], Gr); Gi = fmaf(c.y, gv[4 * k + 1][1], Gi);
              Gr = fmaf(c.z, gv[4 * k + 2][0], Gr); Gi = fmaf(c.z, gv[4 * k + 2][1], Gi);
              Gr = fmaf(c.w, gv[4 * k + 3][0], Gr); Gi = fmaf(c.w, gv[4 * k + 3][1], Gi);
            }
          }
          const float2 xv = *reinterpret_cast<const float2*>(xq);
          const float2 yv = *reinterpret_cast<const float2*>(yq);
          if (A.do_x) {
            float2* p = reinterpret_cast<float2*>(pxl + 2 * (size_t)(m1 + l1) * CW);
            float2 o = *p;
            o.x = fmaf(Gr, yv.x, o.x); o.x = fmaf(Gi, yv.y, o.x);
            o.y = fmaf(Gi, yv.x, o.y); o.y = fmaf(-Gr, yv.y, o.y);
            *p = o;
          }
          if (A.do_y) {
            float2* p = reinterpret_cast<float2*>(pyl + 2 * (size_t)(m - m1 + l2) * CW);
            float2 o = *p;
            o.x = fmaf(Gr, xv.x, o.x); o.x = fmaf(Gi, xv.y, o.x);
            o.y = fmaf(Gi, xv.x, o.y); o.y = fmaf(-Gr, xv.y, o.y);
            *p = o;
          }
          cptr += nlp;
          xq += 2 * CW;
          yq -= 2 * CW;
        }
      }
    }

    const bool last_of_x = (ph + 1 == A.njobs) || (A.triples[A.items[A.jobs[ph + 1]].x & 0xffff].xi != xi);
    __syncthreads();
    if (A.do_y) diag_flush(privy, A.priv_floats, nwarps, A.yg[yi], CW, WC, A.n, ch0, cell0, A.cg, A.y_atomic != 0);
    if (A.do_x && last_of_x) {
      diag_flush(privx, A.priv_floats, nwarps, A.xg[xi], CW, WC, A.n, ch0, cell0, A.cg, A.x_atomic != 0);
      cur_xi = -1;
    }
    __syncthreads();
  }
}

}  // namespace

// Items of a diagonal product: for every (xi, yi) pair (a maximal run of the schedule) and every row
// index m reachable by some l, the dense coefficient table [m1 in band][l among the valid ones].
void build_diag_items(DevicePlan& p, const std::vector<PartSig>& xs, const std::vector<PartSig>& ys,
                      const std::vector<PartSig>& rs, int* max_nl) {
  build_schedule(xs, ys, rs, true, false, &p.sched);
  const auto& tr = p.sched.triples;
  *max_nl = 0;
  p.h_jobs.push_back(0);
  size_t ti = 0;
  while (ti < tr.size()) {
    size_t tj = ti;
    while (tj < tr.size() && tr[tj].xi == tr[ti].xi && tr[tj].yi == tr[ti].yi) tj++;
    const int l1 = tr[ti].l1, l2 = tr[ti].l2;
    const int lmax = tr[tj - 1].l;  // triples of a pair are in ascending l
    struct It { int4 v; int cost; };
    std::vector<It> its;
    for (int m = -lmax; m <= lmax; m++) {
      // valid l: those of the pair with l >= |m|  (a suffix of the run)
      size_t tf = ti;
      while (tf < tj && tr[tf].l < std::abs(m)) tf++;
      const int nl = (int)(tj - tf);
      if (nl == 0) continue;
      const int nlp = (nl + 3) / 4 * 4;
      const int lo = std::max(-l1, m - l2), hi = std::min(l1, m + l2);
      if (hi < lo) continue;
      while (p.sched.coeffs.size() % 4) p.sched.coeffs.push_back(0.f);
      const int coff = (int)p.sched.coeffs.size();
      for (int m1 = lo; m1 <= hi; m1++)
        for (int j = 0; j < nlp; j++)
          p.sched.coeffs.push_back(j < nl ? (float)cg_coefficient(l1, l2, tr[tf + j].l, m1, m - m1) : 0.f);
      its.push_back({make_int4((int)tf | (nl << 16), m, coff, nlp), (hi - lo + 1) * (nl + 4)});
      *max_nl = std::max(*max_nl, nl);
    }
    std::stable_sort(its.begin(), its.end(), [](const It& u, const It& v) { return u.cost > v.cost; });
    for (const auto& it : its) p.h_items.push_back(it.v);
    p.h_jobs.push_back((int)p.h_items.size());
    ti = tj;
  }
}

namespace {

struct DiagSetup {
  DiagArgs a;
  DevicePlan* plan = nullptr;
  int max_nl = 0;
  int status = GELIB_OK;
};

bool same_channels(const VecCall& c, int* n) {
  *n = c.x.empty() ? 0 : c.x[0].n;
  for (const auto& p : c.x) if (p.n != *n) return false;
  for (const auto& p : c.y) if (p.n != *n) return false;
  return true;
}

int setup(const VecCall& c, DiagArgs& a, DevicePlan** plan_out, int* max_nl_out) {
  int n = 0;
  if (!same_channels(c, &n) || n == 0) return -1;
  std::vector<int> key = {4 /*family*/, (int)c.x.size(), (int)c.y.size(), (int)c.r.size(), n};
  for (const auto& p : c.x) key.push_back(p.l);
  for (const auto& p : c.y) key.push_back(p.l);
  for (const auto& p : c.r) key.push_back(p.l);
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  DevicePlan* plan = get_plan(key, [&](DevicePlan& p) {
    int mx = 0;
    build_diag_items(p, xs, ys, rs, &mx);
  });
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->ntriples > 65535) return -1;
  int mx = 0;
  for (const auto& it : plan->h_items) mx = std::max(mx, it.x >> 16);
  *max_nl_out = mx;
  *plan_out = plan;

  int CW = 1;
  while (CW < 32 && CW < n) CW *= 2;
  a.CW = CW;
  a.WC = 32 / CW;
  a.n = n;
  int row = 0;
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    if (!c.xg.empty()) a.xg[i] = c.xg[i];
    a.xrow0[i] = row;
    row += 2 * c.x[i].l + 1;
  }
  a.xrows = row;
  row = 0;
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    if (!c.yg.empty()) a.yg[i] = c.yg[i];
    a.yrow0[i] = row;
    row += 2 * c.y[i].l + 1;
  }
  a.yrows = row;
  for (size_t i = 0; i < c.r.size(); i++) a.r[i] = c.r[i];
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.cg = c.cg;
  a.triples = plan->triples;
  a.coeffs = plan->coeffs;
  a.items = plan->items;
  a.jobs = plan->jobs;
  a.njobs = plan->njobs;
  a.offs_extra = c.offs_extra;
  a.accumulate = (c.flags & GELIB_OVERWRITE) ? 0 : 1;
  a.do_x = c.xg.empty() ? 0 : 1;
  a.do_y = c.yg.empty() ? 0 : 1;
  a.x_atomic = c.xg_bcast ? 1 : 0;
  a.y_atomic = c.yg_bcast ? 1 : 0;
  a.priv_floats = 0;
  a.job_stride = 1;
  return GELIB_OK;
}

}  // namespace

int launch_diag_fwd(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addDiagCGproduct";
  {
    const int st = launch_diag_fwd_fast(c, s);  // one cell per CTA, 32 or 64 channels per warp row
    if (st != -1) return st;
  }
  DiagArgs a;
  DevicePlan* plan = nullptr;
  int max_nl = 0;
  const int st = setup(c, a, &plan, &max_nl);
  if (st != GELIB_OK) return st;
  if (plan->nitems == 0 || c.cg.ncells == 0) return GELIB_OK;
  const size_t smem = (size_t)2 * a.WC * (a.xrows + a.yrows) * a.CW * sizeof(float);
  if (smem > 200 * 1024) return -1;
  const long long groups = (c.cg.ncells + a.WC - 1) / a.WC;
  const int slices = (a.n + a.CW - 1) / a.CW;
  if (groups > 0x7fffffffLL || slices > 65535) return -1;

  // The plan's job table has one entry per (l1,l2) pair.  With many cells one CTA walks all pairs (x and y
  // are staged once); with few cells the pairs are spread over blockIdx.z to fill the machine.
  const long long ctas = groups * slices;
  a.job_stride = (ctas < 4096 && plan->njobs > 1) ? std::max(1, plan->njobs / 16) : plan->njobs;
  const int nz = (plan->njobs + a.job_stride - 1) / a.job_stride;
  const dim3 grid((unsigned)groups, (unsigned)slices, (unsigned)nz);
  cudaError_t e;
  if (max_nl <= 4) {
    e = cudaFuncSetAttribute(diag_fwd_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) diag_fwd_kernel<4><<<grid, 128, smem, s>>>(a);
  } else {
    e = cudaFuncSetAttribute(diag_fwd_kernel<12>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) diag_fwd_kernel<12><<<grid, 128, smem, s>>>(a);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "diag forward kernel launch");
  count_launch();
  return GELIB_OK;
}

int launch_diag_bwd(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addDiagCGproduct_back";
  {
    const int st = launch_diag_bwd_fast(c, s);  // one cell per CTA, 32 channels per warp row
    if (st != -1) return st;
  }
  DiagArgs a;
  DevicePlan* plan = nullptr;
  int max_nl = 0;
  const int st = setup(c, a, &plan, &max_nl);
  if (st != GELIB_OK) return st;
  if (plan->nitems == 0 || c.cg.ncells == 0) return GELIB_OK;
  int lmax1 = 0, lmax2 = 0;
  for (const auto& p : c.x) lmax1 = std::max(lmax1, p.l);
  for (const auto& p : c.y) lmax2 = std::max(lmax2, p.l);
  a.priv_floats = 2 * a.WC * (2 * std::max(lmax1, lmax2) + 1) * a.CW;
  int nwarps = 8;
  size_t smem = 0;
  for (;; nwarps /= 2) {
    smem = ((size_t)2 * a.WC * (a.xrows + a.yrows) * a.CW + (size_t)2 * nwarps * a.priv_floats) * sizeof(float);
    if (smem <= 110 * 1024 || nwarps == 2) break;
  }
  if (smem > 220 * 1024) return -1;
  const long long groups = (c.cg.ncells + a.WC - 1) / a.WC;
  const int slices = (a.n + a.CW - 1) / a.CW;
  if (groups > 0x7fffffffLL || slices > 65535) return -1;
  const dim3 grid((unsigned)groups, (unsigned)slices);
  cudaError_t e;
  if (max_nl <= 4) {
    e = cudaFuncSetAttribute(diag_bwd_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) diag_bwd_kernel<4><<<grid, nwarps * 32, smem, s>>>(a);
  } else {
    e = cudaFuncSetAttribute(diag_bwd_kernel<12>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) diag_bwd_kernel<12><<<grid, nwarps * 32, smem, s>>>(a);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "diag backward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
