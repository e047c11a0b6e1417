// Gradient of y in the Clebsch-Gordan product when x has ONE channel per part (the spherical harmonics of a point
// cloud) and needs no gradient itself: the backward of a first layer  CGproduct(spharms(X), v).
//
//   H[m1,m2][n2] = sum_l C_l[m1,m2] g_l[cell, m1+m2, offs_l + n2]        (every output l of the pair (l1,l2) at once)
//   yg_l2[cell, m2, n2] += H[m1,m2][n2] conj(x_l1[cell, m1])
//
// Replaces, for this shape, SO3part_addCGproduct_back1_kernel (cuda/SO3part_addCGproduct_back1.cu:32-114 of GElib) and
// the loop Gvec::add_CGproduct_back1 (core/Gvec.hpp:335-345).  The general narrow kernel (cg_narrow.cu) forms, per
// triple, the dense (2l+1) x (2l2+1) product with the zero-padded matrix A = C x; here the work per cell is the band
// only, and the band is walked once per pair instead of once per triple: at maxl 6, 7651 coefficient multiply-adds
// (packed f32x2: one instruction per complex number) + 2828 products per cell instead of about 17000 dense terms.
//
// A lane owns one (cell, n2): 32 / CW cells per warp, CW the power of two >= n2; warps are independent and small
// (about 4 KB of shared memory, 64 registers), so 32 of them share an SM and cover the latency of the loads.  A warp
// walks the list of groups -- (pair, row m, up to four output l), pairs ordered by l2 -- with the next group's record
// and its values of g (one 8-byte load per l, 8 x CW contiguous bytes per cell) fetched while the current group is
// worked on.  Per band entry it forms H from the registers (coefficients: one 16-byte load through the read-only
// cache, the same address in every lane, requested an entry ahead) and adds H conj(x[m1]) to the lane's own slot of
// row m2 in a shared-memory block of the warp (plain load / add / store: nobody else touches the slot).  The block
// holds the rows of one l2; when the pairs of that l2 are done the lane adds its column to yg in global memory.
// No shuffles, no barriers after the start, no atomics unless yg is broadcast over cells.
#include <algorithm>
#include <map>

#include "plan.h"
#include "spharm_point.h"

namespace gelib_b200 {

namespace {

constexpr int kGroupL = 4;  // output l per group
constexpr int kRec = 3;     // int4 per group record

struct Narrow1Args {
  PartView x[kMaxParts], g[kMaxParts], yg[kMaxParts];
  int xrow0[kMaxParts];  // first row of each x part in the cell's staged rows
  int nx, ng, xrows, yrows_max;
  int n2, CW, WC;
  CellGrid cg;
  // three int4 per group:
  //   {nl | band length<<8 | last group of its l2<<16 | yi<<20, x row of the first band entry (m1 = lo),
  //    y row of the first entry inside the l2 block (m2 = m - lo, descending), index of the first coefficient quad}
  //   4 x {ri, float offset of the row inside the cell's part (rows are dense: row * 2 n_r + 2 offs)}
  const int4* recs;
  int ngroups;
  const float4* coef;  // per band entry four coefficients, zero beyond the group's l
  int offs_extra;
  int y_atomic;
  int warp_bytes;      // shared memory per warp
  // fused first layer: x is not read but generated, part l = the spherical harmonics Y_l of the cell's point
  const float* sph;
  long long sph_sb, sph_sm;
  int sph_lmax;
};

typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

struct GroupRegs {
  int4 h;
  f32x2 g[kGroupL];
  float4 cq;  // lane k: the coefficient quad of band entry k
};

__device__ __forceinline__ void fetch_group(const Narrow1Args& A, int gi, const long long* gbase, int goff, bool ok, GroupRegs& R) {
  const int4* rec = A.recs + kRec * gi;
  R.h = __ldg(rec);
  const int nl = R.h.x & 255;
  const int lane = threadIdx.x & 31;
  R.cq = __ldg(A.coef + R.h.w + min(lane, ((R.h.x >> 8) & 255) - 1));
#pragma unroll
  for (int q = 0; q < kGroupL / 2; q++) {
    R.g[2 * q] = R.g[2 * q + 1] = 0ull;
    if (2 * q < nl) {  // uniform over the warp: groups of one or two l touch one record word
      const int4 w = __ldg(rec + 1 + q);  // two l per int4
      if (ok) R.g[2 * q] = __ldcs(reinterpret_cast<const f32x2*>(reinterpret_cast<const float*>(gbase[w.x]) + w.y + goff));
      if (ok && 2 * q + 1 < nl)
        R.g[2 * q + 1] = __ldcs(reinterpret_cast<const f32x2*>(reinterpret_cast<const float*>(gbase[w.z]) + w.w + goff));
    }
  }
}

// One band entry: H from the registers, H conj(x[m1]) into the lane's slot of row m2.
template <int NL>
__device__ __forceinline__ void band_entry(const float4 c, const GroupRegs& G, const float2 xv, float2* slot) {
  f32x2 h = mul2(pack2(c.x, c.x), G.g[0]);
  if (NL > 1) h = fma2(pack2(c.y, c.y), G.g[1], h);
  if (NL > 2) h = fma2(pack2(c.z, c.z), G.g[2], h);
  if (NL > 3) h = fma2(pack2(c.w, c.w), G.g[3], h);
  float hr, hi;
  unpack2(h, hr, hi);
  float2 a = *slot;
  a.x = fmaf(hr, xv.x, a.x); a.x = fmaf(hi, xv.y, a.x);
  a.y = fmaf(hi, xv.x, a.y); a.y = fmaf(-hr, xv.y, a.y);
  *slot = a;
}

// The band of one group, two entries per turn: the coefficients of an entry are requested while the entry before
// it is worked on (two register sets, used alternately).  Rows m2 = m - m1 descend as m1 ascends.
template <int NL>
__device__ __forceinline__ void run_band(const float4* cf, int cnt, const GroupRegs& G, const float2* xp, float2* ya) {
  float4 c0 = cf[0], c1;
  int k = 0;
  for (; k + 2 < cnt; k += 2) {
    c1 = cf[k + 1];
    band_entry<NL>(c0, G, xp[k], ya - 32 * k);
    c0 = cf[k + 2];
    band_entry<NL>(c1, G, xp[k + 1], ya - 32 * (k + 1));
  }
  if (k + 1 < cnt) {
    c1 = cf[k + 1];
    band_entry<NL>(c0, G, xp[k], ya - 32 * k);
    band_entry<NL>(c1, G, xp[k + 1], ya - 32 * (k + 1));
  } else {
    band_entry<NL>(c0, G, xp[k], ya - 32 * k);
  }
}

__device__ __forceinline__ void run_group(float4* cf, const GroupRegs& G, const float2* xs, float2* yacc) {
  const int cnt = (G.h.x >> 8) & 255;
  __syncwarp();                       // the band of the group before has been read
  cf[threadIdx.x & 31] = G.cq;        // the group's coefficients: one quad per lane, read back by every lane
  __syncwarp();
  const float2* xp = xs + G.h.y;
  float2* ya = yacc + 32 * G.h.z;
  switch (G.h.x & 255) {
    case 1: run_band<1>(cf, cnt, G, xp, ya); break;
    case 2: run_band<2>(cf, cnt, G, xp, ya); break;
    case 3: run_band<3>(cf, cnt, G, xp, ya); break;
    default: run_band<4>(cf, cnt, G, xp, ya); break;
  }
}

template <bool kSph>  // x generated from the cell's point (fused first layer) instead of read
__global__ void __launch_bounds__(256, 4) cg_narrow1_bwd_kernel(const __grid_constant__ Narrow1Args A) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int CW = A.CW, WC = A.WC;
  const int lc = lane / CW, n2l = lane % CW;
  const long long cell = ((long long)blockIdx.x * nwarps + warp) * WC + lc;
  const bool cell_ok = cell < A.cg.ncells;
  const bool ok = cell_ok && n2l < A.n2;
  // per warp: [g part bases: WC x kMaxParts pointers][x rows of the WC cells][yacc: the rows of one l2 x 32 lanes]
  unsigned char* wb = smem_raw + (size_t)warp * A.warp_bytes;
  long long* gbase = reinterpret_cast<long long*>(wb) + lc * kMaxParts;
  float2* xs = reinterpret_cast<float2*>(wb + 512 + 8 * WC * kMaxParts) + lc * A.xrows;
  float4* cbuf = reinterpret_cast<float4*>(wb + 8 * WC * kMaxParts);  // 32 coefficient quads of the group at work
  float2* yacc = reinterpret_cast<float2*>(wb + 512 + 8 * WC * kMaxParts + 8 * WC * A.xrows) + lane;

  for (int p = n2l; p < A.ng; p += CW)
    gbase[p] = reinterpret_cast<long long>(A.g[p].base + (cell_ok ? cell_offset(A.g[p], A.cg, cell) : 0));
  if (kSph) {
    if (n2l == 0) {
      const float* pt = A.sph + (cell_ok ? cell * A.sph_sb : 0);
      spharm_point(cell_ok ? pt[0] : 0.f, cell_ok ? pt[A.sph_sm] : 0.f, cell_ok ? pt[2 * A.sph_sm] : 1.f, A.sph_lmax,
                   reinterpret_cast<float*>(xs), A.xrow0, 1);
    }
  } else {
    for (int i = 0; i < A.nx; i++) {
      const PartView& xp = A.x[i];
      const float* xb = xp.base + (cell_ok ? cell_offset(xp, A.cg, cell) : 0);
      for (int m = n2l; m <= 2 * xp.l; m += CW)
        xs[A.xrow0[i] + m] = cell_ok ? __ldg(reinterpret_cast<const float2*>(xb + (long long)m * xp.sm)) : make_float2(0.f, 0.f);
    }
  }
  for (int r = 0; r < A.yrows_max; r++) yacc[32 * r] = make_float2(0.f, 0.f);
  __syncwarp();

  // The lane's column of the finished l2 goes to global memory and the block is cleared for the next l2.
  auto flush = [&](int yi) {
    const PartView& yp = A.yg[yi];
    float* yb = ok ? yp.base + cell_offset(yp, A.cg, cell) + 2 * n2l : nullptr;
    for (int m = 0; m <= 2 * yp.l; m++) {
      const float2 v = yacc[32 * m];
      yacc[32 * m] = make_float2(0.f, 0.f);
      if (ok) {
        float* q = yb + (long long)m * yp.sm;
        if (A.y_atomic) {
          atomicAdd(q, v.x);
          atomicAdd(q + 1, v.y);
        } else {
          float2 o = *reinterpret_cast<float2*>(q);
          o.x += v.x;
          o.y += v.y;
          *reinterpret_cast<float2*>(q) = o;
        }
      }
    }
  };

  // two groups in flight: the record and the g values of one are fetched while the other is worked on
  const int goff = 2 * (A.offs_extra + n2l);
  GroupRegs ga, gb;
  if (A.ngroups > 0) fetch_group(A, 0, gbase, goff, ok, ga);
  for (int gi = 0; gi < A.ngroups; gi += 2) {
    if (gi + 1 < A.ngroups) fetch_group(A, gi + 1, gbase, goff, ok, gb);
    run_group(cbuf, ga, xs, yacc);
    if (ga.h.x & 0x10000) flush((ga.h.x >> 20) & 0xff);
    if (gi + 1 < A.ngroups) {
      if (gi + 2 < A.ngroups) fetch_group(A, gi + 2, gbase, goff, ok, ga);
      run_group(cbuf, gb, xs, yacc);
      if (gb.h.x & 0x10000) flush((gb.h.x >> 20) & 0xff);
    }
  }
}

}  // namespace

// Returns -1 when the call does not qualify (the caller then takes the kernel of cg_narrow.cu).
int launch_cg_narrow1_bwd(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addCGproduct_back";
  if (c.x.empty() || c.y.empty() || c.r.empty() || !c.dense_channels) return -1;
  if (!c.xg.empty() || c.yg.empty()) return -1;  // the gradient of y only
  const int n2 = c.y[0].n;
  if (n2 < 1 || n2 > 32) return -1;
  for (const auto& p : c.x) if (p.n != 1 || p.l > 100) return -1;
  for (const auto& p : c.y) if (p.n != n2 || p.l > 100) return -1;
  for (const auto& p : c.x)
    for (const auto& q : c.y)
      if (2 * std::min(p.l, q.l) + 1 > 32) return -1;  // a band is at most 32 entries: one coefficient quad per lane
  for (const auto& p : c.r) if (p.l > 200 || p.sm != 2LL * p.n) return -1;  // the records bake the row pitch in
  for (const auto& p : c.r) {
    if (reinterpret_cast<uintptr_t>(p.base) % 8 || (2LL * p.n) % 2) return -1;
    if ((long long)(2 * p.l + 1) * 2 * p.n + 2LL * p.n >= 0x7fffffffLL) return -1;  // row offsets are 32-bit
  }
  if (c.sph && ((int)c.x.size() != c.sph_lmax + 1 || c.sph_lmax > kSphPointMaxL)) return -1;
  if (c.sph)
    for (size_t i = 0; i < c.x.size(); i++) if (c.x[i].l != (int)i) return -1;
  Narrow1Args a;
  int row = 0;
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    a.xrow0[i] = row;
    row += 2 * c.x[i].l + 1;
  }
  a.xrows = row;
  a.yrows_max = 0;
  for (size_t i = 0; i < c.y.size(); i++) {
    a.yg[i] = c.yg[i];
    a.yrows_max = std::max(a.yrows_max, 2 * c.y[i].l + 1);
  }
  for (size_t i = 0; i < c.r.size(); i++) a.g[i] = c.r[i];
  a.nx = (int)c.x.size();
  a.ng = (int)c.r.size();
  a.n2 = n2;
  int CW = 1;
  while (CW < n2) CW *= 2;
  a.CW = CW;
  a.WC = 32 / CW;
  a.y_atomic = c.yg_bcast ? 1 : 0;
  a.sph = c.sph;
  a.sph_sb = c.sph_sb;
  a.sph_sm = c.sph_sm;
  a.sph_lmax = c.sph_lmax;
  size_t wbytes = (size_t)8 * a.WC * kMaxParts + 512 + (size_t)8 * a.WC * a.xrows + (size_t)256 * a.yrows_max;
  wbytes = (wbytes + 15) / 16 * 16;
  a.warp_bytes = (int)wbytes;
  const int nwarps = 8;
  const size_t smem = (size_t)nwarps * wbytes;
  if (smem > 200 * 1024) return -1;

  std::vector<int> key = {12 /*family*/, (int)c.x.size(), (int)c.y.size(), (int)c.r.size()};
  for (const auto& p : c.x) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.y) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.r) { key.push_back(p.l); key.push_back(p.n); }
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  const int* xrow0 = a.xrow0;
  DevicePlan* plan = get_plan(key, [&](DevicePlan& p) {
    build_schedule(xs, ys, rs, false, false, &p.sched);
    // pairs ordered by yi: the warp's block holds the rows of one l2 at a time
    std::map<std::pair<int, int>, std::vector<const Triple*>> pairs;
    for (const Triple& t : p.sched.triples) pairs[{t.yi, t.xi}].push_back(&t);
    std::vector<float>& coef = p.h_floats;
    int last_yi = -1;
    for (const auto& kv : pairs) {
      const auto& ts = kv.second;
      const int yi = kv.first.first, xi = kv.first.second;
      if (last_yi >= 0 && yi != last_yi) p.h_items[p.h_items.size() - kRec].x |= 0x10000;
      last_yi = yi;
      const int l1 = xs[xi].l, l2 = ys[yi].l;
      int lm = 0;
      for (const Triple* t : ts) lm = std::max<int>(lm, t->l);
      for (int m = -lm; m <= lm; m++) {
        const int lo = std::max(-l1, m - l2), hi = std::min(l1, m + l2);
        std::vector<const Triple*> act;
        for (const Triple* t : ts)
          if (t->l >= std::abs(m)) act.push_back(t);
        for (size_t c0 = 0; c0 < act.size(); c0 += kGroupL) {
          const int nl = (int)std::min<size_t>(kGroupL, act.size() - c0);
          int w[2 * kGroupL] = {0};
          for (int k = 0; k < nl; k++) {
            const Triple* t = act[c0 + k];
            w[2 * k] = t->ri;
            w[2 * k + 1] = (m + t->l) * 2 * rs[t->ri].n + 2 * t->offs;
          }
          p.h_items.push_back(make_int4(nl | ((hi - lo + 1) << 8) | (yi << 20), xrow0[xi] + lo + l1, m - lo + l2,
                                        (int)(coef.size() / 4)));
          p.h_items.push_back(make_int4(w[0], w[1], w[2], w[3]));
          p.h_items.push_back(make_int4(w[4], w[5], w[6], w[7]));
          for (int m1 = lo; m1 <= hi; m1++)
            for (int k = 0; k < kGroupL; k++)
              coef.push_back(k < nl ? (float)cg_coefficient(l1, l2, act[c0 + k]->l, m1, m - m1) : 0.f);
        }
      }
    }
    if (!p.h_items.empty()) p.h_items[p.h_items.size() - kRec].x |= 0x10000;
  });
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->nitems == 0 || c.cg.ncells == 0) return GELIB_OK;
  a.cg = c.cg;
  a.recs = plan->items;
  a.ngroups = plan->nitems / kRec;
  a.coef = reinterpret_cast<const float4*>(plan->floats);
  a.offs_extra = c.offs_extra;
  const long long blocks = (c.cg.ncells + (long long)a.WC * nwarps - 1) / ((long long)a.WC * nwarps);
  if (blocks > 0x7fffffffLL) return -1;
  cudaError_t e;
  if (a.sph) {
    e = cudaFuncSetAttribute(cg_narrow1_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) cg_narrow1_bwd_kernel<true><<<(unsigned)blocks, nwarps * 32, smem, s>>>(a);
  } else {
    e = cudaFuncSetAttribute(cg_narrow1_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) cg_narrow1_bwd_kernel<false><<<(unsigned)blocks, nwarps * 32, smem, s>>>(a);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "single-channel backward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
