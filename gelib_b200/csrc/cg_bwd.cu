// Backward Clebsch-Gordan product: both gradients of every (l1,l2)->l triple from ONE read of g.
//
//   xg_l1[cell, m1, n1] += sum_{m2,n2} C[m1,m2] g_l[cell, m1+m2, offs + n1*N2 + n2] conj(y_l2[cell, m2, n2])
//   yg_l2[cell, m2, n2] += sum_{m1,n1} C[m1,m2] g_l[cell, m1+m2, offs + n1*N2 + n2] conj(x_l1[cell, m1, n1])
//
// Replaces SO3part_addCGproduct_back0_kernel / _back1_kernel and their launchers
// (cuda/SO3part_addCGproduct_back0.cu:32-294, cuda/SO3part_addCGproduct_back1.cu:32-175 of GElib), which
// read g twice, one of them with a channel-strided access, and the launch-per-triple loops
// Gvec::add_CGproduct_back0 / _back1 (core/Gvec.hpp:323-345).
//
// Data movement.  g is the only large stream.  A warp takes one slab of it at a time -- one row m of one
// triple, a tile of TA*WA x TBU*UB*WB channels -- straight from global memory into registers with
// 16-byte streaming loads (a lane holds TA rows x TBU units of UB adjacent complex numbers).  For every
// band entry (m1, m2 = m-m1) of that row the lane forms its partial sums over the n2 it holds (for xg)
// and over the n1 it holds (for yg) against x and y rows staged in shared memory; the partial sums are
// then combined across the lanes that share an n1 (resp. an n2) with a halving butterfly of warp
// shuffles.  Rows and units are assigned to a lane's registers in an order XOR-permuted by the lane's
// position, so every butterfly step exchanges the same register names in both partners and needs no
// selects.  Each warp accumulates into its own shared-memory copy of the gradient rows of the current
// phase (one x part and a group of y parts); after a phase the copies are summed in warp order and added
// to global memory by the CTA, which owns its cells exclusively.  The result is therefore deterministic
// and needs no atomics, except when an output is broadcast over cells (its gradient is the sum over
// cells: atomicAdd).  The band coefficients of a phase are copied to shared memory at its start, so the
// inner loop touches global memory only for g; all shared-memory addressing is 32-bit.
#include <algorithm>

#include "plan.h"

namespace gelib_b200 {

namespace {

struct BwdArgs {
  PartView x[kMaxParts], y[kMaxParts], g[kMaxParts], xg[kMaxParts], yg[kMaxParts];
  int xoff[kMaxParts], yoff[kMaxParts + 1];  // float offsets of the staged parts inside a cell block
  int xnp[kMaxParts], ynp[kMaxParts];        // padded channel counts (multiples of the tile)
  int xl[kMaxParts], yl[kMaxParts];
  int nx, ny, ng;
  int cell_floats;   // staged floats per cell
  int coef_floats;   // capacity of the shared coefficient block
  int px_floats;     // floats of one warp's private xg accumulator (all WC cells)
  int py_floats;     // same for the largest y group
  CellGrid cg;
  const float* coeffs;
  const int4* items;   // x: ri | yi<<4 | l<<8 | (m+l)<<20, y: a0 | b0<<16, z: coefficient index in the phase, w: offs
  const int4* phases;  // two per phase: {item_begin, item_end, coef_begin, coef_count}, {xi, y_first, y_count, flags}
  int nphases;
  int offs_extra;
  int do_x, do_y;
  int x_atomic, y_atomic;
};

constexpr int ilog2(int v) { return v <= 1 ? 0 : 1 + ilog2(v >> 1); }

// Bits of `pos` that steer the halving steps, mapped onto register-index bits (step s <-> bit log2(N)-1-s).
template <int N, int W>
__device__ __forceinline__ int perm_bits(int pos) {
  constexpr int NH = ilog2(N) < ilog2(W) ? ilog2(N) : ilog2(W);
  int r = 0;
#pragma unroll
  for (int s = 0; s < NH; s++) r |= ((pos >> s) & 1) << (ilog2(N) - 1 - s);
  return r;
}

// Sum N elements of E floats each over the W lanes whose lane ids differ in bits [LSH, LSH+log2 W).
// Halving steps first (the kept half is the low registers thanks to the XOR permutation of the data),
// plain all-reduce steps once a single element is left.  On return elements [0, max(1, N/W)) are final.
template <int N, int E, int W, int LSH>
__device__ __forceinline__ void butterfly(float* v) {
  int n = N;
#pragma unroll
  for (int s = 0; s < ilog2(W); s++) {
    const int mask = (1 << s) << LSH;
    if (n > 1) {
      n >>= 1;
#pragma unroll
      for (int i = 0; i < n * E; i++) v[i] += __shfl_xor_sync(0xffffffffu, v[i + n * E], mask);
    } else {
#pragma unroll
      for (int i = 0; i < E; i++) v[i] += __shfl_xor_sync(0xffffffffu, v[i], mask);
    }
  }
}

__device__ __forceinline__ void stage_parts_padded(float* dst_cell, const PartView* parts, const int* off,
                                                   const int* np, int nparts, const CellGrid& cg, long long cell,
                                                   bool cell_ok) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = parts[i];
    const float* src = cell_ok ? p.base + cell_offset(p, cg, cell) : nullptr;
    float* dst = dst_cell + off[i];
    const int n = p.n, rows = 2 * p.l + 1, npad = np[i];
    const int total = rows * npad;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int m = e / npad, ch = e - m * npad;
      float2 v = make_float2(0.f, 0.f);
      if (cell_ok && ch < n) v = __ldg(reinterpret_cast<const float2*>(src + (long long)m * p.sm + 2 * ch));
      *reinterpret_cast<float2*>(dst + 2 * e) = v;
    }
  }
}

// Adds the warps' private copies of one part's gradient rows to global memory.  `priv` is warp 0's copy of
// the part for cell 0; copies of other warps / cells are priv_stride / cell_stride floats further.
__device__ __forceinline__ void flush_part(const float* priv, int priv_stride, int cell_stride, int nwarps,
                                           const PartView& out, const long long* cell_off, int npad, int WC,
                                           long long cell0, const CellGrid& cg, bool atomic) {
  const int rows = 2 * out.l + 1, n = out.n;
  const int per_cell = rows * n;
  for (int e = threadIdx.x; e < WC * per_cell; e += blockDim.x) {
    const int c = e / per_cell, q = e - c * per_cell;
    const int row = q / n, ch = q - row * n;
    if (cell0 + c >= cg.ncells) continue;
    const float* src = priv + c * cell_stride + 2 * (row * npad + ch);
    float sr = 0.f, si = 0.f;
    for (int w = 0; w < nwarps; w++) {
      const float2 v = *reinterpret_cast<const float2*>(src + w * priv_stride);
      sr += v.x;
      si += v.y;
    }
    float* p = out.base + cell_off[c * kMaxParts] + (long long)row * out.sm + 2 * ch;
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

template <int TA, int TBU, int WA, int WB, bool VEC>
__global__ void __launch_bounds__(256, 2) cg_bwd_kernel(const __grid_constant__ BwdArgs A) {
  constexpr int UB = VEC ? 2 : 1;  // complex numbers per unit (one 16- or 8-byte load)
  constexpr int WC = 32 / (WA * WB);
  constexpr int TILE_A = TA * WA, TILE_B = TBU * UB * WB;
  static_assert(WC * WA * WB == 32, "lane layout must fill a warp");
  extern __shared__ __align__(16) float smem[];
  // [0, OFFS): offsets of the CTA's cells into the g, xg and yg parts, three tables of [WC][kMaxParts]
  constexpr int OFFS = 6 * WC * kMaxParts;
  long long* goff = reinterpret_cast<long long*>(smem);
  long long* xgoff = goff + WC * kMaxParts;
  long long* ygoff = xgoff + WC * kMaxParts;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int lb = lane % WB, la = (lane / WB) % WA, lc = lane / (WA * WB);
  const long long cell0 = (long long)blockIdx.x * WC;
  const bool cell_ok = cell0 + lc < A.cg.ncells;
  const bool do_x = A.do_x != 0, do_y = A.do_y != 0;
  fill_cell_offsets(goff, A.g, A.ng, A.cg, cell0, WC);
  if (do_x) fill_cell_offsets(xgoff, A.xg, A.nx, A.cg, cell0, WC);
  if (do_y) fill_cell_offsets(ygoff, A.yg, A.ny, A.cg, cell0, WC);

  // float indices into smem[] of the remaining regions
  const int STAGE = OFFS;
  const int COEF = STAGE + WC * A.cell_floats;
  const int PRIVX = COEF + A.coef_floats;
  const int PRIVY = PRIVX + nwarps * A.px_floats;
  for (int c = 0; c < WC; c++) {
    const bool ok = cell0 + c < A.cg.ncells;
    stage_parts_padded(smem + STAGE + c * A.cell_floats, A.x, A.xoff, A.xnp, A.nx, A.cg, cell0 + c, ok);
    stage_parts_padded(smem + STAGE + c * A.cell_floats, A.y, A.yoff, A.ynp, A.ny, A.cg, cell0 + c, ok);
  }

  const int rp = perm_bits<TA, WB>(lb);    // register row i holds channel row i ^ rp of the lane's TA rows
  const int cp = perm_bits<TBU, WA>(la);   // register unit u holds unit u ^ cp of the lane's TBU units
  constexpr int NHX = ilog2(TA) < ilog2(WB) ? ilog2(TA) : ilog2(WB);
  constexpr int NHY = ilog2(TBU) < ilog2(WA) ? ilog2(TBU) : ilog2(WA);
  constexpr int OWNX = TA >> NHX, OWNY = TBU >> NHY;
  const bool writer_x = (lb >> NHX) == 0, writer_y = (la >> NHY) == 0;
  const int mypx = PRIVX + warp * A.px_floats;
  const int mypy = PRIVY + warp * A.py_floats;
  const int blk = STAGE + lc * A.cell_floats;
  // lane-constant float offsets of the lane's rows / units inside a tile row
  int xo[TA], yo[TBU];
#pragma unroll
  for (int i = 0; i < TA; i++) xo[i] = 2 * (la * TA + (i ^ rp));
#pragma unroll
  for (int u = 0; u < TBU; u++) yo[u] = 2 * ((u ^ cp) * WB + lb) * UB;

  for (int ph = 0; ph < A.nphases; ph++) {
    const int4 d0 = __ldg(&A.phases[2 * ph]), d1 = __ldg(&A.phases[2 * ph + 1]);
    const int ib = d0.x, ie = d0.y;
    const int xi = d1.x, yfirst = d1.y, ycount = d1.z;
    const bool first_of_x = d1.w & 1, last_of_x = d1.w & 2;
    const int l1 = A.xl[xi], n1 = A.x[xi].n, n1p = A.xnp[xi];
    const int px_cell = 2 * (2 * l1 + 1) * n1p;
    const int ybase = A.yoff[yfirst];
    const int py_cell = A.yoff[yfirst + ycount] - ybase;
    // zero this warp's private rows (x only when a new l1 block starts), fetch the phase's coefficients
    if (first_of_x)
      for (int e = lane; e < WC * px_cell; e += 32) smem[mypx + e] = 0.f;
    for (int e = lane; e < WC * py_cell; e += 32) smem[mypy + e] = 0.f;
    for (int e = threadIdx.x; e < d0.w; e += blockDim.x) smem[COEF + e] = __ldg(A.coeffs + d0.z + e);
    __syncthreads();

    const int xrow0 = blk + A.xoff[xi];

    for (int it = ib + warp; it < ie; it += nwarps) {
      const int4 item = __ldg(&A.items[it]);
      const int ri = item.x & 15, yi = (item.x >> 4) & 15, l = (item.x >> 8) & 0xfff, m = (item.x >> 20) - l;
      const int a0 = item.y & 0xffff, b0 = item.y >> 16;
      const int l2 = A.yl[yi], n2 = A.y[yi].n, n2p = A.ynp[yi];

      // ---- g slab -> registers
      float g[TA][TBU][2 * UB];
      {
        const PartView& gp = A.g[ri];
        const float* grow = gp.base + goff[lc * kMaxParts + ri] + (long long)(m + l) * gp.sm +
                            2LL * (item.w + A.offs_extra) + 2 * b0;
        const bool full = cell_ok && a0 + TILE_A <= n1 && b0 + TILE_B <= n2;
#pragma unroll
        for (int i = 0; i < TA; i++) {
          const int n1i = a0 + (xo[i] >> 1);
          const float* gr = grow + 2LL * n1i * n2;
#pragma unroll
          for (int u = 0; u < TBU; u++) {
            const bool ok = full || (cell_ok && n1i < n1 && b0 + (yo[u] >> 1) < n2);
            if constexpr (VEC) {
              float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
              if (ok) v = __ldcs(reinterpret_cast<const float4*>(gr + yo[u]));
              g[i][u][0] = v.x; g[i][u][1] = v.y; g[i][u][2] = v.z; g[i][u][3] = v.w;
            } else {
              float2 v = make_float2(0.f, 0.f);
              if (ok) v = __ldcs(reinterpret_cast<const float2*>(gr + yo[u]));
              g[i][u][0] = v.x; g[i][u][1] = v.y;
            }
          }
        }
      }

      // ---- band loop: running float indices into smem[]
      const int lo = max(-l1, m - l2), hi = min(l1, m + l2);
      const int xstep = 2 * n1p, ystep = 2 * n2p;
      int xrow = xrow0 + 2 * a0 + (lo + l1) * xstep;                      // x row m1 = lo, tile column a0
      int yrow = blk + A.yoff[yi] + 2 * b0 + (m - lo + l2) * ystep;       // y row m2 = m - lo
      int pxrow = mypx + lc * px_cell + 2 * a0 + (lo + l1) * xstep;
      int pyrow = mypy + lc * py_cell + (A.yoff[yi] - ybase) + 2 * b0 + (m - lo + l2) * ystep;
      int cidx = COEF + item.z;
      for (int k = lo; k <= hi; k++) {
        const float c = smem[cidx];
        float xv[TA][2], yv[TBU][2 * UB];
#pragma unroll
        for (int i = 0; i < TA; i++) {
          const float2 v = *reinterpret_cast<const float2*>(&smem[xrow + xo[i]]);
          xv[i][0] = v.x; xv[i][1] = v.y;
        }
#pragma unroll
        for (int u = 0; u < TBU; u++) {
          if constexpr (VEC) {
            const float4 v = *reinterpret_cast<const float4*>(&smem[yrow + yo[u]]);
            yv[u][0] = v.x; yv[u][1] = v.y; yv[u][2] = v.z; yv[u][3] = v.w;
          } else {
            const float2 v = *reinterpret_cast<const float2*>(&smem[yrow + yo[u]]);
            yv[u][0] = v.x; yv[u][1] = v.y;
          }
        }

        if (do_x) {
          float tx[TA * 2];
#pragma unroll
          for (int i = 0; i < TA; i++) {
            float sr = 0.f, si = 0.f;
#pragma unroll
            for (int u = 0; u < TBU; u++)
#pragma unroll
              for (int e = 0; e < UB; e++) {
                const float gr = g[i][u][2 * e], gi = g[i][u][2 * e + 1];
                const float yr = yv[u][2 * e], yim = yv[u][2 * e + 1];
                sr = fmaf(gr, yr, sr); sr = fmaf(gi, yim, sr);
                si = fmaf(gi, yr, si); si = fmaf(-gr, yim, si);
              }
            tx[2 * i] = sr; tx[2 * i + 1] = si;
          }
          butterfly<TA, 2, WB, 0>(tx);
          if (writer_x) {
#pragma unroll
            for (int i = 0; i < OWNX; i++) {
              float2* p = reinterpret_cast<float2*>(&smem[pxrow + xo[i]]);
              float2 o = *p;
              o.x = fmaf(c, tx[2 * i], o.x);
              o.y = fmaf(c, tx[2 * i + 1], o.y);
              *p = o;
            }
          }
        }
        if (do_y) {
          float ty[TBU * 2 * UB];
#pragma unroll
          for (int u = 0; u < TBU; u++)
#pragma unroll
            for (int e = 0; e < UB; e++) {
              float sr = 0.f, si = 0.f;
#pragma unroll
              for (int i = 0; i < TA; i++) {
                const float gr = g[i][u][2 * e], gi = g[i][u][2 * e + 1];
                sr = fmaf(gr, xv[i][0], sr); sr = fmaf(gi, xv[i][1], sr);
                si = fmaf(gi, xv[i][0], si); si = fmaf(-gr, xv[i][1], si);
              }
              ty[(u * UB + e) * 2] = sr; ty[(u * UB + e) * 2 + 1] = si;
            }
          butterfly<TBU, 2 * UB, WA, ilog2(WB)>(ty);
          if (writer_y) {
#pragma unroll
            for (int u = 0; u < OWNY; u++) {
              if constexpr (VEC) {
                float4* p = reinterpret_cast<float4*>(&smem[pyrow + yo[u]]);
                float4 o = *p;
                o.x = fmaf(c, ty[4 * u], o.x); o.y = fmaf(c, ty[4 * u + 1], o.y);
                o.z = fmaf(c, ty[4 * u + 2], o.z); o.w = fmaf(c, ty[4 * u + 3], o.w);
                *p = o;
              } else {
                float2* p = reinterpret_cast<float2*>(&smem[pyrow + yo[u]]);
                float2 o = *p;
                o.x = fmaf(c, ty[2 * u], o.x); o.y = fmaf(c, ty[2 * u + 1], o.y);
                *p = o;
              }
            }
          }
        }
        cidx++;
        xrow += xstep; pxrow += xstep;
        yrow -= ystep; pyrow -= ystep;
      }
    }

    // ---- end of the phase: combine the warps' copies into global memory
    __syncthreads();
    if (do_y)
      for (int j = 0; j < ycount; j++) {
        const int yi = yfirst + j;
        flush_part(smem + PRIVY + (A.yoff[yi] - ybase), A.py_floats, py_cell, nwarps, A.yg[yi], ygoff + yi, A.ynp[yi],
                   WC, cell0, A.cg, A.y_atomic != 0);
      }
    if (do_x && last_of_x)
      flush_part(smem + PRIVX, A.px_floats, px_cell, nwarps, A.xg[xi], xgoff + xi, n1p, WC, cell0, A.cg,
                 A.x_atomic != 0);
    __syncthreads();
  }
}

struct BwdCfg {
  int TA, TBU, WA, WB;
};
constexpr BwdCfg kCfgs[] = {
    {4, 4, 8, 4},  // 32 x 32 channels (16 without vector loads), 1 cell per warp
    {2, 2, 4, 4},  //  8 x 16, 2 cells
    {1, 2, 1, 4},  //  1 x 16, 8 cells
    {2, 1, 2, 2},  //  4 x  4, 8 cells
    {4, 1, 4, 1},  // 16 x  2, 8 cells
};
constexpr int kNumCfgs = sizeof(kCfgs) / sizeof(kCfgs[0]);

template <int TA, int TBU, int WA, int WB>
cudaError_t launch_cfg(const BwdArgs& a, unsigned grid, int threads, size_t smem, bool vec, cudaStream_t s) {
  auto k = vec ? cg_bwd_kernel<TA, TBU, WA, WB, true> : cg_bwd_kernel<TA, TBU, WA, WB, false>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  k<<<grid, threads, smem, s>>>(a);
  return cudaGetLastError();
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int align4(int v) { return (v + 3) / 4 * 4; }

}  // namespace

int launch_cg_bwd(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addCGproduct_back";
  const bool vec = c.vec_ok;
  const int UB = vec ? 2 : 1;
  int n1 = 1, n2 = 1;
  for (const auto& p : c.x) n1 = std::max(n1, p.n);
  for (const auto& p : c.y) n2 = std::max(n2, p.n);
  for (const auto& p : c.x) if (p.l > 2047 || p.n > 65535) return -1;
  for (const auto& p : c.y) if (p.l > 2047 || p.n > 65535) return -1;
  for (const auto& p : c.r) if (p.l > 2047) return -1;
  int best = 0;
  double best_cost = 1e300;
  for (int i = 0; i < kNumCfgs; i++) {
    const int ta = kCfgs[i].TA * kCfgs[i].WA, tb = kCfgs[i].TBU * UB * kCfgs[i].WB;
    const double cost = (double)ceil_div(n1, ta) * ta * ceil_div(n2, tb) * tb;
    if (cost < best_cost * 0.999) {
      best_cost = cost;
      best = i;
    }
  }
  const BwdCfg cfg = kCfgs[best];
  const int WC = 32 / (cfg.WA * cfg.WB);
  const int tile_a = cfg.TA * cfg.WA, tile_b = cfg.TBU * UB * cfg.WB;

  BwdArgs a;
  int off = 0, pxmax = 0;
  std::vector<int> ysize(c.y.size());
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    if (!c.xg.empty()) a.xg[i] = c.xg[i];
    a.xl[i] = c.x[i].l;
    a.xnp[i] = ceil_div(c.x[i].n, tile_a) * tile_a;
    a.xoff[i] = off;
    const int sz = align4(2 * (2 * c.x[i].l + 1) * a.xnp[i]);  // keep every part 16-byte aligned
    off += sz;
    pxmax = std::max(pxmax, WC * sz);
  }
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    if (!c.yg.empty()) a.yg[i] = c.yg[i];
    a.yl[i] = c.y[i].l;
    a.ynp[i] = ceil_div(c.y[i].n, tile_b) * tile_b;
    a.yoff[i] = off;
    ysize[i] = align4(2 * (2 * c.y[i].l + 1) * a.ynp[i]);
    off += ysize[i];
  }
  a.yoff[c.y.size()] = off;
  for (size_t i = 0; i < c.r.size(); i++) a.g[i] = c.r[i];
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.ng = (int)c.r.size();
  a.cell_floats = off;

  // ---- phases: for each x part, consecutive y parts are grouped while their rows fit the per-warp budget
  const int y_budget = std::max(1280 / WC, *std::max_element(ysize.begin(), ysize.end()));  // floats per cell
  std::vector<std::pair<int, int>> ygroups;  // (first, count)
  for (size_t i = 0; i < c.y.size();) {
    size_t j = i;
    int sum = 0;
    while (j < c.y.size() && (j == i || sum + ysize[j] <= y_budget)) sum += ysize[j++];
    ygroups.push_back({(int)i, (int)(j - i)});
    i = j;
  }
  int pymax = 0;
  for (auto& gq : ygroups) pymax = std::max(pymax, WC * (a.yoff[gq.first + gq.second] - a.yoff[gq.first]));
  a.px_floats = pxmax;
  a.py_floats = pymax;

  std::vector<int> key = {3 /*family*/, best, vec ? 1 : 0, (int)c.x.size(), (int)c.y.size(), (int)c.r.size()};
  for (const auto& p : c.x) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.y) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.r) key.push_back(p.l);
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  DevicePlan* plan = get_plan(key, [&](DevicePlan& p) {
    build_schedule(xs, ys, rs, false, true, &p.sched);
    const auto& tr = p.sched.triples;  // ordered by (xi, yi, l); coefficients are contiguous in that order
    struct It { int4 v; int cost; };
    size_t ti = 0;
    for (size_t xi = 0; xi < xs.size(); xi++) {
      for (size_t gi = 0; gi < ygroups.size(); gi++) {
        const int yf = ygroups[gi].first, yc = ygroups[gi].second;
        std::vector<It> its;
        int coef_begin = -1, coef_end = 0;
        while (ti < tr.size() && tr[ti].xi == (int)xi && tr[ti].yi < yf + yc) {
          const Triple& t = tr[ti];
          if (coef_begin < 0) coef_begin = t.coff;
          int cpos = t.coff;
          for (int m = -t.l; m <= t.l; m++) {
            const int lo = std::max<int>(-t.l1, m - t.l2), hi = std::min<int>(t.l1, m + t.l2);
            for (int a0 = 0; a0 < xs[t.xi].n; a0 += tile_a)
              for (int b0 = 0; b0 < ys[t.yi].n; b0 += tile_b)
                its.push_back({make_int4(t.ri | (t.yi << 4) | (t.l << 8) | ((m + t.l) << 20), a0 | (b0 << 16),
                                         cpos - coef_begin, t.offs),
                               hi - lo + 3});
            cpos += hi - lo + 1;
          }
          coef_end = cpos;
          ti++;
        }
        if (its.empty()) continue;
        std::stable_sort(its.begin(), its.end(), [](const It& u, const It& v) { return u.cost > v.cost; });
        const int ib = (int)p.h_items.size();
        for (const auto& it : its) p.h_items.push_back(it.v);
        p.h_jobs.push_back(ib);
        p.h_jobs.push_back((int)p.h_items.size());
        p.h_jobs.push_back(coef_begin);
        p.h_jobs.push_back(coef_end - coef_begin);
        p.h_jobs.push_back((int)xi);
        p.h_jobs.push_back(yf);
        p.h_jobs.push_back(yc);
        p.h_jobs.push_back(0);  // flags, filled below
      }
    }
    // first / last phase of every x part
    const size_t np = p.h_jobs.size() / 8;
    for (size_t q = 0; q < np; q++) {
      const bool first = q == 0 || p.h_jobs[8 * (q - 1) + 4] != p.h_jobs[8 * q + 4];
      const bool last = q + 1 == np || p.h_jobs[8 * (q + 1) + 4] != p.h_jobs[8 * q + 4];
      p.h_jobs[8 * q + 7] = (first ? 1 : 0) | (last ? 2 : 0);
    }
    p.h_jobs.push_back(0);  // keeps njobs = size - 1 meaningful for the generic uploader
  });
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->nitems == 0 || c.cg.ncells == 0) return GELIB_OK;
  const int nphases = (int)(plan->h_jobs.size() / 8);
  int coef_max = 4;
  for (int q = 0; q < nphases; q++) coef_max = std::max(coef_max, plan->h_jobs[8 * q + 3]);
  a.coef_floats = align4(coef_max);

  int nwarps = 8;
  size_t smem = 0;
  for (;; nwarps /= 2) {
    smem = ((size_t)6 * WC * kMaxParts + (size_t)WC * off + a.coef_floats + (size_t)nwarps * (pxmax + pymax)) *
           sizeof(float);
    if (smem <= 110 * 1024 || nwarps == 2) break;
  }
  if (smem > 220 * 1024) return -1;  // caller falls back to the strided kernels

  a.cg = c.cg;
  a.coeffs = plan->coeffs;
  a.items = plan->items;
  a.phases = reinterpret_cast<const int4*>(plan->jobs);
  a.nphases = nphases;
  a.offs_extra = c.offs_extra;
  a.do_x = c.xg.empty() ? 0 : 1;
  a.do_y = c.yg.empty() ? 0 : 1;
  a.x_atomic = c.xg_bcast ? 1 : 0;
  a.y_atomic = c.yg_bcast ? 1 : 0;

  const long long groups = (c.cg.ncells + WC - 1) / WC;
  if (groups > 0x7fffffffLL) return fail(GELIB_SKIPPED, fn, "number of cells exceeds 2^31-1");
  cudaError_t e = cudaSuccess;
  const int threads = nwarps * 32;
  switch (best) {
    case 0: e = launch_cfg<4, 4, 8, 4>(a, (unsigned)groups, threads, smem, vec, s); break;
    case 1: e = launch_cfg<2, 2, 4, 4>(a, (unsigned)groups, threads, smem, vec, s); break;
    case 2: e = launch_cfg<1, 2, 1, 4>(a, (unsigned)groups, threads, smem, vec, s); break;
    case 3: e = launch_cfg<2, 1, 2, 2>(a, (unsigned)groups, threads, smem, vec, s); break;
    default: e = launch_cfg<4, 1, 4, 1>(a, (unsigned)groups, threads, smem, vec, s); break;
  }
  if (e != cudaSuccess) return check_cuda(e, fn, "backward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
