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
// selects.  The reduced sums are added, scaled by the coefficient, to gradient rows of the CTA's cells kept
// in shared memory (same layout as the staged x,y rows) with shared-memory atomics: all warps of the CTA
// work through one cost-sorted list of slabs without any barrier, and the rows go to global memory once,
// at the end, by the CTA that owns the cells (atomicAdd only when an output is broadcast over cells, whose
// gradient is the sum over cells).  The order in which warps add into a row is not fixed, so gradients are
// reproducible to rounding (about 1e-7 relative), not bitwise.  All shared-memory addressing is 32-bit.
#include <algorithm>
#include <cstdlib>
#include <string>

#include "plan.h"

namespace gelib_b200 {

namespace {

struct BwdArgs {
  PartView x[kMaxParts], y[kMaxParts], g[kMaxParts], xg[kMaxParts], yg[kMaxParts];
  int xoff[kMaxParts], yoff[kMaxParts];  // float offsets of the staged parts inside a cell block
  int xnp[kMaxParts], ynp[kMaxParts];    // padded channel counts (multiples of the tile)
  int nx, ny, ng;
  int cell_floats;   // staged floats per cell (the gradient accumulators use the same layout)
  CellGrid cg;
  const float* coeffs;
  // two int4 per item:
  //   {ri | xi<<4 | yi<<8 | full<<31, l | (m+l)<<12, a0 | b0<<16, coefficient index}
  //   {offs, l1 | l2<<12, n1p | n2p<<16, unused}
  const int4* items;
  int nitems;
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

// Adds the CTA's accumulated gradient rows of every part of one vector to global memory.
__device__ __forceinline__ void flush_parts(const float* acc_cell0, int cell_floats, const PartView* out,
                                            const long long* cell_off, const int* off, const int* np, int nparts,
                                            int WC, long long cell0, const CellGrid& cg, bool atomic) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = out[i];
    const int rows = 2 * p.l + 1, n = p.n, npad = np[i];
    const int per_cell = rows * n;
    for (int e = threadIdx.x; e < WC * per_cell; e += blockDim.x) {
      const int c = e / per_cell, q = e - c * per_cell;
      const int row = q / n, ch = q - row * n;
      if (cell0 + c >= cg.ncells) continue;
      const float2 v = *reinterpret_cast<const float2*>(acc_cell0 + c * cell_floats + off[i] + 2 * (row * npad + ch));
      float* dst = p.base + cell_off[c * kMaxParts + i] + (long long)row * p.sm + 2 * ch;
      if (atomic) {
        atomicAdd(dst, v.x);
        atomicAdd(dst + 1, v.y);
      } else {
        float2 o = *reinterpret_cast<float2*>(dst);
        o.x += v.x;
        o.y += v.y;
        *reinterpret_cast<float2*>(dst) = o;
      }
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

  // float indices into smem[]: staged x,y rows of the cells, then gradient accumulators in the same layout
  const int STAGE = OFFS;
  const int ACC = STAGE + WC * A.cell_floats;
  for (int c = 0; c < WC; c++) {
    const bool ok = cell0 + c < A.cg.ncells;
    stage_parts_padded(smem + STAGE + c * A.cell_floats, A.x, A.xoff, A.xnp, A.nx, A.cg, cell0 + c, ok);
    stage_parts_padded(smem + STAGE + c * A.cell_floats, A.y, A.yoff, A.ynp, A.ny, A.cg, cell0 + c, ok);
  }
  for (int e = threadIdx.x; e < WC * A.cell_floats; e += blockDim.x) smem[ACC + e] = 0.f;
  __syncthreads();

  const int rp = perm_bits<TA, WB>(lb);    // register row i holds channel row i ^ rp of the lane's TA rows
  const int cp = perm_bits<TBU, WA>(la);   // register unit u holds unit u ^ cp of the lane's TBU units
  constexpr int NHX = ilog2(TA) < ilog2(WB) ? ilog2(TA) : ilog2(WB);
  constexpr int NHY = ilog2(TBU) < ilog2(WA) ? ilog2(TBU) : ilog2(WA);
  constexpr int OWNX = TA >> NHX, OWNY = TBU >> NHY;
  const bool writer_x = (lb >> NHX) == 0, writer_y = (la >> NHY) == 0;
  const int blk = STAGE + lc * A.cell_floats;
  const int accd = ACC - STAGE;  // distance from a staged value to its gradient accumulator
  // lane-constant float offsets of the lane's rows / units inside a tile row
  int xo[TA], yo[TBU];
#pragma unroll
  for (int i = 0; i < TA; i++) xo[i] = 2 * (la * TA + (i ^ rp));
#pragma unroll
  for (int u = 0; u < TBU; u++) yo[u] = 2 * ((u ^ cp) * WB + lb) * UB;

  for (int it = warp; it < A.nitems; it += nwarps) {
    const int4 i0 = __ldg(&A.items[2 * it]), i1 = __ldg(&A.items[2 * it + 1]);
    const int ri = i0.x & 15, xi = (i0.x >> 4) & 15, yi = (i0.x >> 8) & 15;
    const int l = i0.y & 0xfff, m = (i0.y >> 12) - l;
    const int a0 = i0.z & 0xffff, b0 = i0.z >> 16;
    const int l1 = i1.y & 0xfff, l2 = i1.y >> 12;
    const int n1p = i1.z & 0xffff, n2p = i1.z >> 16;

    // ---- g slab -> registers
    float g[TA][TBU][2 * UB];
    {
      const PartView& gp = A.g[ri];
      const int n2 = A.y[yi].n;
      const float* grow = gp.base + goff[lc * kMaxParts + ri] + (long long)(m + l) * gp.sm +
                          2LL * (i1.x + A.offs_extra) + 2 * b0;
      if (i0.x < 0 && cell_ok) {  // full tile: no bounds checks
#pragma unroll
        for (int i = 0; i < TA; i++) {
          const float* gr = grow + 2LL * (a0 + (xo[i] >> 1)) * n2;
#pragma unroll
          for (int u = 0; u < TBU; u++) {
            if constexpr (VEC) {
              const float4 v = __ldcs(reinterpret_cast<const float4*>(gr + yo[u]));
              g[i][u][0] = v.x; g[i][u][1] = v.y; g[i][u][2] = v.z; g[i][u][3] = v.w;
            } else {
              const float2 v = __ldcs(reinterpret_cast<const float2*>(gr + yo[u]));
              g[i][u][0] = v.x; g[i][u][1] = v.y;
            }
          }
        }
      } else {
        const int n1 = A.x[xi].n;
#pragma unroll
        for (int i = 0; i < TA; i++) {
          const int n1i = a0 + (xo[i] >> 1);
          const float* gr = grow + 2LL * n1i * n2;
#pragma unroll
          for (int u = 0; u < TBU; u++) {
            const bool ok = cell_ok && n1i < n1 && b0 + (yo[u] >> 1) < n2;
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
    }

    // ---- band loop: running float indices into smem[]
    const int lo = max(-l1, m - l2), hi = min(l1, m + l2);
    const int xstep = 2 * n1p, ystep = 2 * n2p;
    int xrow = blk + A.xoff[xi] + 2 * a0 + (lo + l1) * xstep;       // x row m1 = lo, tile column a0
    int yrow = blk + A.yoff[yi] + 2 * b0 + (m - lo + l2) * ystep;   // y row m2 = m - lo
    const float* cptr = A.coeffs + i0.w;
    for (int k = lo; k <= hi; k++) {
      const float c = __ldg(cptr++);
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
            float* p = &smem[xrow + accd + xo[i]];
            atomicAdd(p, c * tx[2 * i]);
            atomicAdd(p + 1, c * tx[2 * i + 1]);
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
            float* p = &smem[yrow + accd + yo[u]];
#pragma unroll
            for (int e = 0; e < 2 * UB; e++) atomicAdd(p + e, c * ty[2 * UB * u + e]);
          }
        }
      }
      xrow += xstep;
      yrow -= ystep;
    }
  }

  // ---- every warp is done: add the accumulated rows to global memory (the CTA owns its cells)
  __syncthreads();
  if (do_x)
    flush_parts(smem + ACC, A.cell_floats, A.xg, xgoff, A.xoff, A.xnp, A.nx, WC, cell0, A.cg, A.x_atomic != 0);
  if (do_y)
    flush_parts(smem + ACC, A.cell_floats, A.yg, ygoff, A.yoff, A.ynp, A.ny, WC, cell0, A.cg, A.y_atomic != 0);
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
  // Calls whose channel counts are multiples of 32 go to the uncoupled-gradient kernel of cg_bwd_pair.cu (about
  // 0.6 of this file's kernel's instructions per band entry); everything else stays here.  Option "bwd" (initially
  // GELIB_B200_BWD): "simt" keeps everything on this file's kernel, "pair" / "tcgen05" name the kernel to try first,
  // and with a trailing "!" a call that does not qualify for it is refused instead of falling back (tests use that
  // to be sure which kernel ran).
  const int mode = bwd_mode();
  if (mode == kBwdTc || mode == kBwdTcStrict) {
    const int rc = launch_cg_bwd_tc(c, s);
    if (rc != -1) return rc;
    if (mode == kBwdTcStrict) return fail(GELIB_INVALID, fn, "the call does not qualify for the tcgen05 kernel");
  } else if (mode != kBwdSimt) {
    const int rc = launch_cg_bwd_pair(c, s, mode == kBwdAuto ? 32 : 0);
    if (rc != -1) return rc;
    if (mode == kBwdPairStrict) return fail(GELIB_INVALID, fn, "the call does not qualify for the pair kernel");
  }
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
  int off = 0;
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    if (!c.xg.empty()) a.xg[i] = c.xg[i];
    a.xnp[i] = ceil_div(c.x[i].n, tile_a) * tile_a;
    a.xoff[i] = off;
    off += align4(2 * (2 * c.x[i].l + 1) * a.xnp[i]);  // keep every part 16-byte aligned
  }
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    if (!c.yg.empty()) a.yg[i] = c.yg[i];
    a.ynp[i] = ceil_div(c.y[i].n, tile_b) * tile_b;
    a.yoff[i] = off;
    off += align4(2 * (2 * c.y[i].l + 1) * a.ynp[i]);
  }
  for (size_t i = 0; i < c.r.size(); i++) a.g[i] = c.r[i];
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.ng = (int)c.r.size();
  a.cell_floats = off;
  for (size_t i = 0; i < c.x.size(); i++) if (a.xnp[i] > 65535) return -1;
  for (size_t i = 0; i < c.y.size(); i++) if (a.ynp[i] > 65535) return -1;
  const size_t smem = ((size_t)6 * WC * kMaxParts + (size_t)2 * WC * off) * sizeof(float);
  if (smem > 220 * 1024) return -1;  // caller falls back to the strided kernels
  const int nwarps = 8;

  std::vector<int> key = {3 /*family*/, best, vec ? 1 : 0, (int)c.x.size(), (int)c.y.size(), (int)c.r.size()};
  for (const auto& p : c.x) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.y) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.r) key.push_back(p.l);
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  const int* xnp = a.xnp;
  const int* ynp = a.ynp;
  DevicePlan* plan = get_plan(key, [&](DevicePlan& p) {
    build_schedule(xs, ys, rs, false, true, &p.sched);
    struct It { int4 v0, v1; int cost; };
    std::vector<It> its;
    for (const Triple& t : p.sched.triples) {
      int cpos = t.coff;
      for (int m = -t.l; m <= t.l; m++) {
        const int lo = std::max<int>(-t.l1, m - t.l2), hi = std::min<int>(t.l1, m + t.l2);
        for (int a0 = 0; a0 < xs[t.xi].n; a0 += tile_a)
          for (int b0 = 0; b0 < ys[t.yi].n; b0 += tile_b) {
            const bool full = a0 + tile_a <= xs[t.xi].n && b0 + tile_b <= ys[t.yi].n;
            its.push_back({make_int4(t.ri | (t.xi << 4) | (t.yi << 8) | (full ? (int)0x80000000 : 0),
                                     t.l | ((m + t.l) << 12), a0 | (b0 << 16), cpos),
                           make_int4(t.offs, t.l1 | (t.l2 << 12), xnp[t.xi] | (ynp[t.yi] << 16), 0), hi - lo + 2});
          }
        cpos += hi - lo + 1;
      }
    }
    // longest first, dealt round robin to the warps: a balanced static schedule without barriers
    std::stable_sort(its.begin(), its.end(), [](const It& u, const It& v) { return u.cost > v.cost; });
    for (const auto& it : its) {
      p.h_items.push_back(it.v0);
      p.h_items.push_back(it.v1);
    }
  });
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->nitems == 0 || c.cg.ncells == 0) return GELIB_OK;

  a.cg = c.cg;
  a.coeffs = plan->coeffs;
  a.items = plan->items;
  a.nitems = plan->nitems / 2;
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
