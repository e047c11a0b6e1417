// Clebsch-Gordan product of a narrow x (a few channels, e.g. spherical harmonics with one channel per l) with a
// y of up to 32 channels: forward and both gradients.
//
// The tiled kernels (cg_fwd.cu, cg_bwd.cu) get their operand reuse from an n1 x n2 channel tile; with one or two
// x channels there is no tile, and every multiply-add would need its own shared-memory operand.  Here the reuse
// comes from y instead.  A lane owns one (cell, n2); for the current y part it keeps the whole column
// y[-l2..l2][n2] in registers (the kernel body is instantiated per l2, loops over m2 fully unrolled).  For each
// (x part, x channel, output l) the lanes of a cell build, in shared memory, the small matrix
//     A[m][m2] = C[m-m2, m2] x[m-m2]      (zero outside the band)
// and the output row m is the dense product sum_m2 A[m][m2] y[m2][n2]: one broadcast shared-memory load per two
// multiply-adds, 128 contiguous bytes stored per cell and row.  Warps are independent (each owns its cells), so
// there are no block barriers and no atomics.
// Backward: yg[m2][n2] += sum_m conj(A[m][m2]) g[m][n2] accumulates in registers next to the y column;
// xg[m1] += C[m1,m2] sum_n2 g[m][n2] conj(y[m2][n2]) needs a sum over the lanes of the cell, done once per row m
// for all m2 together with a halving butterfly (the lanes' y columns are loaded in an XOR-permuted slot order so
// that no step needs a select), after which lane j holds the sum for one m2 and adds it to the x gradient of the
// cell in shared memory.
// Arithmetic: SO3part::add_CGproduct_kernel / _back0_kernel / _back1_kernel (SO3/SO3part.hpp:205-257 of GElib),
// triple walk of Gvec::add_CGproduct* (core/Gvec.hpp:311-345).
#include <algorithm>

#include "plan.h"
#include "spharm_point.h"

namespace gelib_b200 {

namespace {

constexpr int kMaxL2 = 8;  // y parts up to l = 8 have an unrolled body

struct NarrowArgs {
  PartView x[kMaxParts], y[kMaxParts], r[kMaxParts], xg[kMaxParts], yg[kMaxParts];
  int xrow0[kMaxParts];   // first staged row of each x part (rows of n1max complex numbers)
  int xl[kMaxParts], yl[kMaxParts];
  int nx, ny, nr;
  int n1max, n2, CW, WC;  // CW lanes per cell (power of two >= n2), WC = 32 / CW cells per warp
  int xrows;              // staged x rows per cell
  int xcell_floats;       // floats of one cell's staged x rows (multiple of 4)
  int cx_floats;          // floats of one cell's A matrix buffer
  int warp_floats;        // shared-memory floats per warp
  CellGrid cg;
  const Triple* triples;  // coff = offset of the dense (2l1+1) x (2l2+1) coefficient matrix
  const float* coeffs;
  const int2* pairs;      // [yi * nx + xi] = {first triple, number of triples}
  int offs_extra;
  int accumulate;
  int do_x, do_y, x_atomic, y_atomic;
  // fused first layer: x is not read but generated, part l = the spherical harmonics Y_l of the cell's point
  const float* sph;           // points (cell, 3) or nullptr
  long long sph_sb, sph_sm;   // strides between cells / between coordinates, in floats
  int sph_lmax;
};

__device__ __forceinline__ float2 cmul(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }

// Builds A[m][j] = C[m1][j] x[m1], m1 = m - (j - l2), for the lanes' cell; rows padded to LYP entries.
template <int LY>
__device__ __forceinline__ void build_A(float* cx, const float* xs, const float* __restrict__ Cm, int l, int l1, int l2,
                                        int n1max, int n1i, int lic, int CW) {
  constexpr int LYP = LY + 1;
  const int total = (2 * l + 1) * LYP;
  for (int e = lic; e < total; e += CW) {
    const int mi = e / LYP, j = e - mi * LYP;
    const int m1 = (mi - l) - (j - l2);
    float2 v = make_float2(0.f, 0.f);
    if (j < LY && m1 >= -l1 && m1 <= l1) {
      const float c = __ldg(Cm + (m1 + l1) * LY + j);
      const float2 xv = *reinterpret_cast<const float2*>(xs + 2 * ((m1 + l1) * n1max + n1i));
      v = make_float2(c * xv.x, c * xv.y);
    }
    *reinterpret_cast<float2*>(cx + 2 * e) = v;
  }
}

template <int LY>
__device__ __forceinline__ void fwd_l2(const NarrowArgs& A, const float* xs_cell, float* cx, const long long* roff, int yi,
                                       long long cell, int n2l, int lic, bool ok) {
  constexpr int LYP = LY + 1;
  const int l2 = (LY - 1) / 2;
  float2 yreg[LYP];
  {
    const PartView& yp = A.y[yi];
    const float* yb = yp.base + (ok ? cell_offset(yp, A.cg, cell) : 0) + 2 * n2l;
#pragma unroll
    for (int j = 0; j < LY; j++)
      yreg[j] = ok ? __ldg(reinterpret_cast<const float2*>(yb + (long long)j * yp.sm)) : make_float2(0.f, 0.f);
    yreg[LY] = make_float2(0.f, 0.f);
  }
  const bool acc_mode = A.accumulate != 0;
  for (int xi = 0; xi < A.nx; xi++) {
    const int l1 = A.xl[xi], n1 = A.x[xi].n;
    const int2 pr = __ldg(&A.pairs[yi * A.nx + xi]);
    const float* xs = xs_cell + 2 * A.xrow0[xi] * A.n1max;
    for (int t = pr.x; t < pr.x + pr.y; t++) {
      const Triple tr = A.triples[t];
      const int l = tr.l;
      const PartView& rp = A.r[tr.ri];
      for (int n1i = 0; n1i < n1; n1i++) {
        __syncwarp();
        build_A<LY>(cx, xs, A.coeffs + tr.coff, l, l1, l2, A.n1max, n1i, lic, A.CW);
        __syncwarp();
        float* rb = rp.base + roff[tr.ri] + 2LL * (tr.offs + A.offs_extra + n1i * A.n2 + n2l);
        for (int mi = 0; mi <= 2 * l; mi++) {
          float ar = 0.f, ai = 0.f;
          const float* row = cx + 2 * mi * LYP;
#pragma unroll
          for (int j = 0; j < LYP; j += 2) {
            const float4 a = *reinterpret_cast<const float4*>(row + 2 * j);
            ar = fmaf(a.x, yreg[j].x, ar); ar = fmaf(-a.y, yreg[j].y, ar);
            ai = fmaf(a.x, yreg[j].y, ai); ai = fmaf(a.y, yreg[j].x, ai);
            ar = fmaf(a.z, yreg[j + 1].x, ar); ar = fmaf(-a.w, yreg[j + 1].y, ar);
            ai = fmaf(a.z, yreg[j + 1].y, ai); ai = fmaf(a.w, yreg[j + 1].x, ai);
          }
          if (ok) {
            float2* p = reinterpret_cast<float2*>(rb + (long long)mi * rp.sm);
            float2 v = make_float2(ar, ai);
            if (acc_mode) {
              const float2 o = *p;
              v.x += o.x;
              v.y += o.y;
              *p = v;
            } else {
              __stcs(p, v);
            }
          }
        }
      }
    }
  }
}

__global__ void __launch_bounds__(256) cg_narrow_fwd_kernel(const __grid_constant__ NarrowArgs A) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int CW = A.CW, WC = A.WC;
  const int lc = lane / CW, lic = lane % CW;
  const long long cell = ((long long)blockIdx.x * nwarps + warp) * WC + lc;
  const bool cell_ok = cell < A.cg.ncells;
  const bool ok = cell_ok && lic < A.n2;
  // per warp: [output offsets: WC x kMaxParts long long][x rows of the WC cells][A matrices of the WC cells]
  float* wbase = smem + (size_t)warp * A.warp_floats;
  long long* roff = reinterpret_cast<long long*>(wbase) + lc * kMaxParts;
  float* xs_cell = wbase + 2 * WC * kMaxParts + (size_t)lc * A.xcell_floats;
  float* cx = wbase + 2 * WC * kMaxParts + (size_t)WC * A.xcell_floats + (size_t)lc * A.cx_floats;
  for (int p = lic; p < A.nr; p += CW) roff[p] = cell_ok ? cell_offset(A.r[p], A.cg, cell) : 0;
  if (A.sph) {  // one lane per cell generates the harmonics of the cell's point straight into the staged rows
    if (lic == 0) {
      const float* pt = A.sph + (cell_ok ? cell * A.sph_sb : 0);
      spharm_point(cell_ok ? pt[0] : 0.f, cell_ok ? pt[A.sph_sm] : 0.f, cell_ok ? pt[2 * A.sph_sm] : 1.f, A.sph_lmax, xs_cell,
                   A.xrow0, A.n1max);
    }
  } else {
    for (int i = 0; i < A.nx; i++) {
      const PartView& xp = A.x[i];
      const float* xb = xp.base + (cell_ok ? cell_offset(xp, A.cg, cell) : 0);
      const int total = (2 * xp.l + 1) * xp.n;
      for (int e = lic; e < total; e += CW) {
        const int m = e / xp.n, ch = e - m * xp.n;
        const float2 v = cell_ok ? __ldg(reinterpret_cast<const float2*>(xb + (long long)m * xp.sm + 2 * ch)) : make_float2(0.f, 0.f);
        *reinterpret_cast<float2*>(xs_cell + 2 * ((A.xrow0[i] + m) * A.n1max + ch)) = v;
      }
    }
  }
  __syncwarp();
  for (int yi = 0; yi < A.ny; yi++) {
    switch (A.yl[yi]) {
      case 0: fwd_l2<1>(A, xs_cell, cx, roff, yi, cell, lic, lic, ok); break;
      case 1: fwd_l2<3>(A, xs_cell, cx, roff, yi, cell, lic, lic, ok); break;
      case 2: fwd_l2<5>(A, xs_cell, cx, roff, yi, cell, lic, lic, ok); break;
      case 3: fwd_l2<7>(A, xs_cell, cx, roff, yi, cell, lic, lic, ok); break;
      case 4: fwd_l2<9>(A, xs_cell, cx, roff, yi, cell, lic, lic, ok); break;
      case 5: fwd_l2<11>(A, xs_cell, cx, roff, yi, cell, lic, lic, ok); break;
      case 6: fwd_l2<13>(A, xs_cell, cx, roff, yi, cell, lic, lic, ok); break;
      case 7: fwd_l2<15>(A, xs_cell, cx, roff, yi, cell, lic, lic, ok); break;
      default: fwd_l2<17>(A, xs_cell, cx, roff, yi, cell, lic, lic, ok); break;
    }
  }
}


// ---- backward --------------------------------------------------------------------------------------------------

constexpr int ilog2n(int v) { return v <= 1 ? 0 : 1 + ilog2n(v >> 1); }
constexpr int pow2ceil(int v) { return v <= 1 ? 1 : 2 * pow2ceil((v + 1) / 2); }

// Butterfly over the lanes of a cell (lane bits [0, log2 CW)), CW >= NS: log2(NS) halving steps (the slot order
// of the data is XOR-permuted per lane, so the kept half is always the low slots), then plain all-reduce steps
// of slot 0 over the remaining lane bits.
template <int NS>
__device__ __forceinline__ void cell_butterfly(float (&v)[2 * NS], int CW) {
  int n = NS;
#pragma unroll
  for (int s = 0; s < ilog2n(NS); s++) {
    n >>= 1;
#pragma unroll
    for (int i = 0; i < 2 * n; i++) v[i] += __shfl_xor_sync(0xffffffffu, v[i + 2 * n], 1 << s);
  }
#pragma unroll
  for (int s = ilog2n(NS); s < 5; s++) {
    if ((1 << s) < CW) {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1 << s);
      v[1] += __shfl_xor_sync(0xffffffffu, v[1], 1 << s);
    }
  }
}

template <int LY>
__device__ __forceinline__ void bwd_l2(const NarrowArgs& A, const float* xs_cell, float* xg_cell, float* cx,
                                       const long long* goff, int yi, long long cell, int n2l, int lic, bool ok) {
  constexpr int NS = pow2ceil(LY);  // slots per lane
  const int l2 = (LY - 1) / 2;
  const int CW = A.CW;
  // slot s holds m2 index j = s ^ p; the halving steps use lane bits 0.. and slot bits from the top
  int p = 0;
#pragma unroll
  for (int s = 0; s < ilog2n(NS); s++) p |= ((lic >> s) & 1) << (ilog2n(NS) - 1 - s);
  const bool writer = (lic >> ilog2n(NS)) == 0;  // lanes beyond NS hold copies after the all-reduce steps
  constexpr int LYP = LY + 1;
  float2 yreg[NS], ygacc[LYP];  // y column in permuted slot order (for the butterfly); yg column in natural order
  const PartView& yp = A.y[yi];
  {
    const float* yb = yp.base + (ok ? cell_offset(yp, A.cg, cell) : 0) + 2 * n2l;
#pragma unroll
    for (int sl = 0; sl < NS; sl++) {
      const int j = sl ^ p;
      yreg[sl] = (ok && j < LY) ? __ldg(reinterpret_cast<const float2*>(yb + (long long)j * yp.sm)) : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < LYP; j++) ygacc[j] = make_float2(0.f, 0.f);
  }
  const int jown = p;  // after the butterfly slot 0 of this lane is the sum for m2 index p
  for (int xi = 0; xi < A.nx; xi++) {
    const int l1 = A.xl[xi], n1 = A.x[xi].n;
    const int2 pr = __ldg(&A.pairs[yi * A.nx + xi]);
    const float* xs = xs_cell + 2 * A.xrow0[xi] * A.n1max;
    float* xgs = xg_cell + 2 * A.xrow0[xi] * A.n1max;
    for (int t = pr.x; t < pr.x + pr.y; t++) {
      const Triple tr = A.triples[t];
      const int l = tr.l;
      const PartView& gp = A.r[tr.ri];
      const float* Cm = A.coeffs + tr.coff;
      for (int n1i = 0; n1i < n1; n1i++) {
        __syncwarp();
        if (A.do_y) build_A<LY>(cx, xs, Cm, l, l1, l2, A.n1max, n1i, lic, CW);
        __syncwarp();
        const float* gb = gp.base + goff[tr.ri] + 2LL * (tr.offs + A.offs_extra + n1i * A.n2 + n2l);
        float2 gnext = ok ? __ldcs(reinterpret_cast<const float2*>(gb)) : make_float2(0.f, 0.f);
        for (int mi = 0; mi <= 2 * l; mi++) {
          const float2 g = gnext;
          if (mi < 2 * l && ok) gnext = __ldcs(reinterpret_cast<const float2*>(gb + (long long)(mi + 1) * gp.sm));
          if (A.do_y) {
            const float* row = cx + 2 * mi * LYP;
#pragma unroll
            for (int j = 0; j < LYP; j += 2) {  // g conj(A), two entries per broadcast load
              const float4 a = *reinterpret_cast<const float4*>(row + 2 * j);
              ygacc[j].x = fmaf(g.x, a.x, ygacc[j].x); ygacc[j].x = fmaf(g.y, a.y, ygacc[j].x);
              ygacc[j].y = fmaf(g.y, a.x, ygacc[j].y); ygacc[j].y = fmaf(-g.x, a.y, ygacc[j].y);
              ygacc[j + 1].x = fmaf(g.x, a.z, ygacc[j + 1].x); ygacc[j + 1].x = fmaf(g.y, a.w, ygacc[j + 1].x);
              ygacc[j + 1].y = fmaf(g.y, a.z, ygacc[j + 1].y); ygacc[j + 1].y = fmaf(-g.x, a.w, ygacc[j + 1].y);
            }
          }
          if (A.do_x) {
            float tv[2 * NS];
#pragma unroll
            for (int sl = 0; sl < NS; sl++) {  // g conj(y)
              tv[2 * sl] = fmaf(g.x, yreg[sl].x, g.y * yreg[sl].y);
              tv[2 * sl + 1] = fmaf(g.y, yreg[sl].x, -g.x * yreg[sl].y);
            }
            cell_butterfly<NS>(tv, CW);
            const int m1 = (mi - l) - (jown - l2);
            if (writer && jown < LY && m1 >= -l1 && m1 <= l1) {
              const float c = __ldg(Cm + (m1 + l1) * LY + jown);
              float2* q = reinterpret_cast<float2*>(xgs + 2 * ((m1 + l1) * A.n1max + n1i));
              float2 o = *q;
              o.x = fmaf(c, tv[0], o.x);
              o.y = fmaf(c, tv[1], o.y);
              *q = o;
            }
          }
        }
      }
    }
  }
  if (A.do_y && ok) {
    const PartView& ygp = A.yg[yi];
    float* yb = ygp.base + cell_offset(ygp, A.cg, cell) + 2 * n2l;
#pragma unroll
    for (int j = 0; j < LY; j++) {
      float* q = yb + (long long)j * ygp.sm;
      if (A.y_atomic) {
        atomicAdd(q, ygacc[j].x);
        atomicAdd(q + 1, ygacc[j].y);
      } else {
        float2 o = *reinterpret_cast<float2*>(q);
        o.x += ygacc[j].x;
        o.y += ygacc[j].y;
        *reinterpret_cast<float2*>(q) = o;
      }
    }
  }
}

__global__ void __launch_bounds__(256) cg_narrow_bwd_kernel(const __grid_constant__ NarrowArgs A) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int CW = A.CW, WC = A.WC;
  const int lc = lane / CW, lic = lane % CW;
  const long long cell = ((long long)blockIdx.x * nwarps + warp) * WC + lc;
  const bool cell_ok = cell < A.cg.ncells;
  const bool ok = cell_ok && lic < A.n2;
  // per warp: [g offsets][x rows of the WC cells][xg rows of the WC cells][A matrices of the WC cells]
  float* wbase = smem + (size_t)warp * A.warp_floats;
  long long* goff = reinterpret_cast<long long*>(wbase) + lc * kMaxParts;
  float* xs_cell = wbase + 2 * WC * kMaxParts + (size_t)lc * A.xcell_floats;
  float* xg_cell = wbase + 2 * WC * kMaxParts + (size_t)(WC + lc) * A.xcell_floats;
  float* cx = wbase + 2 * WC * kMaxParts + (size_t)2 * WC * A.xcell_floats + (size_t)lc * A.cx_floats;
  for (int q = lic; q < A.nr; q += CW) goff[q] = cell_ok ? cell_offset(A.r[q], A.cg, cell) : 0;
  for (int e = lic; e < A.xcell_floats; e += CW) xg_cell[e] = 0.f;
  if (A.sph) {  // one lane per cell generates the harmonics of the cell's point straight into the staged rows
    if (lic == 0) {
      const float* pt = A.sph + (cell_ok ? cell * A.sph_sb : 0);
      spharm_point(cell_ok ? pt[0] : 0.f, cell_ok ? pt[A.sph_sm] : 0.f, cell_ok ? pt[2 * A.sph_sm] : 1.f, A.sph_lmax, xs_cell,
                   A.xrow0, A.n1max);
    }
  } else {
    for (int i = 0; i < A.nx; i++) {
      const PartView& xp = A.x[i];
      const float* xb = xp.base + (cell_ok ? cell_offset(xp, A.cg, cell) : 0);
      const int total = (2 * xp.l + 1) * xp.n;
      for (int e = lic; e < total; e += CW) {
        const int m = e / xp.n, ch = e - m * xp.n;
        const float2 v = cell_ok ? __ldg(reinterpret_cast<const float2*>(xb + (long long)m * xp.sm + 2 * ch)) : make_float2(0.f, 0.f);
        *reinterpret_cast<float2*>(xs_cell + 2 * ((A.xrow0[i] + m) * A.n1max + ch)) = v;
      }
    }
  }
  __syncwarp();
  for (int yi = 0; yi < A.ny; yi++) {
    switch (A.yl[yi]) {
      case 0: bwd_l2<1>(A, xs_cell, xg_cell, cx, goff, yi, cell, lic, lic, ok); break;
      case 1: bwd_l2<3>(A, xs_cell, xg_cell, cx, goff, yi, cell, lic, lic, ok); break;
      case 2: bwd_l2<5>(A, xs_cell, xg_cell, cx, goff, yi, cell, lic, lic, ok); break;
      case 3: bwd_l2<7>(A, xs_cell, xg_cell, cx, goff, yi, cell, lic, lic, ok); break;
      case 4: bwd_l2<9>(A, xs_cell, xg_cell, cx, goff, yi, cell, lic, lic, ok); break;
      case 5: bwd_l2<11>(A, xs_cell, xg_cell, cx, goff, yi, cell, lic, lic, ok); break;
      case 6: bwd_l2<13>(A, xs_cell, xg_cell, cx, goff, yi, cell, lic, lic, ok); break;
      default: bwd_l2<15>(A, xs_cell, xg_cell, cx, goff, yi, cell, lic, lic, ok); break;
    }
  }
  __syncwarp();
  if (A.do_x && cell_ok) {
    for (int i = 0; i < A.nx; i++) {
      const PartView& xp = A.xg[i];
      float* xb = xp.base + cell_offset(xp, A.cg, cell);
      const int total = (2 * xp.l + 1) * xp.n;
      for (int e = lic; e < total; e += CW) {
        const int m = e / xp.n, ch = e - m * xp.n;
        const float2 v = *reinterpret_cast<const float2*>(xg_cell + 2 * ((A.xrow0[i] + m) * A.n1max + ch));
        float* q = xb + (long long)m * xp.sm + 2 * ch;
        if (A.x_atomic) {
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
  }
}

// Plan shared by the narrow kernels: triples in (xi, yi, l) order with dense coefficient matrices, pair index.
DevicePlan* narrow_plan(const VecCall& c) {
  std::vector<int> key = {6 /*family*/, (int)c.x.size(), (int)c.y.size(), (int)c.r.size()};
  for (const auto& p : c.x) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.y) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.r) key.push_back(p.l);
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  return get_plan(key, [&](DevicePlan& p) {
    build_schedule(xs, ys, rs, false, false, &p.sched);
    std::vector<int2> pairs(xs.size() * ys.size(), make_int2(0, 0));
    for (size_t t = 0; t < p.sched.triples.size(); t++) {
      Triple& tr = p.sched.triples[t];
      tr.coff = (int)p.sched.coeffs.size();
      for (int m1 = -tr.l1; m1 <= tr.l1; m1++)
        for (int m2 = -tr.l2; m2 <= tr.l2; m2++)
          p.sched.coeffs.push_back(std::abs(m1 + m2) <= tr.l ? (float)cg_coefficient(tr.l1, tr.l2, tr.l, m1, m2) : 0.f);
      int2& pr = pairs[(size_t)tr.yi * xs.size() + tr.xi];
      if (pr.y == 0) pr.x = (int)t;
      pr.y++;
    }
    for (const int2& q : pairs) {  // stored in the int job array, two ints per pair
      p.h_jobs.push_back(q.x);
      p.h_jobs.push_back(q.y);
    }
  });
}

// Fills the fields common to forward and backward; returns false when the call does not qualify.
bool narrow_setup(const VecCall& c, NarrowArgs& a) {
  if (c.x.empty() || c.y.empty() || c.r.empty() || !c.dense_channels) return false;
  const int n2 = c.y[0].n;
  int n1max = 0, lmaxr = 0;
  for (const auto& p : c.y) if (p.n != n2 || p.l > kMaxL2) return false;
  for (const auto& p : c.x) n1max = std::max(n1max, p.n);
  for (const auto& p : c.r) lmaxr = std::max(lmaxr, p.l);
  if (n2 > 32 || n2 < 1 || n1max > 4 || n1max < 1) return false;
  int CW = 1;
  while (CW < n2) CW *= 2;
  a.CW = CW;
  a.WC = 32 / CW;
  a.n2 = n2;
  a.n1max = n1max;
  int row = 0;
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    if (!c.xg.empty()) a.xg[i] = c.xg[i];
    a.xl[i] = c.x[i].l;
    a.xrow0[i] = row;
    row += 2 * c.x[i].l + 1;
  }
  a.xrows = row;
  a.xcell_floats = (2 * row * n1max + 3) / 4 * 4;
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    if (!c.yg.empty()) a.yg[i] = c.yg[i];
    a.yl[i] = c.y[i].l;
  }
  for (size_t i = 0; i < c.r.size(); i++) a.r[i] = c.r[i];
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.nr = (int)c.r.size();
  a.cx_floats = (2 * (2 * lmaxr + 1) * (2 * kMaxL2 + 2) + 3) / 4 * 4;
  a.cg = c.cg;
  a.offs_extra = c.offs_extra;
  a.accumulate = (c.flags & GELIB_OVERWRITE) ? 0 : 1;
  a.do_x = c.xg.empty() ? 0 : 1;
  a.do_y = c.yg.empty() ? 0 : 1;
  a.x_atomic = c.xg_bcast ? 1 : 0;
  a.y_atomic = c.yg_bcast ? 1 : 0;
  a.sph = c.sph;
  a.sph_sb = c.sph_sb;
  a.sph_sm = c.sph_sm;
  a.sph_lmax = c.sph_lmax;
  if (c.sph) {  // parts l = 0..lmax in order, one channel each, and no gradient with respect to them
    if (n1max != 1 || (int)c.x.size() != c.sph_lmax + 1 || c.sph_lmax > kSphPointMaxL || !c.xg.empty()) return false;
    for (size_t i = 0; i < c.x.size(); i++) if (c.x[i].l != (int)i) return false;
  }
  return true;
}

}  // namespace

int launch_cg_narrow_fwd(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addCGproduct";
  NarrowArgs a;
  if (!narrow_setup(c, a) || c.r_bcast) return -1;
  a.warp_floats = 2 * a.WC * kMaxParts + a.WC * a.xcell_floats + a.WC * a.cx_floats;
  const int nwarps = 8;
  const size_t smem = (size_t)nwarps * a.warp_floats * sizeof(float);
  if (smem > 200 * 1024) return -1;
  DevicePlan* plan = narrow_plan(c);
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->ntriples == 0 || c.cg.ncells == 0) return GELIB_OK;
  a.triples = plan->triples;
  a.coeffs = plan->coeffs;
  a.pairs = reinterpret_cast<const int2*>(plan->jobs);
  const long long blocks = (c.cg.ncells + (long long)a.WC * nwarps - 1) / ((long long)a.WC * nwarps);
  if (blocks > 0x7fffffffLL) return -1;
  cudaError_t e = cudaFuncSetAttribute(cg_narrow_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) cg_narrow_fwd_kernel<<<(unsigned)blocks, nwarps * 32, smem, s>>>(a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "narrow forward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200

namespace gelib_b200 {

int launch_cg_narrow_bwd(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addCGproduct_back";
  if (c.xg.empty() && narrow1_enabled()) {  // only the gradient of y is wanted: single-channel x has a kernel of its own
    const int st = launch_cg_narrow1_bwd(c, s);
    if (st != -1) return st;
  }
  NarrowArgs a;
  if (!narrow_setup(c, a)) return -1;
  for (const auto& p : c.y) {
    if (p.l > 7) return -1;  // 16 slots per lane at most
    int ns = 1;
    while (ns < 2 * p.l + 1) ns *= 2;
    if (ns > a.CW) return -1;  // the butterfly needs at least as many lanes per cell as slots
  }
  a.warp_floats = 2 * a.WC * kMaxParts + 2 * a.WC * a.xcell_floats + a.WC * a.cx_floats;
  const int nwarps = 8;
  const size_t smem = (size_t)nwarps * a.warp_floats * sizeof(float);
  if (smem > 200 * 1024) return -1;
  DevicePlan* plan = narrow_plan(c);
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->ntriples == 0 || c.cg.ncells == 0) return GELIB_OK;
  a.triples = plan->triples;
  a.coeffs = plan->coeffs;
  a.pairs = reinterpret_cast<const int2*>(plan->jobs);
  const long long blocks = (c.cg.ncells + (long long)a.WC * nwarps - 1) / ((long long)a.WC * nwarps);
  if (blocks > 0x7fffffffLL) return -1;
  cudaError_t e = cudaFuncSetAttribute(cg_narrow_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) cg_narrow_bwd_kernel<<<(unsigned)blocks, nwarps * 32, smem, s>>>(a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "narrow backward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
