// Backward Clebsch-Gordan product through the uncoupled gradient of each (l1,l2) pair: both gradients of every
// triple from ONE read of g, for channel counts that are multiples of 32.  Default backward kernel for such calls.
//
//   xg_l1[cell, m1, n1] += sum_{l,m2,n2} C_l[m1,m2] g_l[cell, m1+m2, offs_l + n1*N2 + n2] conj(y_l2[cell, m2, n2])
//   yg_l2[cell, m2, n2] += sum_{l,m1,n1} C_l[m1,m2] g_l[cell, m1+m2, offs_l + n1*N2 + n2] conj(x_l1[cell, m1, n1])
//
// Replaces SO3part_addCGproduct_back0_kernel / _back1_kernel and their launchers
// (cuda/SO3part_addCGproduct_back0.cu:32-294, cuda/SO3part_addCGproduct_back1.cu:32-175 of GElib), which read g
// twice, and the launch-per-triple loops Gvec::add_CGproduct_back0 / _back1 (core/Gvec.hpp:323-345).
//
// Arithmetic.  For a fixed pair (l1,l2) and a fixed row m = m1+m2, every output l >= |m| of the pair meets the SAME
// band of (m1,m2) and the same rows x[m1], y[m2]; only the coefficient differs.  So the kernel first forms, per band
// entry, the uncoupled gradient  H[n1][n2] = sum_l C_l[m1,m2] g_l[m][n1][n2]  (one real multiply-add per float) and
// contracts H with conj(y[m2]) and conj(x[m1]) once, instead of contracting every g_l separately: at maxl 6 that is
// 7651 combinations + 2149 contractions per cell in place of 7651 contractions (0.78 of the multiply-adds, 0.28 of
// the operand-row reads).
//
// Organisation.  One CTA per cell; the x and y rows of the cell live in shared memory.  A copy warp walks a list of
// groups -- (pair, 32 x 32 channel tile, row m, up to four output l) -- and brings the slabs g_l[m] of a group
// (32 rows of 256 bytes each), the group's coefficients and its two consumer descriptors into a four-stage ring:
// one thread issues two tensor copies per slab (cp.async.bulk.tensor, 128-byte swizzle, so both read patterns
// below are conflict-free without padding) and two bulk copies, all completing on the stage's mbarrier.  Views that a
// rank-5 tensor map cannot describe take four copy warps with 16-byte cp.async and rows padded to 272 bytes instead
// (one bulk copy per row was tried first and was bound by the copy engine's rate of 256-byte requests).
// Eight consumer warps share every group: warps 0-3 produce xg (lane = n1, each warp one quarter of n2, so the sum
// over n2 stays inside a lane), warps 4-7 produce yg (lane = n2, each warp one quarter of n1).  A warp copies its
// quarter of each slab into registers, forms H with packed f32x2 multiply-adds (one instruction per complex number
// and slab) and loops over the band, two entries at a time; the running sums for every m1 (resp. m2) of the pair live
// in a private shared-memory block of the warp (one 8-byte slot per lane and row: plain load / add / store,
// conflict-free) until the pair-tile ends, then go straight to global memory with one vector reduction
// (red.global.add.v2.f32) per complex number: the cell's rows stay in L2 until the CTA is done, and no CTA-wide
// accumulator, barrier or flush pass is left.  No shuffles and no atomics inside the band loop.  The four warps of a
// role, and the pairs that share a row, add in no fixed order, so gradients are reproducible to rounding (about 1e-7
// relative), not bitwise.
// Measured and slower: a second set of eight consumer warps on alternate groups (96 registers per thread: 18.4 ms
// against 15.3), groups of five to seven slabs (three stages instead of four), packed arithmetic for the
// contraction as well (needs the operands staged twice).
//
// Every wait on an mbarrier is bounded; on a timeout the kernel records it in a host-mapped status word, leaves its
// loops, lets its copies in flight land, and returns; the C ABI reports the failure on the next call.
#include <algorithm>
#include <array>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>

#include "plan.h"
#include "tc_common.h"
#include "tma_maps.h"

namespace gelib_b200 {

namespace {

using namespace tc;

constexpr int kSplit = 4;                            // warps per role: each takes 32 / kSplit of the other channel index (8 was tried: 19.7 ms)
constexpr int kCW = 32 / kSplit;                     // complex numbers per lane and slab
constexpr int kSetWarps = 2 * kSplit;                // warps that share a group: two roles x kSplit
constexpr int kGroupSlabs = 4;                       // slabs per group
constexpr int kMaxBand = 17;                         // band entries per group: 2*8+1
constexpr int kMaxStages = 4;
constexpr int kHeaderBytes = 768;                    // mbarriers, cell offsets, cell coordinates of the tensor maps
constexpr int kRec = 7;                              // int4 per group record

// A stage of the ring: the group's slabs, one coefficient quad per band entry, the two consumer descriptors
// (32 bytes each).  Two ways to fill it:
//   kTma = true   one thread issues two tensor copies (cp.async.bulk.tensor, 32 rows x 128 bytes, 128-byte swizzle)
//                 per slab and two bulk copies for coefficients and descriptors; a slab is 8192 bytes and a row's
//                 16-byte chunk c sits at chunk c ^ (row & 7) of its half row, so both read patterns are
//                 conflict-free without padding;
//   kTma = false  four warps issue 16-byte cp.async; slab rows are padded to 272 bytes.  For views whose strides
//                 or cell grid a five-dimensional tensor map cannot describe.
template <bool kTma>
struct Stage {
  static constexpr int kRowPitch = kTma ? 256 : 272;
  static constexpr int kSlotBytes = 32 * kRowPitch;
  static constexpr int kCoefOff = kGroupSlabs * kSlotBytes;
  static constexpr int kDescOff = kCoefOff + kMaxBand * 16;
  static constexpr int kBytes = (kDescOff + 64 + 1023) / 1024 * 1024;
  static constexpr int kProducers = kTma ? 1 : 4;    // copy warps
  // Sets of consumer warps; set s takes the groups with index = s mod kSets.  One set is what is built by default:
  // a second set leaves 96 registers per thread (five warps per scheduler) and measured 18.4 ms against 15.3.
#ifndef PAIR_SETS
#define PAIR_SETS 1
#endif
  static constexpr int kSets = kTma ? PAIR_SETS : 1;
  static constexpr int kConsumers = kSets * kSetWarps;
  static constexpr int kThreads = (kConsumers + kProducers) * 32;
  static constexpr int kMaxRegs = kTma && kSets == 2 ? 96 : 168;  // a scheduler's 16384 registers / its warps, in steps of 8
};

struct PairArgs {
  PartView x[kMaxParts], y[kMaxParts], g[kMaxParts], xg[kMaxParts], yg[kMaxParts];
  int xoff[kMaxParts], yoff[kMaxParts];  // float offsets of the staged parts inside the cell block
  int nx, ny, ng;
  int cell_floats;                       // staged floats per cell (the x rows, then the y rows)
  int nstages;
  CellGrid cg;
  // seven int4 per group.  [0..1] descriptor of the xg warps, [2..3] of the yg warps:
  //   {nslab | band length<<8 | last<<16 | accumulator rows of the pair<<24,
  //    byte offset in shared memory of the other operand's row for the first band entry (tile column 0),
  //    its signed step in bytes, byte offset of the first entry's row in a warp's private rows, its step (+-256),
  //    index of the gradient part the pair-tile adds to, float offset of the tile's first channel in a row, 0}
  //   last: bit 16 on the last group of the pair-tile, bit 17 on the last group of either parity
  // [4..6] for the producer:
  //   {nslab | band length<<8 | n2<<16, index of the first coefficient quad, 4 x {ri | (m+l)<<8 | map<<16 | colblk<<21,
  //    c1}, 0, 0}: the tile's first channel inside part ri is c1 * n2 + 32 * colblk
  const int4* recs;
  int ngroups;
  const float4* coef;                    // per band entry the coefficients of the group's slabs, zero-padded to 4
  int offs_extra;
  int do_x, do_y, x_atomic, y_atomic;
  unsigned tk[kMaxParts][6];             // tensor maps: (cell dim A, cell dim B) = (b, g0, g1) x these multipliers
  int skip_group;                        // test hook: the producer never signals this group (-1: none)
  int* status;                           // host-mapped; set to 1 when a wait ran out
};

// The mbarrier gets one arrival from this thread once all cp.async it has issued so far have landed (the count the
// barrier was initialised with already includes it).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Packed single precision (two lanes of one 64-bit register per instruction): the combination H = sum_l c_l G_l
// takes one instruction per complex number and slab instead of two.
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

// H = sum_l c_l G_l for the warp's 8 complex numbers, contracted with the conjugate of the other operand's 8.
template <int LM>
__device__ __forceinline__ void contract(const f32x2 (&G)[kGroupSlabs][kCW], const float4 c, const float4 (&w)[kCW / 2], float& sr,
                                         float& si) {
  float v[2 * kCW];
#pragma unroll
  for (int t = 0; t < kCW / 2; t++) {
    v[4 * t] = w[t].x; v[4 * t + 1] = w[t].y; v[4 * t + 2] = w[t].z; v[4 * t + 3] = w[t].w;
  }
  float H[2 * kCW];
  const f32x2 c0 = pack2(c.x, c.x), c1 = pack2(c.y, c.y), c2 = pack2(c.z, c.z), c3 = pack2(c.w, c.w);
#pragma unroll
  for (int j = 0; j < kCW; j++) {
    f32x2 h;
    if (LM == 1) {
      h = G[0][j];
    } else {
      h = mul2(c0, G[0][j]);
      h = fma2(c1, G[1][j], h);
      if (LM > 2) h = fma2(c2, G[2][j], h);
      if (LM > 3) h = fma2(c3, G[3][j], h);
    }
    unpack2(h, H[2 * j], H[2 * j + 1]);
  }
  float sr0 = 0.f, si0 = 0.f, sr1 = 0.f, si1 = 0.f;
#pragma unroll
  for (int e = 0; e < 2 * kCW; e += 4) {
    sr0 = fmaf(H[e], v[e], sr0);
    si0 = fmaf(H[e + 1], v[e], si0);
    sr1 = fmaf(H[e + 2], v[e + 2], sr1);
    si1 = fmaf(H[e + 3], v[e + 2], si1);
    sr0 = fmaf(H[e + 1], v[e + 1], sr0);
    si0 = fmaf(-H[e], v[e + 1], si0);
    sr1 = fmaf(H[e + 3], v[e + 3], sr1);
    si1 = fmaf(-H[e + 2], v[e + 3], si1);
  }
  sr = sr0 + sr1;
  si = si0 + si1;
  if (LM == 1) {
    sr *= c.x;
    si *= c.x;
  }
}

// The band of one group for one warp.  The loads of entry k+1 are issued before the arithmetic of entry k (two
// register sets, used alternately).  All positions are byte offsets into the CTA's shared memory.
// G: the warp's quarter of the group's slabs; coef: the group's coefficient quads; o: the other operand's row chunk
// for the first entry (4 x 16 bytes), ostep its signed step; a: the lane's slot in the warp's private accumulator
// row of the first entry, astep its signed step.
// Shared-memory accesses by 32-bit address with the offset folded into the instruction: the band loop keeps three
// address registers (coefficients, operand row, accumulator slot) and no 64-bit address arithmetic.  They are
// volatile, so they stay in program order: the loop below is written in the order it should issue.
template <int OFF>
__device__ __forceinline__ float4 lds128o(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a), "n"(OFF));
  return v;
}
__device__ __forceinline__ float2 lds64a(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void sts64a(uint32_t a, float2 v) {
  asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(a), "f"(v.x), "f"(v.y) : "memory");
}

struct BandEntry {
  float4 c, w[kCW / 2];
};
__device__ __forceinline__ void load_entry(BandEntry& e, uint32_t coef, uint32_t o) {
  e.c = lds128o<0>(coef);
  e.w[0] = lds128o<0>(o);
  e.w[1] = lds128o<16>(o);
  if (kCW > 4) {
    e.w[kCW / 2 - 2] = lds128o<32>(o);
    e.w[kCW / 2 - 1] = lds128o<48>(o);
  }
}
template <int LM>
__device__ __forceinline__ void use_entry(const f32x2 (&G)[kGroupSlabs][kCW], const BandEntry& e, uint32_t a) {
  float2 s = lds64a(a);
  float r, i;
  contract<LM>(G, e.c, e.w, r, i);
  s.x += r;
  s.y += i;
  sts64a(a, s);
}
// The band of one group for one warp.  The loads of entry k+1 are issued before the arithmetic of entry k (two
// register sets, used alternately).  All positions are 32-bit shared-memory addresses.
// G: the warp's quarter of the group's slabs; coef: the group's coefficient quads; o: the other operand's row chunk
// for the first entry, ostep its signed step in bytes; a: the lane's slot in the warp's private accumulator row of the
// first entry, astep its signed step.
template <int LM>
__device__ __forceinline__ void band_loop(const f32x2 (&G)[kGroupSlabs][kCW], uint32_t coef, int cnt, uint32_t o, int ostep,
                                          uint32_t a, int astep) {
  BandEntry A, B;
  load_entry(A, coef, o);
  int k = 0;
  for (; k + 2 < cnt; k += 2) {
    load_entry(B, coef + 16, o + ostep);
    use_entry<LM>(G, A, a);
    coef += 32;
    o += 2 * ostep;
    load_entry(A, coef, o);
    use_entry<LM>(G, B, a + astep);
    a += 2 * astep;
  }
  // one or two entries are left, the first of them loaded
  if (k + 1 < cnt) {
    load_entry(B, coef + 16, o + ostep);
    use_entry<LM>(G, A, a);
    use_entry<LM>(G, B, a + astep);
  } else {
    use_entry<LM>(G, A, a);
  }
}

__device__ __forceinline__ void stage_parts(float* dst_cell, const PartView* parts, const int* off, int nparts,
                                            const CellGrid& cg, long long cell) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = parts[i];
    const float* src = p.base + cell_offset(p, cg, cell);
    float* dst = dst_cell + off[i];
    const int n = p.n, total = (2 * p.l + 1) * n;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int m = e / n, ch = e - m * n;
      *reinterpret_cast<float2*>(dst + 2 * e) = __ldg(reinterpret_cast<const float2*>(src + (long long)m * p.sm + 2 * ch));
    }
  }
}

// One complex number added to global memory without a return value.
__device__ __forceinline__ void red_add2(float* dst, float2 v) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(__cvta_generic_to_global(dst)), "f"(v.x), "f"(v.y) : "memory");
}

// One tensor copy: 32 rows x 128 bytes of a slab (rank-5 map; the box is 32 x 32 x 1 x 1 x 1 floats).
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const void* map, int c0, int c1, int c2, int c3, int c4, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
      : "memory");
}
// A bulk copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) that completes on the mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

template <bool kTma>
__global__ void __maxnreg__(Stage<kTma>::kMaxRegs)
    cg_bwd_pair_kernel(const __grid_constant__ PairArgs A, const __grid_constant__ TmaMaps M, const int J) {
  using S = Stage<kTma>;
  constexpr int kConsumers = S::kConsumers;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);           // [kMaxStages]
  uint64_t* empty = full + kMaxStages;                               // [kMaxStages]
  long long* goff = reinterpret_cast<long long*>(smem_raw + 128);    // [kMaxParts] cell offsets into the g parts
  long long* xgoff = goff + kMaxParts;
  long long* ygoff = xgoff + kMaxParts;
  int* tcoord = reinterpret_cast<int*>(smem_raw + 512);              // [kMaxParts][2] the cell's coordinates in the maps
  float* stage_f = reinterpret_cast<float*>(smem_raw + kHeaderBytes);   // staged x,y rows of the cell
  float2* priv = reinterpret_cast<float2*>(stage_f + A.cell_floats);    // [kConsumers][J][32] private partial rows
  const int ring_off = (kHeaderBytes + 4 * A.cell_floats + kConsumers * J * 256 + 1023) & ~1023;
  unsigned char* ring = smem_raw + ring_off;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long cell = blockIdx.x;
  const int NS = A.nstages;

  if (kTma && (smem_u32(smem_raw) & 1023u) != 0) {  // the swizzle pattern is a function of the address
    if (threadIdx.x == 0) *A.status = 1;
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; s++) {
      // tensor copies: one arrival, by the thread that states the bytes to come; cp.async: one per producer lane
      mbar_init(&full[s], kTma ? 1 : 32 * S::kProducers);
      mbar_init(&empty[s], kSetWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int e = threadIdx.x; e < A.ng; e += blockDim.x) goff[e] = cell_offset(A.g[e], A.cg, cell);
  if (kTma) {
    for (int e = threadIdx.x; e < A.ng; e += blockDim.x) {
      const unsigned c = (unsigned)cell;
      const unsigned g1 = c % (unsigned)A.cg.G1, t = c / (unsigned)A.cg.G1;
      const unsigned g0 = t % (unsigned)A.cg.G0, b = t / (unsigned)A.cg.G0;
      tcoord[2 * e] = (int)(b * A.tk[e][0] + g0 * A.tk[e][1] + g1 * A.tk[e][2]);
      tcoord[2 * e + 1] = (int)(b * A.tk[e][3] + g0 * A.tk[e][4] + g1 * A.tk[e][5]);
    }
  }
  if (A.do_x)
    for (int e = threadIdx.x; e < A.nx; e += blockDim.x) xgoff[e] = cell_offset(A.xg[e], A.cg, cell);
  if (A.do_y)
    for (int e = threadIdx.x; e < A.ny; e += blockDim.x) ygoff[e] = cell_offset(A.yg[e], A.cg, cell);
  stage_parts(stage_f, A.x, A.xoff, A.nx, A.cg, cell);
  stage_parts(stage_f, A.y, A.yoff, A.ny, A.cg, cell);
  for (int e = threadIdx.x; e < kConsumers * J * 32; e += blockDim.x) priv[e] = make_float2(0.f, 0.f);
  __syncthreads();

  if (warp >= kConsumers) {
    // ---- producers: a group per stage
    const int pw = warp - kConsumers;
    bool ok = true;
    // Records are fetched 32 groups at a time, one group per lane, a batch ahead of their use, and handed round
    // with shuffles: the latency of the loads is paid once per batch, off the copy loop.
    auto fetch = [&](int g, int4& b0, int4& b1, int4& b2) {
      const int gg = g < A.ngroups ? g : A.ngroups - 1;
      b0 = __ldg(&A.recs[kRec * gg + 4]); b1 = __ldg(&A.recs[kRec * gg + 5]); b2 = __ldg(&A.recs[kRec * gg + 6]);
    };
    int4 b0 = make_int4(0, 0, 0, 0), b1 = b0, b2 = b0, nb0 = b0, nb1 = b0, nb2 = b0;
    if (A.ngroups > 0) fetch(lane, b0, b1, b2);
    // cp.async: lane t moves chunk t of two rows at a time (global reads of 512 contiguous bytes per instruction);
    // a slab takes 16 such instructions, four per warp
    const int rowi = 8 * pw + (lane >> 4), cc = lane & 15;   // first row this lane copies, and its 16-byte chunk
    const uint32_t ring_a = smem_u32(ring);
    int st = 0, phase = 0;
    bool first_round = true;
    for (int gi = 0; gi < A.ngroups; gi++) {
      const int k = gi & 31;
      if (k == 0 && gi + 32 < A.ngroups) fetch(gi + 32 + lane, nb0, nb1, nb2);
      int4 p0, p1, p2;
      p0.x = __shfl_sync(0xffffffffu, b0.x, k); p0.y = __shfl_sync(0xffffffffu, b0.y, k);
      p0.z = __shfl_sync(0xffffffffu, b0.z, k); p0.w = __shfl_sync(0xffffffffu, b0.w, k);
      p1.x = __shfl_sync(0xffffffffu, b1.x, k); p1.y = __shfl_sync(0xffffffffu, b1.y, k);
      p1.z = __shfl_sync(0xffffffffu, b1.z, k); p1.w = __shfl_sync(0xffffffffu, b1.w, k);
      p2.x = __shfl_sync(0xffffffffu, b2.x, k); p2.y = __shfl_sync(0xffffffffu, b2.y, k);
      if (!first_round) ok = mbar_wait(&empty[st], phase ^ 1);
      if (!ok) break;
      const int nslab = p0.x & 7, cnt = (p0.x >> 8) & 0xff, n2 = (p0.x >> 16) & 0xffff;
      const uint32_t sbase = ring_a + st * S::kBytes;
      const int sw[8] = {p0.z, p0.w, p1.x, p1.y, p1.z, p1.w, p2.x, p2.y};
      if (kTma) {
        if (lane == 0 && gi != A.skip_group) {
          const uint32_t bar = smem_u32(&full[st]);
          mbar_arrive_expect(bar, (uint32_t)(nslab * S::kSlotBytes + 64 + cnt * 16));
#pragma unroll
          for (int s = 0; s < kGroupSlabs; s++) {
            if (s < nslab) {
              const unsigned w = (unsigned)sw[2 * s];
              const int ri = w & 0xff, row = (w >> 8) & 0xff, slot = (w >> 16) & 0x1f, col = (int)(w >> 21) * 64;
              const int ca = tcoord[2 * ri], cb = tcoord[2 * ri + 1];
              tma_load_5d(sbase + s * S::kSlotBytes, &M.m[slot], col, sw[2 * s + 1], row, cb, ca, bar);
              tma_load_5d(sbase + s * S::kSlotBytes + 4096, &M.m[slot], col + 32, sw[2 * s + 1], row, cb, ca, bar);
            }
          }
          bulk_load(sbase + S::kCoefOff, A.coef + p0.y, (uint32_t)cnt * 16, bar);
          bulk_load(sbase + S::kDescOff, &A.recs[kRec * gi], 64, bar);
        }
      } else {
#pragma unroll
        for (int s = 0; s < kGroupSlabs; s++) {
          if (s < nslab) {
            const unsigned w = (unsigned)sw[2 * s];
            const int ri = w & 0xff, row = (w >> 8) & 0xff;
            const long long off = (long long)sw[2 * s + 1] * n2 + (int)(w >> 21) * 32;   // first channel of the tile
            const PartView& gp = A.g[ri];
            const float* src = gp.base + goff[ri] + (long long)row * gp.sm +
                               2LL * (off + A.offs_extra + (long long)rowi * n2) + 4 * cc;
            const uint32_t dst = sbase + s * S::kSlotBytes + rowi * S::kRowPitch + cc * 16;
            const long long step = 4LL * n2;  // two rows of the part, in floats
#pragma unroll
            for (int it = 0; it < 4; it++) cp_async16(dst + it * 2 * S::kRowPitch, src + it * step);
          }
        }
        if (pw == 0) {
          if (lane < cnt) cp_async16(sbase + S::kCoefOff + lane * 16, A.coef + p0.y + lane);
          if (lane < 4) cp_async16(sbase + S::kDescOff + lane * 16, &A.recs[kRec * gi + lane]);
        }
        if (gi != A.skip_group) cp_async_arrive(&full[st]);
      }
      if (++st == NS) {
        st = 0;
        phase ^= 1;
        first_round = false;
      }
      if (k == 31) {
        b0 = nb0; b1 = nb1; b2 = nb2;
      }
    }
    if (!kTma) cp_async_wait_all();  // nothing of this warp is in flight when the CTA gives its shared memory back
    if (!ok && lane == 0) *A.status = 1;
  } else {
    // ---- consumers
    const int set = warp / kSetWarps, role = (warp % kSetWarps) / kSplit, q = warp % kSplit;
    const bool active = role == 0 ? (A.do_x != 0) : (A.do_y != 0);
    float2* mine = priv + (warp * J) * 32 + lane;
    const int mine_off = kHeaderBytes + 4 * A.cell_floats + (warp * J * 32 + lane) * 8;  // the same as a byte offset
    const PartView* outs = role == 0 ? A.xg : A.yg;
    const long long* outoff = role == 0 ? xgoff : ygoff;
    const int last_bit = S::kSets == 1 ? 0x10000 : 0x20000;
    // Where the warp's quarter of a slab sits inside a slot.  xg warps read row `lane`, columns 8q..8q+7, as four
    // 16-byte chunks; yg warps read rows 8q..8q+7, column `lane`, as eight 8-byte loads (lanes adjacent).
    int goffs[kCW];
#pragma unroll
    for (int t = 0; t < kCW; t++) {
      if (kTma) {
        goffs[t] = role == 0 ? (q >> 1) * 4096 + lane * 128 + ((((q & 1) * 4 + (t & 3)) ^ (lane & 7)) << 4)
                             : (lane >> 4) * 4096 + (kCW * q + t) * 128 + (((((lane & 15) >> 1) ^ t) & 7) << 4) + (lane & 1) * 8;
      } else {
        goffs[t] = role == 0 ? lane * S::kRowPitch + q * (8 * kCW) + (t & 3) * 16 : (kCW * q + t) * S::kRowPitch + lane * 8;
      }
    }
    bool ok = true;
    int st = set % NS, phase = (set / NS) & 1;
    for (int gi = set; gi < A.ngroups; gi += S::kSets) {
      ok = mbar_wait(&full[st], phase);
      if (!ok) break;
      if (active) {
        const unsigned char* sbase = ring + st * S::kBytes;
        const int4 d0 = *reinterpret_cast<const int4*>(sbase + S::kDescOff + role * 32);
        const int4 d1 = *reinterpret_cast<const int4*>(sbase + S::kDescOff + role * 32 + 16);
        const int nslab = d0.x & 7, cnt = (d0.x >> 8) & 0xff;
        f32x2 G[kGroupSlabs][kCW];
        if (role == 0) {
#pragma unroll
          for (int s = 0; s < kGroupSlabs; s++) {
            if (s < nslab) {
#pragma unroll
              for (int t = 0; t < kCW / 2; t++) {
                const ulonglong2 w = *reinterpret_cast<const ulonglong2*>(sbase + s * S::kSlotBytes + goffs[t]);
                G[s][2 * t] = w.x; G[s][2 * t + 1] = w.y;
              }
            }
          }
        } else {
#pragma unroll
          for (int s = 0; s < kGroupSlabs; s++) {
            if (s < nslab) {
#pragma unroll
              for (int r = 0; r < kCW; r++) G[s][r] = *reinterpret_cast<const f32x2*>(sbase + s * S::kSlotBytes + goffs[r]);
            }
          }
        }
        const uint32_t s0 = smem_u32(smem_raw), cf = s0 + ring_off + st * S::kBytes + S::kCoefOff;
        const uint32_t o = s0 + d0.y + q * (8 * kCW), a = s0 + mine_off + d0.w;
        switch (nslab) {
          case 1: band_loop<1>(G, cf, cnt, o, d0.z, a, d1.x); break;
          case 2: band_loop<2>(G, cf, cnt, o, d0.z, a, d1.x); break;
          case 3: band_loop<3>(G, cf, cnt, o, d0.z, a, d1.x); break;
          default: band_loop<4>(G, cf, cnt, o, d0.z, a, d1.x); break;
        }
        if (d0.x & last_bit) {  // the set's last group of the pair-tile: the warp's partial rows go to global memory
          const int rows = (d0.x >> 24) & 0xff;
          const PartView& op = outs[d1.y];
          float* dst = op.base + outoff[d1.y] + d1.z + 2 * lane;
          for (int j = 0; j < rows; j++) {
            const float2 v = mine[j * 32];
            mine[j * 32] = make_float2(0.f, 0.f);
            red_add2(dst + j * op.sm, v);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);  // the stage (slabs, coefficients, descriptors) is free again
      st += S::kSets;
      if (st >= NS) {  // NS >= kSets
        st -= NS;
        phase ^= 1;
      }
    }
    if (!ok && lane == 0) *A.status = 1;
  }
}

}  // namespace

namespace {

// The maps of the g parts of one call; `info` is the plan's list {maps fit, number of maps, then per map: part, N2, rows}.
bool encode_maps(const VecCall& c, const std::vector<int>& info, PairArgs& a, TmaMaps& maps) {
  if (info.size() < 2 || !info[0]) return false;
  return encode_part_maps(c.r, c.cg, c.offs_extra, info[1], info.data() + 2, a.tk, maps);
}

}  // namespace

// Returns -1 when the call does not qualify (the caller then takes the kernel of cg_bwd.cu).
int launch_cg_bwd_pair(const VecCall& c, cudaStream_t s, int min_groups) {
  static const char* fn = "SO3vec_addCGproduct_back";
  if (!c.vec_ok) return -1;
  if (c.x.empty() || c.y.empty() || c.r.empty()) return -1;
  int lmax = 0;
  for (const auto& p : c.x) { if (p.n % 32 || p.n > 32768) return -1; lmax = std::max(lmax, p.l); }
  for (const auto& p : c.y) { if (p.n % 32 || p.n > 32768) return -1; lmax = std::max(lmax, p.l); }
  for (const auto& p : c.r) if (p.l > 16) return -1;
  if (lmax > 8) return -1;
  if (c.cg.ncells > 0x7fffffffLL) return -1;
  int* status = async_status_word(kStatusBwdPair);
  if (!status) return -1;
  const int J = 2 * lmax + 1;

  PairArgs a;
  int off = 0;
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    if (!c.xg.empty()) a.xg[i] = c.xg[i];
    a.xoff[i] = off;
    off += 2 * (2 * c.x[i].l + 1) * c.x[i].n;
  }
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    if (!c.yg.empty()) a.yg[i] = c.yg[i];
    a.yoff[i] = off;
    off += 2 * (2 * c.y[i].l + 1) * c.y[i].n;
  }
  for (size_t i = 0; i < c.r.size(); i++) a.g[i] = c.r[i];
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.ng = (int)c.r.size();
  a.cell_floats = off;
  auto fixed_bytes = [&](int consumers) {
    return ((size_t)kHeaderBytes + (size_t)4 * off + (size_t)consumers * J * 256 + 1023) & ~(size_t)1023;
  };
  auto stages_that_fit = [&](size_t fixed, size_t stage_bytes) {
    int ns = kMaxStages;
    while (ns >= 2 && fixed + (size_t)ns * stage_bytes > 227 * 1024) ns--;
    return ns;
  };
  if (stages_that_fit(fixed_bytes(Stage<false>::kConsumers), Stage<false>::kBytes) < 2) return -1;

  std::vector<int> key = {10 /*family*/, (int)c.x.size(), (int)c.y.size(), (int)c.r.size()};
  for (const auto& p : c.x) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.y) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.r) key.push_back(p.l);
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  const int *xoff = a.xoff, *yoff = a.yoff;
  DevicePlan* plan = get_plan(key, [&](DevicePlan& p) {
    build_schedule(xs, ys, rs, false, true, &p.sched);
    // triples of each (xi, yi) pair, in schedule order (l ascending)
    std::map<std::pair<int, int>, std::vector<const Triple*>> pairs;
    for (const Triple& t : p.sched.triples) pairs[{t.xi, t.yi}].push_back(&t);
    std::vector<float>& quads = p.h_floats;
    // tensor maps of a call: one per (g part, N2); h_jobs = {maps fit, number of maps, then per map: part, N2, rows}
    std::map<std::pair<int, int>, int> slots;
    std::vector<int> slot_rows;
    bool maps_fit = true;
    for (const auto& kv : pairs) {
      const auto& ts = kv.second;
      const int xi = kv.first.first, yi = kv.first.second;
      const int l1 = xs[xi].l, l2 = ys[yi].l, n1 = xs[xi].n, n2 = ys[yi].n;
      int lm = 0;
      for (const Triple* t : ts) lm = std::max<int>(lm, t->l);
      for (int a0 = 0; a0 < n1; a0 += 32)
        for (int b0 = 0; b0 < n2; b0 += 32) {
          const size_t first_rec = p.h_items.size();
          for (int m = -lm; m <= lm; m++) {
            const int lo = std::max(-l1, m - l2), hi = std::min(l1, m + l2);
            const int cnt = hi - lo + 1, jlo = lo + l1, j2hi = m - lo + l2;
            std::vector<const Triple*> act;
            for (const Triple* t : ts)
              if (t->l >= std::abs(m)) act.push_back(t);
            for (size_t c0 = 0; c0 < act.size(); c0 += kGroupSlabs) {
              const int nslab = (int)std::min<size_t>(kGroupSlabs, act.size() - c0);
              int sw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
              for (int sidx = 0; sidx < nslab; sidx++) {
                const Triple* t = act[c0 + sidx];
                // the part's channels of one (cell, row) as a matrix with rows of n2: the tile starts at row c1,
                // column 32 * colblk, and its 32 rows are 32 consecutive rows of that matrix
                const int off = t->offs + a0 * n2 + b0, c1 = off / n2, colblk = (off % n2) / 32;
                auto it = slots.find({t->ri, n2});
                if (it == slots.end()) {
                  it = slots.emplace(std::make_pair((int)t->ri, n2), (int)slots.size()).first;
                  slot_rows.push_back(0);
                }
                const int slot = it->second;
                if (slot >= kMaxMaps || colblk >= 1024) maps_fit = false;
                slot_rows[slot] = std::max(slot_rows[slot], c1 + 32);
                sw[2 * sidx] = (int)((unsigned)t->ri | ((unsigned)(m + t->l) << 8) | ((unsigned)(slot & 0x1f) << 16) |
                                     ((unsigned)(colblk & 0x3ff) << 21));
                sw[2 * sidx + 1] = c1;
              }
              const int head = nslab | (cnt << 8);
              // xg warps: y rows downwards from m2 = m - lo, accumulator rows upwards from m1 = lo
              p.h_items.push_back(make_int4(head | ((2 * l1 + 1) << 24), kHeaderBytes + 4 * (yoff[yi] + 2 * b0 + 2 * n2 * j2hi),
                                            -8 * n2, 256 * jlo));
              p.h_items.push_back(make_int4(256, xi, 2 * a0, 0));
              // yg warps: x rows upwards from m1 = lo, accumulator rows downwards from m2 = m - lo
              p.h_items.push_back(make_int4(head | ((2 * l2 + 1) << 24), kHeaderBytes + 4 * (xoff[xi] + 2 * a0 + 2 * n1 * jlo),
                                            8 * n1, 256 * j2hi));
              p.h_items.push_back(make_int4(-256, yi, 2 * b0, 0));
              p.h_items.push_back(make_int4(head | (n2 << 16), (int)(quads.size() / 4), sw[0], sw[1]));
              p.h_items.push_back(make_int4(sw[2], sw[3], sw[4], sw[5]));
              p.h_items.push_back(make_int4(sw[6], sw[7], 0, 0));
              for (int m1 = lo; m1 <= hi; m1++)
                for (int sidx = 0; sidx < kGroupSlabs; sidx++) {
                  float cf = 0.f;
                  if (sidx < nslab) {
                    const Triple* t = act[c0 + sidx];
                    // band order of the schedule's table: rows m ascending, m1 ascending within a row
                    int pos = t->coff;
                    for (int mm = -t->l; mm < m; mm++)
                      pos += std::min<int>(l1, mm + l2) - std::max<int>(-l1, mm - l2) + 1;
                    cf = p.sched.coeffs[pos + (m1 - lo)];
                  }
                  quads.push_back(cf);
                }
            }
          }
          // mark the last group of the pair-tile in both descriptors (bit 16), and the last group of either parity
          // (bit 17: with two sets of consumer warps, each set's last group of the tile)
          for (size_t b = 1; b <= 2 && p.h_items.size() >= first_rec + b * kRec; b++) {
            const int bits = b == 1 ? 0x30000 : 0x20000;
            p.h_items[p.h_items.size() - b * kRec].x |= bits;
            p.h_items[p.h_items.size() - b * kRec + 2].x |= bits;
          }
        }
    }
    p.h_jobs.assign(2 + 3 * slots.size(), 0);
    p.h_jobs[0] = maps_fit ? 1 : 0;
    p.h_jobs[1] = (int)slots.size();
    for (const auto& kv : slots) {
      p.h_jobs[2 + 3 * kv.second] = kv.first.first;
      p.h_jobs[3 + 3 * kv.second] = kv.first.second;
      p.h_jobs[4 + 3 * kv.second] = slot_rows[kv.second];
    }
    long long entries = 0;  // band entries of all groups: the last word of the list
    for (size_t g = 0; g < p.h_items.size(); g += kRec) entries += (p.h_items[g].x >> 8) & 0xff;
    p.h_jobs.push_back((int)std::min<long long>(entries, 0x7fffffffLL));
  });
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->nitems == 0 || c.cg.ncells == 0) return GELIB_OK;
  // a cell with only a few groups does not fill the pipeline of 12 warps: the one-slab-per-warp kernel is faster there
  // Automatic choice: the kernel pays a fixed cost per group (handshake, slab loads into registers) that short bands
  // do not repay.  Measured against the kernel of cg_bwd.cu at 32 channels: maxl 4 (188 groups, 3.1 entries per
  // group) 7.98 against 8.15 ms, maxl 3 (92 groups, 2.5 entries per group) 7.37 against 6.25, maxl 2 6.12 against 4.08;
  // at 64 channels maxl 3 (368 groups, 2.5 entries per group) 3.46 against 2.91.
  if (min_groups > 0) {
    const long long ng = plan->nitems / kRec, entries = plan->h_jobs.empty() ? 0 : plan->h_jobs.back();
    if (ng < min_groups || entries < 3 * ng) return -1;
  }

  a.cg = c.cg;
  a.recs = plan->items;
  a.ngroups = plan->nitems / kRec;
  a.coef = reinterpret_cast<const float4*>(plan->floats);
  a.offs_extra = c.offs_extra;
  a.do_x = c.xg.empty() ? 0 : 1;
  a.do_y = c.yg.empty() ? 0 : 1;
  a.x_atomic = c.xg_bcast ? 1 : 0;
  a.y_atomic = c.yg_bcast ? 1 : 0;
  a.skip_group = inject_timeout() ? 0 : -1;
  a.status = status;

  TmaMaps maps;
  memset(&maps, 0, sizeof(maps));
  const size_t fixed_tma = fixed_bytes(Stage<true>::kConsumers), fixed = fixed_bytes(Stage<false>::kConsumers);
  const bool tma = pair_tma() && stages_that_fit(fixed_tma, Stage<true>::kBytes) >= 3 && encode_maps(c, plan->h_jobs, a, maps);
  cudaError_t e;
  if (tma) {
    a.nstages = stages_that_fit(fixed_tma, Stage<true>::kBytes);
    const size_t smem = fixed_tma + (size_t)a.nstages * Stage<true>::kBytes;
    e = cudaFuncSetAttribute(cg_bwd_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) {
      cg_bwd_pair_kernel<true><<<(unsigned)c.cg.ncells, Stage<true>::kThreads, smem, s>>>(a, maps, J);
      e = cudaGetLastError();
    }
  } else {
    a.nstages = stages_that_fit(fixed, Stage<false>::kBytes);
    const size_t smem = fixed + (size_t)a.nstages * Stage<false>::kBytes;
    e = cudaFuncSetAttribute(cg_bwd_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) {
      cg_bwd_pair_kernel<false><<<(unsigned)c.cg.ncells, Stage<false>::kThreads, smem, s>>>(a, maps, J);
      e = cudaGetLastError();
    }
  }
  if (e != cudaSuccess) return check_cuda(e, fn, "pair backward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
