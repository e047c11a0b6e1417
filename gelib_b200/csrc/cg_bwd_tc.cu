// Backward Clebsch-Gordan product on the 5th-generation tensor cores (tcgen05 + tensor memory), for channel
// counts that are multiples of 32.  Same mathematics as cg_bwd.cu; replaces the same reference code
// (cuda/SO3part_addCGproduct_back0.cu:32-294, cuda/SO3part_addCGproduct_back1.cu:32-175 and the loops
// Gvec::add_CGproduct_back0 / _back1, core/Gvec.hpp:323-345 of GElib).
//
// Formulation.  A slab is one row m of one triple (l1,l2)->l restricted to a 32 x 32 channel tile of g:
// G[n1][n2], 8 KB.  For the slab, against ALL rows m2 of y_l2 and ALL rows m1 of x_l1,
//     P[n1][(m2,part)] = sum_{n2,c} G_c[n1][n2] By[(n2,c)][(m2,part)]      (part = re | im of g conj(y))
//     Q[n2][(m1,part)] = sum_{n1,c} G_c[n1][n2] Bx[(n1,c)][(m1,part)]
// with By[(n2,re)] = (y_r | -y_i), By[(n2,im)] = (y_i | y_r) and the same for x, are real GEMMs with K = 64.  Four
// slabs that share (l1,l2) and the tile are stacked to M = 128 rows; N = 16 or 32 covers the 2(2l+1) rows of
// the other operand.  Only the band |m - m2| <= l1 (resp. |m - m1| <= l2) of the result is used: the
// epilogue scales those columns by the Clebsch-Gordan coefficient and adds them to the gradient rows,
//     xg[m1][n1] += C(m1, m-m1) P[n1][m2 = m-m1],      yg[m2][n2] += C(m-m2, m2) Q[n2][m1 = m-m2].
// The MMAs run as tcgen05.mma kind::tf32 with the 3xTF32 split (a = a_hi + a_lo with a_hi the upper 19 bits;
// a_lo b_hi + a_hi b_lo + a_hi b_hi, FP32 accumulation in tensor memory), which keeps FP32-level accuracy.
//
// Data movement.  One CTA per (cell, product): the P CTA holds the y tables and the x gradient rows, the Q CTA the x
// tables and the y gradient rows; the two CTAs of a cell start next to each other, so the second read of a slab
// normally comes from L2.  At start the CTA writes its tables to shared memory once, already split and in the
// K-major core-matrix layout the B operand descriptor wants (rows 2*mi and 2*mi+1 = the two parts).  Sixteen warps
// each own one slab at a time: cp.async brings it into the warp's 8 KB ring slot (16-byte chunks XOR-swizzled by
// row); the warp reads it row-per-lane (P: lane = n1, columns (n2,c)) or column-per-lane (Q: lane = n2, columns
// (n1,c)), splits it and stores it to tensor memory as the A operand, one K half (32 of the 64 columns) at a time;
// A never passes through shared memory again.  Four sets of four warps own 128 tensor-memory columns each (A hi 32,
// A lo 32, two accumulators of 32): the warp whose store completes an operand half (a shared-memory arrival counter)
// issues its 12 MMAs and a tcgen05.commit; the second half is read and the ring slot refilled while the first
// half's MMAs run, and the previous group's accumulator is added to the gradient rows while the second half's run.
// The epilogue reads the accumulator row of its lane with tcgen05.ld at the columns of the band and adds into
// gradient rows in shared memory with batched 64-bit compare-and-swap; the rows go to global memory once at the
// end.  Gradients are reproducible to rounding, not bitwise.
//
// Every wait on an mbarrier is bounded; on a timeout the kernel records it in a host-mapped status word,
// leaves its loops, frees its tensor memory and returns, and the next call reports the failure.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>

#include "plan.h"
#include "tc_common.h"

namespace gelib_b200 {

namespace {

using namespace tc;

constexpr int kWorkers = 16;          // four sets of four slabs, one warp per slab
constexpr int kThreads = 32 * kWorkers;
constexpr int kSlots = 16;            // ring slots (one slab each, one per warp)
constexpr int kSlabBytes = 32 * 32 * 8;
constexpr int kHeaderBytes = 896;     // mbarriers, tensor-memory base, cell offsets, g row pointers
constexpr int kRec = 22;              // int4 per group record

struct TcArgs {
  PartView x[kMaxParts], y[kMaxParts], g[kMaxParts], xg[kMaxParts], yg[kMaxParts];
  int xacc[kMaxParts], yacc[kMaxParts];  // float offsets of the gradient rows inside the accumulator block
  int xbt[kMaxParts], ybt[kMaxParts];    // byte offsets of the operand tables inside the table block
  int xR[kMaxParts], yR[kMaxParts];      // table rows per part: 2(2l+1) rounded up to 8
  int nx, ny, ng;
  int bt_bytes, acc_floats;
  CellGrid cg;
  const float* coeffs;
  // six int4 per group of up to four slabs (nothing in the loops indexes the parameter arrays):
  //   {xi | yi<<4 | l1<<8 | l2<<16, a0 | b0<<16, n1 | n2<<16 (channels of the x and y part), xacc | yacc<<16}
  //   {byte offset of the y table of the tile, its rows, byte offset of the x table of the tile, its rows}
  //   4 x {ri | valid<<8, l | (m+l)<<8, channel offset of the tile inside part ri, coefficient index}
  //   4 x 16 floats: the band coefficients of the slab's row, zero-padded
  const int4* groups;
  int ngroups;
  int offs_extra;
  int x_atomic, y_atomic;
  int* status;  // host-mapped: set to 1 when a wait timed out
};

// ---- PTX wrappers: tc_common.h ------------------------------------------------------------------------------

// Splits 8 values and stores them to columns [col, col+8) of the hi block and of the lo block (32 columns on).
// Eight at a time keeps the live registers low.
__device__ __forceinline__ void split_store8(uint32_t tA, int col, const float (&v)[8]) {
  uint32_t hi[8], lo[8];
#pragma unroll
  for (int i = 0; i < 8; i++) split_tf32(v[i], hi[i], lo[i]);
  tmem_st8(tA + col, hi);
  tmem_st8(tA + 32 + col, lo);
}

// ---- kernel pieces ---------------------------------------------------------------------------------------------

// Everything a worker needs for its slab of one group, kept packed as loaded (registers are scarce here).
struct Work {
  int4 h;      // {xi | yi<<4 | l1<<8 | l2<<16, a0 | b0<<16, n1 | n2<<16, xacc | yacc<<16}
  int4 r;      // {ri | valid<<8, l | (m+l)<<8, channel offset of the tile inside part ri, coefficient index}
  int4 t;      // {y table byte offset, y rows, x table byte offset, x rows}: for the warp that issues the MMAs
  float cvec;  // band coefficient j of the slab's row in lane j (at most 15 entries)
  __device__ __forceinline__ int l1() const { return (h.x >> 8) & 0xff; }
  __device__ __forceinline__ int l2() const { return (h.x >> 16) & 0xff; }
  __device__ __forceinline__ int a0() const { return h.y & 0xffff; }
  __device__ __forceinline__ int b0() const { return (h.y >> 16) & 0xffff; }
  __device__ __forceinline__ int n1() const { return h.z & 0xffff; }
  __device__ __forceinline__ int n2() const { return (h.z >> 16) & 0xffff; }
  __device__ __forceinline__ int xacc() const { return h.w & 0xffff; }
  __device__ __forceinline__ int yacc() const { return (h.w >> 16) & 0xffff; }
  __device__ __forceinline__ int ri() const { return r.x & 0xff; }
  __device__ __forceinline__ bool valid() const { return (r.x >> 8) & 1; }
  __device__ __forceinline__ int m() const { return (r.y >> 8) - (r.y & 0xff); }
};

// All three loads depend on the group number only, so a group's record can be fetched a whole group ahead.
__device__ __forceinline__ void load_work(const TcArgs& A, int g, int q, int lane, Work& w) {
  w.h = __ldg(&A.groups[kRec * g]);
  w.r = __ldg(&A.groups[kRec * g + 2 + q]);
  w.t = __ldg(&A.groups[kRec * g + 1]);
  w.cvec = lane < 16 ? __ldg(reinterpret_cast<const float*>(&A.groups[kRec * g + 6 + 4 * q]) + lane) : 0.f;
}

__device__ __noinline__ void fill_offsets(long long* dst, const PartView* parts, int nparts, const CellGrid& cg, long long cell) {
  for (int p = threadIdx.x; p < nparts; p += blockDim.x) dst[p] = cell_offset(parts[p], cg, cell);
}

// Writes the rows of every part of one vector as split B-operand tables.  Table of (part, 32-channel tile):
// a hi block and a lo block of [16 k-chunks][R rows][4 floats] each; row 2*mi holds (v_r, v_i) pairs, row 2*mi+1
// (-v_i, v_r) pairs of row mi, so that one k-chunk is two complex channels.
__device__ __noinline__ void stage_tables(unsigned char* bt, const PartView* parts, const int* off, const int* Rs,
                                             int nparts, const CellGrid& cg, long long cell) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = parts[i];
    const float* src = p.base + cell_offset(p, cg, cell);
    const int T = p.n >> 5, R = Rs[i];
    const int total = (2 * p.l + 1) * T * 16;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int kc = e & 15, t = (e >> 4) % T, mi = (e >> 4) / T;
      const float4 v = __ldg(reinterpret_cast<const float4*>(src + (long long)mi * p.sm + 2 * (32 * t + 2 * kc)));
      const float re[4] = {v.x, v.y, v.z, v.w}, im[4] = {-v.y, v.x, -v.w, v.z};
      uint32_t rh[4], rl[4], ih[4], il[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        split_tf32(re[k], rh[k], rl[k]);
        split_tf32(im[k], ih[k], il[k]);
      }
      unsigned char* tile = bt + off[i] + t * (512 * R);
      uint4* hi = reinterpret_cast<uint4*>(tile + (kc * R + 2 * mi) * 16);
      uint4* lo = reinterpret_cast<uint4*>(tile + 256 * R + (kc * R + 2 * mi) * 16);
      hi[0] = make_uint4(rh[0], rh[1], rh[2], rh[3]);
      hi[1] = make_uint4(ih[0], ih[1], ih[2], ih[3]);
      lo[0] = make_uint4(rl[0], rl[1], rl[2], rl[3]);
      lo[1] = make_uint4(il[0], il[1], il[2], il[3]);
    }
  }
}

// The 12 MMAs of one K half of a group's product: D[128 x N] (+)= A_lo B_hi + A_hi B_lo + A_hi B_hi over 32 of the
// K = 64 in steps of 8.  tA: tensor-memory column of the set's A block (hi at +0, lo at +32); table: shared address
// of the B table; half: which 32 K values; init: overwrite the accumulator (first half) or add to it.
__device__ __forceinline__ void issue_half(uint32_t tA, uint32_t tD, uint32_t table, int R, int half, bool init) {
  const uint32_t N = R <= 16 ? 16u : 32u;
  // instruction descriptor: D = F32, A = B = TF32, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((N >> 3) << 17) | ((128u >> 4) << 24);
  // shared-memory descriptor, no swizzle, K-major: start >> 4, leading (k-chunk) offset R*16 B, stride (8-row
  // group) offset 128 B, descriptor version 1; a half is 8 k-chunks = 128 R bytes on
  const uint64_t fixed = ((uint64_t)R << 16) | (8ull << 32) | (1ull << 46);
  const uint32_t t0 = table + 128u * R * half;
  const uint64_t dhi = fixed | ((t0 >> 4) & 0x3fffu), dlo = fixed | (((t0 + 256u * R) >> 4) & 0x3fffu);
  const uint64_t kstep = 2ull * R;  // two k-chunks per MMA, in 16-byte units
#pragma unroll
  for (int term = 0; term < 3; term++) {
    const uint32_t a = term == 0 ? tA + 32 : tA;  // a_lo b_hi, a_hi b_lo, a_hi b_hi: smallest terms first
    const uint64_t b = term == 1 ? dlo : dhi;
#pragma unroll
    for (int ks = 0; ks < 4; ks++) mma_tf32_ts(tD, a + 8 * ks, b + ks * kstep, idesc, !init || (term | ks) != 0);
  }
}

// Adds the band of one accumulator row to the gradient rows.  The accumulator of the lane's channel holds, for
// every row index idx of the other operand (lb = its l), the complex sum in columns 2 idx, 2 idx + 1.
//   FOR_X: idx <-> m2, target row m1 = m - m2 of x;   else: idx <-> m1, target row m2 = m - m1 of y.
// cvec: the row's band coefficients, entry j in lane j.
// The additions are 64-bit compare-and-swap updates of the complex gradient entries, four band entries at a
// time (all accumulator reads, all loads, all swaps, then retries of the few that lost a race) so that their
// latencies overlap; shared memory has no native float add, and an atomicAdd per float would serialise a
// loop per entry.
template <bool FOR_X>
__device__ __forceinline__ void epilogue(uint32_t tD, uint32_t accrows, int ntot, int ch, int m, int l1, int l2,
                                         float cvec) {
  const int lo = max(-l1, m - l2), hi = min(l1, m + l2);
  const int lb = FOR_X ? l2 : l1, lt = FOR_X ? l1 : l2;
  const int i0 = FOR_X ? (m - hi + lb) : (lo + lb), i1 = FOR_X ? (m - lo + lb) : (hi + lb);  // the band of idx
  // entry idx: coefficient lane cl0 + cls * idx, target row (m + lb + lt) - idx
  const int cl0 = FOR_X ? (m + lb - lo) : (-lb - lo), cls = FOR_X ? -1 : 1;
  const uint32_t rowb = 8u * ntot;
  const uint32_t chan = accrows + 8u * ch + (uint32_t)(m + lb + lt) * rowb;  // minus idx * rowb: the entry's address
  auto pack = [](float re, float im) { return ((unsigned long long)__float_as_uint(im) << 32) | __float_as_uint(re); };
  for (int j0 = i0; j0 <= i1; j0 += 4) {
    uint32_t dv[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int idx = min(j0 + i, i1);
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(dv[2 * i]), "=r"(dv[2 * i + 1]) : "r"(tD + 2 * idx) : "memory");
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(dv[0]), "+r"(dv[1]), "+r"(dv[2]), "+r"(dv[3]), "+r"(dv[4]), "+r"(dv[5]), "+r"(dv[6]), "+r"(dv[7])::"memory");
    unsigned long long oldv[4], got[4];
    uint32_t ptr[4];
    float2 add[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int idx = min(j0 + i, i1);
      const float c = __shfl_sync(0xffffffffu, cvec, cl0 + cls * idx);
      add[i] = make_float2(c * __uint_as_float(dv[2 * i]), c * __uint_as_float(dv[2 * i + 1]));
      ptr[i] = chan - (uint32_t)idx * rowb;
      oldv[i] = lds_u64(ptr[i]);
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
      if (j0 + i <= i1)
        got[i] = cas_shared_u64(ptr[i], oldv[i],
                                pack(__uint_as_float((uint32_t)oldv[i]) + add[i].x, __uint_as_float((uint32_t)(oldv[i] >> 32)) + add[i].y));
#pragma unroll
    for (int i = 0; i < 4; i++)
      if (j0 + i <= i1)
        while (got[i] != oldv[i]) {  // another warp updated the entry in between: redo on its value
          oldv[i] = got[i];
          got[i] = cas_shared_u64(ptr[i], oldv[i],
                                  pack(__uint_as_float((uint32_t)oldv[i]) + add[i].x, __uint_as_float((uint32_t)(oldv[i] >> 32)) + add[i].y));
        }
  }
}

__device__ __noinline__ void flush_rows(const float* acc, const PartView* out, const long long* cell_off,
                                           const int* off, int nparts, bool atomic) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = out[i];
    const int n = p.n, total = (2 * p.l + 1) * n;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int row = e / n, ch = e - row * n;
      const float2 v = *reinterpret_cast<const float2*>(acc + off[i] + 2 * e);
      float* dst = p.base + cell_off[i] + (long long)row * p.sm + 2 * ch;
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

// ---- the kernel ------------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads, 1) cg_bwd_tc_kernel(const __grid_constant__ TcArgs A) {
  extern __shared__ __align__(128) unsigned char sm[];
  uint64_t* mdone = reinterpret_cast<uint64_t*>(sm);  // [4] MMAs of a set's current K half complete (tcgen05.commit)
  int* ev = reinterpret_cast<int*>(sm + 32);          // [4] arrivals of the set's warps that have stored their A rows
  uint32_t* tbase_s = reinterpret_cast<uint32_t*>(sm + 96);
  long long* goff = reinterpret_cast<long long*>(sm + 128);
  long long* ogoff = goff + kMaxParts;                                      // offsets of the CTA's output vector
  const float** gptr = reinterpret_cast<const float**>(ogoff + kMaxParts);  // g part base of this cell
  long long* gsm = reinterpret_cast<long long*>(gptr + kMaxParts);          // g row stride
  unsigned char* bt = sm + kHeaderBytes;
  float* acc = reinterpret_cast<float*>(bt + A.bt_bytes);
  unsigned char* ring = reinterpret_cast<unsigned char*>(acc + A.acc_floats);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one CTA per (cell, product): product 0 = P (gradient of x, needs the y tables), 1 = Q (gradient of y, x tables);
  // the two CTAs of a cell start next to each other, so the second read of a slab normally comes from L2
  const int product = blockIdx.x & 1;
  const long long cell = blockIdx.x >> 1;

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tbase_s)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x == 32) {
    for (int s = 0; s < 4; s++) {
      mbar_init(mdone + s, 1);
      ev[s] = 0;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  fill_offsets(goff, A.g, A.ng, A.cg, cell);
  if (product == 0)
    fill_offsets(ogoff, A.xg, A.nx, A.cg, cell);
  else
    fill_offsets(ogoff, A.yg, A.ny, A.cg, cell);
  {
    float4* z = reinterpret_cast<float4*>(bt);
    const int n16 = (A.bt_bytes + 4 * A.acc_floats) >> 4;
    for (int e = threadIdx.x; e < n16; e += blockDim.x) z[e] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();
  if (threadIdx.x < A.ng) {
    gptr[threadIdx.x] = A.g[threadIdx.x].base + goff[threadIdx.x] + 2LL * A.offs_extra;
    gsm[threadIdx.x] = A.g[threadIdx.x].sm;
  }
  if (product == 0)
    stage_tables(bt, A.y, A.ybt, A.yR, A.ny, A.cg, cell);
  else
    stage_tables(bt, A.x, A.xbt, A.xR, A.nx, A.cg, cell);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // tables are read by the tensor core (async proxy)
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tbase_s;

  {
    // ------------------------------------------------ one slab of every group of the warp's set
    const int s = warp >> 2, q = warp & 3;
    const uint32_t lanes = (uint32_t)(32 * q) << 16;
    // tensor-memory columns of set s: A operand of one K half (hi 32, lo 32) at 128 s, accumulators of the set's
    // even / odd groups at + 64 / + 96
    const uint32_t tA = tbase + 128 * s + lanes, tD = tA + 64;
    const uint32_t slot_u32 = smem_u32(ring) + warp * kSlabBytes;
    const uint32_t bt_u32 = smem_u32(bt), acc_u32 = smem_u32(acc);
    const int ngs = (A.ngroups - s + 3) >> 2;
    uint32_t par = 0;
    bool ok = true;
    // lane-constant parts of the swizzled slot addresses: row-per-lane reads (P) and column-per-lane reads (Q)
    const uint32_t xrd = slot_u32 + lane * 256, xsw = (lane & 15) << 4;
    const uint32_t yrd = slot_u32 + ((lane & 1) << 3), ysw = (lane >> 1) << 4;
    const int pf_hb = lane >> 4, pf_c = lane & 15;

    auto prefetch = [&](const Work& w) {  // the slab into the warp's ring slot, 16-byte chunks XOR-swizzled by row
      if (w.valid()) {
        const int n2tot = w.n2();
        const float* src = gptr[w.ri()] + (long long)(w.r.y >> 8) * gsm[w.ri()] + 2LL * w.r.z + (long long)pf_hb * 2 * n2tot + 4 * pf_c;
        const long long step = 4LL * n2tot;  // two rows, in floats
#pragma unroll
        for (int i = 0; i < 16; i++) {  // rows 2 i + pf_hb
          const int row = 2 * i + pf_hb;
          cp_async16(slot_u32 + row * 256 + ((pf_c ^ (row & 15)) << 4), src + i * step);
        }
      }
      cp_async_commit();
    };
    // 32 of the slab's 64 K values of this lane's operand row: P: row n1 = lane, columns (n2, re/im) 32 half ..;
    // Q: row n2 = lane, columns (n1, re/im) with n1 = 16 half ..
    auto read_half = [&](int half, float (&v)[32]) {
      if (product == 0) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float4 f = lds128(xrd + (((8 * half + i) << 4) ^ xsw));
          v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; i++) {
          const int n1 = 16 * half + i;
          const float2 f = lds64(yrd + n1 * 256 + (((n1 & 15) << 4) ^ ysw));
          v[2 * i] = f.x, v[2 * i + 1] = f.y;
        }
      }
    };
    auto store_half = [&](const float (&v)[32]) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float t[8];
#pragma unroll
        for (int i = 0; i < 8; i++) t[i] = v[8 * j + i];
        split_store8(tA, 8 * j, t);
      }
    };
    Work cur{}, next{};
    auto add_result = [&](int g) {  // the band of group g's accumulator to the gradient rows (record re-read from L1)
      Work w;
      load_work(A, g, q, lane, w);
      if (w.valid()) {
        const uint32_t tDg = tD + 32 * ((g >> 2) & 1);
        if (product == 0)
          epilogue<true>(tDg, acc_u32 + 4u * w.xacc(), w.n1(), w.a0() + lane, w.m(), w.l1(), w.l2(), w.cvec);
        else
          epilogue<false>(tDg, acc_u32 + 4u * w.yacc(), w.n2(), w.b0() + lane, w.m(), w.l1(), w.l2(), w.cvec);
      }
    };
    auto arrive_and_issue = [&](int k, int half) {
      tmem_wait_st();
      tc_fence_before();
      if (count_event(ev + s, 3)) {  // this warp completed the operand: the MMAs of the K half
        tc_fence_after();
        const uint32_t tDk = tD - lanes + 32 * (k & 1);
        if (product == 0)
          issue_half(tA - lanes, tDk, bt_u32 + cur.t.x, cur.t.y, half, half == 0);
        else
          issue_half(tA - lanes, tDk, bt_u32 + cur.t.z, cur.t.w, half, half == 0);
        mma_commit(mdone + s);
      }
    };

    if (ngs > 0) {
      load_work(A, s, q, lane, next);
      prefetch(next);
    }
    // Per group: first K half of the operand, MMAs; second half read meanwhile, slot refilled, stored when the first
    // MMAs have released the block, MMAs; the previous group's result is added while those run.
    for (int k = 0; k < ngs && ok; k++) {
      cur = next;
      if (k + 1 < ngs) load_work(A, s + 4 * (k + 1), q, lane, next);  // first used by the prefetch below
      float v[32];

      cp_async_wait_all();
      __syncwarp();
      if (cur.valid()) {
        read_half(0, v);
        store_half(v);
      }
      arrive_and_issue(k, 0);
      if (cur.valid()) read_half(1, v);
      __syncwarp();  // every lane has read the slot: refill it with the next slab
      if (k + 1 < ngs) prefetch(next);

      ok = mbar_wait(mdone + s, par);  // the first half's MMAs have consumed the block
      par ^= 1;
      if (!ok) break;
      tc_fence_after();
      if (cur.valid()) store_half(v);
      arrive_and_issue(k, 1);
      if (k > 0) add_result(s + 4 * (k - 1));  // its accumulator is not touched before group k + 1

      ok = mbar_wait(mdone + s, par);
      par ^= 1;
      if (!ok) break;
      tc_fence_after();
    }
    if (ok && ngs > 0) add_result(s + 4 * (ngs - 1));
    cp_async_wait_all();
    if (!ok && lane == 0) *A.status = 1;
  }

  tc_fence_before();
  __syncthreads();
  if (product == 0)
    flush_rows(acc, A.xg, ogoff, A.xacc, A.nx, A.x_atomic != 0);
  else
    flush_rows(acc, A.yg, ogoff, A.yacc, A.ny, A.y_atomic != 0);
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(512u) : "memory");
  }
}

}  // namespace

// ---- launcher --------------------------------------------------------------------------------------------------

namespace {

inline int round_up(int v, int q) { return (v + q - 1) / q * q; }

}  // namespace

// Returns -1 when the call does not qualify (the caller then takes the SIMT kernels).
int launch_cg_bwd_tc(const VecCall& c, cudaStream_t s) {
  static const char* fn = "SO3vec_addCGproduct_back";
  if (!c.vec_ok || !c.in_vec_ok || c.xg.empty() || c.yg.empty()) return -1;
  if (c.x.size() > 15 || c.y.size() > 15 || c.r.size() > 15) return -1;
  for (const auto& p : c.x) if (p.n % 32 || p.l > 7 || p.n > 32768) return -1;
  for (const auto& p : c.y) if (p.n % 32 || p.l > 7 || p.n > 32768) return -1;
  for (const auto& p : c.r) if (p.l > 127) return -1;
  if (!device_has_tcgen05()) return -1;
  int* status = async_status_word(kStatusBwdTc);
  if (!status) return -1;

  // Each CTA works on one product and holds only that product's tables and gradient rows: offsets of the y tables /
  // x gradient rows (P) and of the x tables / y gradient rows (Q) both start at 0.
  TcArgs a;
  int ybt = 0, xbt = 0, xacc = 0, yacc = 0;
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    a.yg[i] = c.yg[i];
    a.yR[i] = round_up(2 * (2 * c.y[i].l + 1), 8);
    a.ybt[i] = ybt;
    ybt += (c.y[i].n / 32) * 512 * a.yR[i];
    a.yacc[i] = yacc;
    yacc += 2 * (2 * c.y[i].l + 1) * c.y[i].n;
  }
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    a.xg[i] = c.xg[i];
    a.xR[i] = round_up(2 * (2 * c.x[i].l + 1), 8);
    a.xbt[i] = xbt;
    xbt += (c.x[i].n / 32) * 512 * a.xR[i];
    a.xacc[i] = xacc;
    xacc += 2 * (2 * c.x[i].l + 1) * c.x[i].n;
  }
  // + 512: an N = 32 read of a table with fewer rows runs into the next k-chunk: keep the last one in bounds
  const int bt = round_up(std::max(xbt, ybt) + 512, 128), acc = std::max(xacc, yacc);
  for (size_t i = 0; i < c.r.size(); i++) a.g[i] = c.r[i];
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.ng = (int)c.r.size();
  a.bt_bytes = bt;
  a.acc_floats = round_up(acc, 32);
  const size_t smem = (size_t)kHeaderBytes + bt + 4 * (size_t)a.acc_floats + (size_t)kSlots * kSlabBytes;
  if (smem > 227 * 1024 || 4 * (size_t)a.acc_floats > 0xffff * 4) return -1;

  std::vector<int> key = {9 /*family*/, (int)c.x.size(), (int)c.y.size(), (int)c.r.size()};
  for (const auto& p : c.x) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.y) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.r) key.push_back(p.l);
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  const int *xaccp = a.xacc, *yaccp = a.yacc, *xbtp = a.xbt, *ybtp = a.ybt, *xR = a.xR, *yR = a.yR;
  DevicePlan* plan = get_plan(key, [&](DevicePlan& p) {
    build_schedule(xs, ys, rs, false, true, &p.sched);
    // slabs keyed by (xi, yi, a0, b0): they share both B operands
    std::map<std::vector<int>, std::vector<int4>> buckets;
    for (const Triple& t : p.sched.triples) {
      int cpos = t.coff;
      for (int m = -t.l; m <= t.l; m++) {
        const int lo = std::max<int>(-t.l1, m - t.l2), hi = std::min<int>(t.l1, m + t.l2);
        for (int a0 = 0; a0 < xs[t.xi].n; a0 += 32)
          for (int b0 = 0; b0 < ys[t.yi].n; b0 += 32)
            buckets[{t.xi, t.yi, a0, b0}].push_back(
                make_int4(t.ri | (1 << 8), t.l | ((m + t.l) << 8), t.offs + a0 * ys[t.yi].n + b0, cpos));
        cpos += hi - lo + 1;
      }
    }
    for (const auto& kv : buckets) {
      const auto& v = kv.second;
      const int xi = kv.first[0], yi = kv.first[1], a0 = kv.first[2], b0 = kv.first[3];
      for (size_t i = 0; i < v.size(); i += 4) {
        const int ns = (int)std::min<size_t>(4, v.size() - i);
        p.h_items.push_back(make_int4(xi | (yi << 4) | (xs[xi].l << 8) | (ys[yi].l << 16), a0 | (b0 << 16),
                                      xs[xi].n | (ys[yi].n << 16), xaccp[xi] | (yaccp[yi] << 16)));
        p.h_items.push_back(make_int4(ybtp[yi] + (b0 >> 5) * 512 * yR[yi], yR[yi], xbtp[xi] + (a0 >> 5) * 512 * xR[xi], xR[xi]));
        for (int j = 0; j < 4; j++) p.h_items.push_back(j < ns ? v[i + j] : make_int4(0, 0, 0, 0));
        for (int j = 0; j < 4; j++) {  // the band coefficients of the slab's row, zero-padded to 16
          float c[16] = {0};
          if (j < ns) {
            const int l = v[i + j].y & 0xff, m = (v[i + j].y >> 8) - l;
            const int K = std::min(xs[xi].l, m + ys[yi].l) - std::max(-xs[xi].l, m - ys[yi].l) + 1;
            for (int e = 0; e < K; e++) c[e] = p.sched.coeffs[v[i + j].w + e];
          }
          for (int e = 0; e < 16; e += 4) {
            int4 w;
            memcpy(&w, c + e, 16);
            p.h_items.push_back(w);
          }
        }
      }
    }
  });
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->nitems == 0 || c.cg.ncells == 0) return GELIB_OK;
  if (c.cg.ncells > 0x3fffffffLL) return fail(GELIB_SKIPPED, fn, "number of cells exceeds 2^30-1");

  a.cg = c.cg;
  a.coeffs = plan->coeffs;
  a.groups = plan->items;
  a.ngroups = plan->nitems / kRec;
  a.offs_extra = c.offs_extra;
  a.x_atomic = c.xg_bcast ? 1 : 0;
  a.y_atomic = c.yg_bcast ? 1 : 0;
  a.status = status;  // unified addressing: the host pointer of mapped memory is valid on the device
  cudaError_t e = cudaFuncSetAttribute(cg_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) {
    cg_bwd_tc_kernel<<<(unsigned)(2 * c.cg.ncells), kThreads, smem, s>>>(a);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return check_cuda(e, fn, "tensor-core backward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
