// Forward Clebsch-Gordan product on the 5th-generation tensor cores (tcgen05 + tensor memory), for channel counts
// that are multiples of 32 and outputs that are overwritten.  Same mathematics as cg_fwd.cu; replaces the same
// reference code (cuda/SO3part_addCGproduct.cu:59-178 and the loop of Gvec::add_CGproduct, core/Gvec.hpp:311-321
// of GElib).
//
// Formulation.  A slab is one row m of one triple (l1,l2)->l restricted to a 32 x 32 channel tile of the output:
//     R[n1][(n2,c')] = sum_{(m2,c)} A[n1][(m2,c)] B[(m2,c)][(n2,c')],
//     A[n1][(m2,c)]  = C(m-m2, m2) x_c[m-m2][n1]     (zero outside the band |m-m2| <= l1),
//     B[(m2,re)]     = (y_r[m2][n2] | y_i[m2][n2]),   B[(m2,im)] = (-y_i | y_r)      for c' = (re | im),
// a real GEMM with K = 2(2 l2 + 1) rounded up to 8 and N = 64.  B depends on the y part and its channel tile only,
// so it is written to shared memory once per cell, split for 3xTF32, in the K-major core-matrix layout of the
// shared-memory descriptor.  Four slabs that share B are stacked to M = 128.  A warp builds the A rows of its slab in
// registers (lane = n1: a shuffle for the coefficient, one shared-memory load of x per band entry), splits them and
// stores them to tensor memory; the warp that completes the operand issues 3 x K/8 MMAs (a_lo b_hi + a_hi b_lo +
// a_hi b_hi, FP32 accumulators in tensor memory) and a tcgen05.commit; every warp then reads its 32 accumulator rows
// back and writes them out: a lane owns 256 contiguous bytes of the output row, the warp 8 KB.
// Four sets of four warps own 128 tensor-memory columns each (A hi 32, A lo 32, accumulator 64), so that up to 16
// slabs are in flight per SM; nothing large is ever read, and the output is written exactly once.
//
// Every wait on an mbarrier is bounded; on a timeout the kernel records it in a host-mapped status word, leaves its
// loop, frees its tensor memory and returns, and the next call reports the failure.
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

#include "plan.h"
#include "tc_common.h"
#include "tma_maps.h"

namespace gelib_b200 {

namespace {

using namespace tc;

constexpr int kWarps = 16;  // four sets of four slabs
constexpr int kThreads = 32 * kWarps;
constexpr int kHeaderBytes = 512;
constexpr int kRec = 22;  // int4 per group record
constexpr int kStagePitch = 272;  // bytes between the rows of a warp's output staging block (256 + 16)

struct FwdTcArgs {
  PartView x[kMaxParts], y[kMaxParts], r[kMaxParts];
  int xoff[kMaxParts];  // float offset of the staged rows of each x part
  int ybt[kMaxParts];   // byte offset of the B tables of each y part
  int yK[kMaxParts];    // K of each y part: 2(2l+1) rounded up to 8
  int nx, ny, nr;
  int bt_bytes, x_floats;
  CellGrid cg;
  // 22 int4 per group of up to four slabs that share the y part and its channel tile:
  //   {byte offset of the B table, K, unused, unused}
  //   unused
  //   4 x {ri | valid<<8 | l1<<16 | l2<<24, l | (m+l)<<8 | (first x row of the band)<<16,
  //        channel offset of the tile inside part ri, float offset of x[row 0][a0] | N2<<16}
  //   4 x 16 floats: the band coefficients of the slab's row, zero-padded
  const int4* groups;
  int ngroups;
  int offs_extra;
  int* status;
  int drop_commit;  // test hook: the MMAs are issued but never committed, so every wait of the kernel runs out
  // Output tiles leave through tensor maps (one per r part: every y part has the same channel count N2 then):
  // two tensor stores per slab from a swizzled staging block instead of one 256-byte bulk store per lane and row.
  int use_tma;
  unsigned tk[kMaxParts][6];  // (outer, inner) cell coordinate of the maps = (b, g0, g1) x these multipliers
};

// One tensor store: 32 rows x 128 bytes of a slab (rank-5 map; the box is 32 x 32 x 1 x 1 x 1 floats).
__device__ __forceinline__ void tma_store_5d(const void* map, uint32_t src, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
               : "memory");
}

struct Slab {
  int4 r;
  float cvec;
  __device__ __forceinline__ int ri() const { return r.x & 0xff; }
  __device__ __forceinline__ bool valid() const { return (r.x >> 8) & 1; }
  __device__ __forceinline__ int l1() const { return (r.x >> 16) & 0xff; }
  __device__ __forceinline__ int l2() const { return (r.x >> 24) & 0xff; }
  __device__ __forceinline__ int row() const { return (r.y >> 8) & 0xff; }  // m + l
  __device__ __forceinline__ int m() const { return ((r.y >> 8) & 0xff) - (r.y & 0xff); }
  __device__ __forceinline__ int n2tot() const { return (r.w >> 16) & 0xffff; }
  __device__ __forceinline__ int xfloat() const { return r.w & 0xffff; }
};

__device__ __noinline__ void fill_offsets(long long* dst, const PartView* parts, int nparts, const CellGrid& cg, long long cell) {
  for (int p = threadIdx.x; p < nparts; p += blockDim.x) dst[p] = cell_offset(parts[p], cg, cell);
}

// x rows of the cell, channel-dense: part i at xoff[i], row mi at + 2 n mi.
__device__ __noinline__ void stage_x(float* dst, const PartView* parts, const int* off, int nparts, const CellGrid& cg,
                                     long long cell) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = parts[i];
    const float* src = p.base + cell_offset(p, cg, cell);
    const int n2 = p.n >> 1, total = (2 * p.l + 1) * n2;  // float4 = two channels
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int mi = e / n2, c2 = e - mi * n2;
      *reinterpret_cast<float4*>(dst + off[i] + 2 * p.n * mi + 4 * c2) =
          __ldg(reinterpret_cast<const float4*>(src + (long long)mi * p.sm + 4 * c2));
    }
  }
}

// B tables of every (y part, 32-channel tile): a hi block and a lo block of [K/4 k-chunks][64 rows][4 floats].
// Row 2 n2 + c' (c' = re | im of the output), k = 2 mi + c:  re row (y_r, -y_i), im row (y_i, y_r).
__device__ __noinline__ void stage_ytables(unsigned char* bt, const PartView* parts, const int* off, const int* Ks,
                                           int nparts, const CellGrid& cg, long long cell) {
  for (int i = 0; i < nparts; i++) {
    const PartView& p = parts[i];
    const float* src = p.base + cell_offset(p, cg, cell);
    const int K = Ks[i], rows = 2 * p.l + 1, kc_n = K >> 2, T = p.n >> 5;
    // one thread per (tile, k-chunk = two rows mi, n2): reads two complex numbers, writes two 16-byte rows twice
    const int total = T * kc_n * 32;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int n2 = e & 31, kc = (e >> 5) % kc_n, t = (e >> 5) / kc_n;
      const int m0 = 2 * kc, m1 = 2 * kc + 1;
      float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
      if (m0 < rows) a = __ldg(reinterpret_cast<const float2*>(src + (long long)m0 * p.sm + 2 * (32 * t + n2)));
      if (m1 < rows) b = __ldg(reinterpret_cast<const float2*>(src + (long long)m1 * p.sm + 2 * (32 * t + n2)));
      const float re[4] = {a.x, -a.y, b.x, -b.y}, im[4] = {a.y, a.x, b.y, b.x};
      uint32_t rh[4], rl[4], ih[4], il[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        split_tf32(re[k], rh[k], rl[k]);
        split_tf32(im[k], ih[k], il[k]);
      }
      unsigned char* tile = bt + off[i] + t * (512 * K);
      uint4* hi = reinterpret_cast<uint4*>(tile + (kc * 64 + 2 * n2) * 16);
      uint4* lo = reinterpret_cast<uint4*>(tile + 256 * K + (kc * 64 + 2 * n2) * 16);
      hi[0] = make_uint4(rh[0], rh[1], rh[2], rh[3]);
      hi[1] = make_uint4(ih[0], ih[1], ih[2], ih[3]);
      lo[0] = make_uint4(rl[0], rl[1], rl[2], rl[3]);
      lo[1] = make_uint4(il[0], il[1], il[2], il[3]);
    }
  }
}

__device__ __forceinline__ void load_slab(const FwdTcArgs& A, int g, int q, int lane, Slab& w) {
  w.r = __ldg(&A.groups[kRec * g + 2 + q]);
  w.cvec = lane < 16 ? __ldg(reinterpret_cast<const float*>(&A.groups[kRec * g + 6 + 4 * q]) + lane) : 0.f;
}

// ---- the kernel ------------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads, 1) cg_fwd_tc_kernel(const __grid_constant__ FwdTcArgs A,
                                                                const __grid_constant__ TmaMaps M) {
  extern __shared__ __align__(1024) unsigned char sm[];
  uint64_t* mdone = reinterpret_cast<uint64_t*>(sm);  // [4] MMAs of a set's group complete (tcgen05.commit)
  int* ev = reinterpret_cast<int*>(sm + 32);          // [4] arrivals of the set's warps that have stored their A rows
  uint32_t* tbase_s = reinterpret_cast<uint32_t*>(sm + 48);
  long long* roff = reinterpret_cast<long long*>(sm + 64);                   // scratch: output offsets of the cell
  float** rptr = reinterpret_cast<float**>(roff + kMaxParts);                // output part base of this cell
  long long* rsm = reinterpret_cast<long long*>(rptr + kMaxParts);           // output row stride
  unsigned char* bt = sm + kHeaderBytes;
  float* xs = reinterpret_cast<float*>(bt + A.bt_bytes);
  // per warp 32 rows of kStagePitch, or (tensor stores) two swizzled half-slabs of 4096 bytes; the block starts at a
  // multiple of 1024 bytes of the shared-memory ADDRESS (the swizzle pattern is a function of the address)
  const uint32_t stage_base = (smem_u32(sm) + kHeaderBytes + A.bt_bytes + 4 * A.x_floats + 1023u) & ~1023u;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long cell = blockIdx.x;

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
  fill_offsets(roff, A.r, A.nr, A.cg, cell);
  stage_x(xs, A.x, A.xoff, A.nx, A.cg, cell);
  stage_ytables(bt, A.y, A.ybt, A.yK, A.ny, A.cg, cell);
  __syncthreads();
  if (threadIdx.x < A.nr) {
    rptr[threadIdx.x] = A.r[threadIdx.x].base + roff[threadIdx.x] + 2LL * A.offs_extra;
    rsm[threadIdx.x] = A.r[threadIdx.x].sm;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // tables are read by the tensor core (async proxy)
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tbase_s;

  {
    const int s = warp >> 2, q = warp & 3;
    const uint32_t lanes = (uint32_t)(32 * q) << 16;
    // tensor-memory columns of set s: A hi 32, A lo 32, accumulator 64
    const uint32_t tA = tbase + 128 * s + lanes, tD = tA + 64;
    const uint32_t bt_u32 = smem_u32(bt), xs_u32 = smem_u32(xs) + 8 * lane;
    const uint32_t stage_u32 = stage_base + warp * (A.use_tma ? 8192 : 32 * kStagePitch);
    // cell coordinates of the tensor maps
    const unsigned cg1 = (unsigned)cell % (unsigned)A.cg.G1, ct = (unsigned)cell / (unsigned)A.cg.G1;
    const unsigned cg0 = ct % (unsigned)A.cg.G0, cb = ct / (unsigned)A.cg.G0;
    const int ngs = (A.ngroups - s + 3) >> 2;
    uint32_t par = 0;
    bool ok = true;

    Slab cur{}, next{};
    int4 hd = make_int4(0, 0, 0, 0), hd_next = make_int4(0, 0, 0, 0);
    if (ngs > 0) {
      load_slab(A, s, q, lane, next);
      hd_next = __ldg(&A.groups[kRec * s]);
    }
    for (int k = 0; k < ngs && ok; k++) {
      cur = next;
      hd = hd_next;  // {B table offset, K}
      if (k + 1 < ngs) {
        load_slab(A, s + 4 * (k + 1), q, lane, next);
        hd_next = __ldg(&A.groups[kRec * (s + 4 * (k + 1))]);
      }
      const int K = hd.y;

      // 1. A rows of the slab: lane = n1, column 2 idx + c = C(m1, m2) x_c[m1][n1] with m2 = idx - l2, m1 = m - m2
      if (cur.valid()) {
        const int l1 = cur.l1(), l2 = cur.l2(), m = cur.m();
        const int lo = max(-l1, m - l2), hi = min(l1, m + l2);
        const int n1f = 2 * ((cur.r.y >> 16) & 0xffff);  // floats per x row
        // x[m1][a0 + lane] for m1 = m + l2 - idx: float offset x0 - idx * n1f
        const uint32_t x0 = xs_u32 + 4u * (uint32_t)(cur.xfloat() + (m + l2 + l1) * n1f);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          if (8 * j < K) {
            uint32_t vh[8], vl[8];
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const int idx = 4 * j + i;
              const int m1 = m + l2 - idx;
              float2 v = make_float2(0.f, 0.f);
              if (m1 >= lo && m1 <= hi) {
                const float c = __shfl_sync(0xffffffffu, cur.cvec, m1 - lo);
                const float2 xv = lds64(x0 - 4u * (uint32_t)(idx * n1f));
                v = make_float2(c * xv.x, c * xv.y);
              }
              split_tf32(v.x, vh[2 * i], vl[2 * i]);
              split_tf32(v.y, vh[2 * i + 1], vl[2 * i + 1]);
            }
            tmem_st8(tA + 8 * j, vh);
            tmem_st8(tA + 32 + 8 * j, vl);
          }
        }
      }
      tmem_wait_st();
      tc_fence_before();
      if (count_event(ev + s, 3)) {
        // this warp completed the operand: the MMAs of the group, smallest terms first
        tc_fence_after();
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
        const uint64_t fixed = (64ull << 16) | (8ull << 32) | (1ull << 46);  // k-chunk stride 1024 B, 8-row group 128 B
        const uint32_t table = bt_u32 + hd.x;
        const uint64_t dhi = fixed | ((table >> 4) & 0x3fffu), dlo = fixed | (((table + 256u * K) >> 4) & 0x3fffu);
        const uint32_t tAs = tA - lanes, tDs = tD - lanes;
        const int ksteps = K >> 3;
#pragma unroll 1
        for (int term = 0; term < 3; term++) {
          const uint32_t a = term == 0 ? tAs + 32 : tAs;
          const uint64_t b = term == 1 ? dlo : dhi;
#pragma unroll 1
          for (int ks = 0; ks < ksteps; ks++) mma_tf32_ts(tDs, a + 8 * ks, b + 128ull * ks, idesc, (term | ks) != 0);
        }
        if (!A.drop_commit) mma_commit(mdone + s);
      }

      // 2. the accumulator rows of the slab: 256 contiguous bytes of the output per lane
      ok = mbar_wait(mdone + s, par);
      par ^= 1;
      if (!ok) break;
      tc_fence_after();
      if (cur.valid()) {
        // Each lane puts its 256-byte output row into the warp's staging block (272-byte pitch: conflict-free) and
        // hands it to the bulk-copy engine: the store stream runs on its own, off the warp's critical path.
        if (A.use_tma) {
          // Lane = output row n1: its 16-byte chunk c of half hlf goes to chunk c ^ (n1 & 7) of row n1 of that half
          // (the 128-byte swizzle of the tensor map: conflict-free here, undone by the copy engine); lane 0 then
          // hands the two half-slabs to the copy engine with one tensor store each.
          if (lane == 0) bulk_wait_read();  // the previous slab has left the staging block (lane 0 issued its stores)
          __syncwarp();
#pragma unroll
          for (int hlf = 0; hlf < 2; hlf++) {
            uint32_t d[32];
            tmem_ld32(tD + 32 * hlf, d);
#pragma unroll
            for (int i = 0; i < 8; i++)
              sts128(stage_u32 + 4096 * hlf + lane * 128 + ((i ^ (lane & 7)) << 4), d[4 * i], d[4 * i + 1], d[4 * i + 2], d[4 * i + 3]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the rows are read by the async proxy
          __syncwarp();
          if (lane == 0) {
            const int ri = cur.ri(), n2t = cur.n2tot();
            const int c1 = cur.r.z / n2t, col = 2 * (cur.r.z - c1 * n2t);
            const int ca = (int)(cb * A.tk[ri][0] + cg0 * A.tk[ri][1] + cg1 * A.tk[ri][2]);
            const int cc = (int)(cb * A.tk[ri][3] + cg0 * A.tk[ri][4] + cg1 * A.tk[ri][5]);
            tma_store_5d(&M.m[ri], stage_u32, col, c1, cur.row(), cc, ca);
            tma_store_5d(&M.m[ri], stage_u32 + 4096, col + 32, c1, cur.row(), cc, ca);
            bulk_commit();
          }
        } else {
          bulk_wait_read();  // the previous slab's rows have left the staging block
#pragma unroll
          for (int hlf = 0; hlf < 2; hlf++) {
            uint32_t d[32];
            tmem_ld32(tD + 32 * hlf, d);
#pragma unroll
            for (int i = 0; i < 8; i++)
              sts128(stage_u32 + lane * kStagePitch + 128 * hlf + 16 * i, d[4 * i], d[4 * i + 1], d[4 * i + 2], d[4 * i + 3]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the rows are read by the async proxy
          float* dst = rptr[cur.ri()] + (long long)cur.row() * rsm[cur.ri()] + 2LL * cur.r.z + 2LL * lane * cur.n2tot();
          bulk_store(dst, stage_u32 + lane * kStagePitch, 256);
          bulk_commit();
        }
      }
      tc_fence_before();  // the reads of the accumulator precede the next group's arrival
    }
    bulk_wait_all();
    if (!ok && lane == 0) *A.status = 1;
  }

  tc_fence_before();
  __syncthreads();
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

// Returns -1 when the call does not qualify or has fewer than min_slabs slabs per cell (the caller then takes the
// SIMT kernel).
int launch_cg_fwd_tc(const VecCall& c, cudaStream_t s, int min_slabs) {
  static const char* fn = "SO3vec_addCGproduct";
  if (!c.vec_ok || !c.in_vec_ok || !(c.flags & GELIB_OVERWRITE) || c.r_bcast) return -1;
  if (c.x.size() > 15 || c.y.size() > 15 || c.r.size() > 15) return -1;
  for (const auto& p : c.x) if (p.n % 32 || p.l > 7 || p.n > 32768) return -1;
  for (const auto& p : c.y) if (p.n % 32 || p.l > 7 || p.n > 32768) return -1;
  for (const auto& p : c.r) if (p.l > 127) return -1;
  if (min_slabs > 0) {  // cheap count of the slabs per cell before any set-up: small calls leave here
    long long slabs = 0;
    for (const auto& px : c.x)
      for (const auto& py : c.y)
        for (const auto& pr : c.r)
          if (pr.l >= std::abs(px.l - py.l) && pr.l <= px.l + py.l) slabs += (long long)(2 * pr.l + 1) * (px.n / 32) * (py.n / 32);
    if (slabs < min_slabs) return -1;
  }
  if (!device_has_tcgen05()) return -1;
  int* status = async_status_word(kStatusFwdTc);
  if (!status) return -1;

  FwdTcArgs a;
  int bt = 0, xf = 0;
  for (size_t i = 0; i < c.y.size(); i++) {
    a.y[i] = c.y[i];
    a.yK[i] = round_up(2 * (2 * c.y[i].l + 1), 8);
    a.ybt[i] = bt;
    bt += (c.y[i].n / 32) * 512 * a.yK[i];
  }
  for (size_t i = 0; i < c.x.size(); i++) {
    a.x[i] = c.x[i];
    a.xoff[i] = xf;
    xf += 2 * (2 * c.x[i].l + 1) * c.x[i].n;
  }
  if (xf > 0xffff) return -1;  // x offsets travel in 16 bits of the records
  for (size_t i = 0; i < c.r.size(); i++) a.r[i] = c.r[i];
  a.nx = (int)c.x.size();
  a.ny = (int)c.y.size();
  a.nr = (int)c.r.size();
  a.bt_bytes = round_up(bt, 128);
  a.x_floats = round_up(xf, 32);
  const size_t front = ((size_t)kHeaderBytes + a.bt_bytes + 4 * (size_t)a.x_floats + 1023) & ~(size_t)1023;
  if (front + 1024 + (size_t)kWarps * 32 * kStagePitch > 227 * 1024) return -1;

  std::vector<int> key = {8 /*family*/, (int)c.x.size(), (int)c.y.size(), (int)c.r.size()};
  for (const auto& p : c.x) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.y) { key.push_back(p.l); key.push_back(p.n); }
  for (const auto& p : c.r) key.push_back(p.l);
  const auto xs = sig_of(c.x), ys = sig_of(c.y), rs = sig_of(c.r);
  const int *xoff = a.xoff, *ybt = a.ybt, *yK = a.yK;
  DevicePlan* plan = get_plan(key, [&](DevicePlan& p) {
    build_schedule(xs, ys, rs, false, true, &p.sched);
    struct S { int4 r; int cidx, K; };
    std::map<std::vector<int>, std::vector<S>> buckets;  // slabs keyed by (yi, b0): they share the B table
    for (const Triple& t : p.sched.triples) {
      int cpos = t.coff;
      for (int m = -t.l; m <= t.l; m++) {
        const int lo = std::max<int>(-t.l1, m - t.l2), hi = std::min<int>(t.l1, m + t.l2);
        for (int a0 = 0; a0 < xs[t.xi].n; a0 += 32)
          for (int b0 = 0; b0 < ys[t.yi].n; b0 += 32)
            buckets[{t.yi, b0}].push_back(
                {make_int4(t.ri | (1 << 8) | (t.l1 << 16) | (t.l2 << 24), t.l | ((m + t.l) << 8) | (xs[t.xi].n << 16),
                           t.offs + a0 * ys[t.yi].n + b0, (xoff[t.xi] + 2 * a0) | (ys[t.yi].n << 16)),
                 cpos, hi - lo + 1});
        cpos += hi - lo + 1;
      }
    }
    for (const auto& kv : buckets) {
      const auto& v = kv.second;
      const int yi = kv.first[0], b0 = kv.first[1];
      for (size_t i = 0; i < v.size(); i += 4) {
        const int ns = (int)std::min<size_t>(4, v.size() - i);
        p.h_items.push_back(make_int4(ybt[yi] + (b0 >> 5) * 512 * yK[yi], yK[yi], 0, 0));
        p.h_items.push_back(make_int4(0, 0, 0, 0));
        for (int j = 0; j < 4; j++) p.h_items.push_back(j < ns ? v[i + j].r : make_int4(0, 0, 0, 0));
        for (int j = 0; j < 4; j++) {
          float cf[16] = {0};
          if (j < ns)
            for (int e = 0; e < v[i + j].K; e++) cf[e] = p.sched.coeffs[v[i + j].cidx + e];
          for (int e = 0; e < 16; e += 4) {
            int4 w;
            memcpy(&w, cf + e, 16);
            p.h_items.push_back(w);
          }
        }
      }
    }
  });
  if (!plan) return GELIB_CUDA_ERROR;
  if (plan->nitems == 0 || c.cg.ncells == 0) return GELIB_OK;
  if (c.cg.ncells > 0x7fffffffLL) return fail(GELIB_SKIPPED, fn, "number of cells exceeds 2^31-1");

  a.cg = c.cg;
  a.groups = plan->items;
  a.ngroups = plan->nitems / kRec;
  a.offs_extra = c.offs_extra;
  // option "inject_timeout" (tests only): exercise the bounded waits and the status word without any fault
  a.drop_commit = inject_timeout();
  a.status = status;  // unified addressing: the host pointer of mapped memory is valid on the device
  // tensor stores when every y part has the same channel count (the rows of an r part are then a matrix with rows of
  // N2 channels in which every tile is 32 consecutive rows) and the views fit rank-5 maps
  TmaMaps maps;
  memset(&maps, 0, sizeof(maps));
  a.use_tma = 0;
  if (pair_tma() && c.offs_extra == 0) {
    bool uniform = true;
    for (const auto& p : c.y) uniform = uniform && p.n == c.y[0].n;
    if (uniform) {
      std::vector<int> info;
      for (size_t i = 0; i < c.r.size(); i++) {
        info.push_back((int)i);
        info.push_back(c.y[0].n);
        info.push_back((c.r[i].n + c.y[0].n - 1) / c.y[0].n);
      }
      if (encode_part_maps(c.r, c.cg, 0, (int)c.r.size(), info.data(), a.tk, maps)) a.use_tma = 1;
    }
  }
  const size_t smem = front + 1024 + (size_t)kWarps * (a.use_tma ? 8192 : 32 * kStagePitch);
  cudaError_t e = cudaFuncSetAttribute(cg_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) {
    cg_fwd_tc_kernel<<<(unsigned)c.cg.ncells, kThreads, smem, s>>>(a, maps);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return check_cuda(e, fn, "tensor-core forward kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
