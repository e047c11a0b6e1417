// Channel mixing of an SO3part by a complex weight matrix, and its two gradients:
//
//   mode 0   r[row][j]  = sum_i x[row][i] W[i][j]              (the product  part * W)
//   mode 1   r[row][i]  = sum_j x[row][j] conj(W[i][j])        (gradient of the part: g * W^H)
//   back_w   Wg[i][j]  += sum_row conj(x[row][i]) g[row][j]    (gradient of the weights: x^H * g)
//
// rows = every (cell, m) of the part; all arrays dense complex64.  In GElib this is torch.matmul per part
// (python/src/gelib/SO3vec.py:174-177, python/src/gelib/SO3weights.py:22-85); with 16 channels the library GEMM runs at
// a tenth of the memory rate, and the mixing of config 5's pipeline cost as much as a fifth of its product.  The
// kernels here are bound by memory: a block stages tiles of rows (and the matrix) in shared memory with coalesced
// asynchronous copies, one tile in flight while the other is worked on, and every thread forms one output element per pass; the weight gradient keeps one (i,j) sum per thread over
// the block's rows and adds it to global memory once.
#include <cuda_pipeline.h>

#include <algorithm>

#include "plan.h"

namespace gelib_b200 {

namespace {

constexpr int kMixMaxN = 64;   // channels on either side
constexpr int kTileRows = 64;  // rows per block and pass

// `count` complex numbers from global to shared memory, asynchronously (8 bytes per copy; the caller commits).
__device__ __forceinline__ void tile_copy_async(float2* dst, const float2* src, int count) {
  for (int e = threadIdx.x; e < count; e += blockDim.x) __pipeline_memcpy_async(dst + e, src + e, 8);
}

template <int MODE>
__global__ void __launch_bounds__(256) mix_kernel(float2* __restrict__ r, const float2* __restrict__ x, const float2* __restrict__ W,
                                                  long long rows, int nk, int nj, int w_cols) {
  extern __shared__ float2 sm[];
  float2* Ms = sm;                 // [nk][nj + 1]: the matrix the rows are multiplied by
  float2* xs = sm + nk * (nj + 1); // [kTileRows][nk]
  for (int e = threadIdx.x; e < nk * nj; e += blockDim.x) {
    const int k = e / nj, j = e - k * nj;
    float2 w;
    if (MODE == 0) {
      w = W[k * w_cols + j];       // W[i = k][j]
    } else {
      w = W[j * w_cols + k];       // conj(W[i = j][j' = k])
      w.y = -w.y;
    }
    Ms[k * (nj + 1) + j] = w;
  }
  for (long long row0 = (long long)blockIdx.x * kTileRows; row0 < rows; row0 += (long long)gridDim.x * kTileRows) {
    const int nr = (int)min((long long)kTileRows, rows - row0);
    __syncthreads();
    for (int e = threadIdx.x; e < nr * nk; e += blockDim.x) xs[e] = __ldcs(x + row0 * nk + e);
    __syncthreads();
    for (int e = threadIdx.x; e < nr * nj; e += blockDim.x) {
      const int row = e / nj, j = e - row * nj;
      const float2* xr = xs + row * nk;
      float sr = 0.f, si = 0.f;
#pragma unroll 4
      for (int k = 0; k < nk; k++) {
        const float2 a = xr[k], b = Ms[k * (nj + 1) + j];
        sr = fmaf(a.x, b.x, sr); sr = fmaf(-a.y, b.y, sr);
        si = fmaf(a.x, b.y, si); si = fmaf(a.y, b.x, si);
      }
      __stcs(r + row0 * nj + e, make_float2(sr, si));
    }
  }
}

// The same product for power-of-two channel counts up to 32 on both sides: the thread keeps its column of the matrix
// in registers and walks the rows of the tile with 16-byte loads of x (two complex numbers per load).
template <int MODE, int NK>
__global__ void __launch_bounds__(256) mix_reg_kernel(float2* __restrict__ r, const float2* __restrict__ x,
                                                      const float2* __restrict__ W, long long rows, int nj, int w_cols) {
  extern __shared__ float2 sm[];  // two tiles [kTileRows][NK]: one is loaded while the other is worked on
  const int j = threadIdx.x % nj, rg = threadIdx.x / nj, nrg = blockDim.x / nj;
  float2 wc[NK];
#pragma unroll
  for (int k = 0; k < NK; k++) {
    if (MODE == 0) {
      wc[k] = W[k * w_cols + j];
    } else {
      wc[k] = W[j * w_cols + k];
      wc[k].y = -wc[k].y;
    }
  }
  const long long stride = (long long)gridDim.x * kTileRows;
  long long row0 = (long long)blockIdx.x * kTileRows;
  if (row0 < rows) tile_copy_async(sm, x + row0 * NK, (int)min((long long)kTileRows, rows - row0) * NK);
  __pipeline_commit();
  for (int buf = 0; row0 < rows; row0 += stride, buf ^= 1) {
    const int nr = (int)min((long long)kTileRows, rows - row0);
    const long long next = row0 + stride;
    if (next < rows) tile_copy_async(sm + (buf ^ 1) * kTileRows * NK, x + next * NK, (int)min((long long)kTileRows, rows - next) * NK);
    __pipeline_commit();
    __pipeline_wait_prior(1);
    __syncthreads();
    const float2* xs = sm + buf * kTileRows * NK;
    for (int row = rg; row < nr; row += nrg) {
      const float4* xr = reinterpret_cast<const float4*>(xs + row * NK);
      float sr = 0.f, si = 0.f, tr = 0.f, ti = 0.f;
#pragma unroll
      for (int k = 0; k < NK / 2; k++) {
        const float4 a = xr[k];
        sr = fmaf(a.x, wc[2 * k].x, sr); sr = fmaf(-a.y, wc[2 * k].y, sr);
        si = fmaf(a.x, wc[2 * k].y, si); si = fmaf(a.y, wc[2 * k].x, si);
        tr = fmaf(a.z, wc[2 * k + 1].x, tr); tr = fmaf(-a.w, wc[2 * k + 1].y, tr);
        ti = fmaf(a.z, wc[2 * k + 1].y, ti); ti = fmaf(a.w, wc[2 * k + 1].x, ti);
      }
      __stcs(r + (row0 + row) * nj + j, make_float2(sr + tr, si + ti));
    }
    __syncthreads();  // the tile may be overwritten by the copy after next
  }
}

__global__ void __launch_bounds__(256) mix_back_w_kernel(float* __restrict__ Wg, const float2* __restrict__ x,
                                                         const float2* __restrict__ g, long long rows, int ni, int nj,
                                                         long long rows_per_block) {
  extern __shared__ float2 sm[];      // two pairs of tiles [kTileRows][ni], [kTileRows][nj]
  const int tile = kTileRows * (ni + nj);
  const long long begin = (long long)blockIdx.x * rows_per_block, end = min(rows, begin + rows_per_block);
  constexpr int kPairs = (kMixMaxN * kMixMaxN + 255) / 256;  // (i,j) sums per thread
  float accr[kPairs], acci[kPairs];
#pragma unroll
  for (int p = 0; p < kPairs; p++) accr[p] = acci[p] = 0.f;
  const int npairs = ni * nj;
  auto copy_tile = [&](int buf, long long row0) {
    const int nr = (int)min((long long)kTileRows, end - row0);
    tile_copy_async(sm + buf * tile, x + row0 * ni, nr * ni);
    tile_copy_async(sm + buf * tile + kTileRows * ni, g + row0 * nj, nr * nj);
  };
  if (begin < end) copy_tile(0, begin);
  __pipeline_commit();
  int buf = 0;
  for (long long row0 = begin; row0 < end; row0 += kTileRows, buf ^= 1) {
    const int nr = (int)min((long long)kTileRows, end - row0);
    if (row0 + kTileRows < end) copy_tile(buf ^ 1, row0 + kTileRows);
    __pipeline_commit();
    __pipeline_wait_prior(1);
    __syncthreads();
    const float2* xs = sm + buf * tile;
    const float2* gs = xs + kTileRows * ni;
#pragma unroll
    for (int p = 0; p < kPairs; p++) {
      const int pair = threadIdx.x + 256 * p;
      if (pair < npairs) {
        const int i = pair / nj, j = pair - i * nj;
        float sr = accr[p], si = acci[p];
        const float2* xa = xs + i;
        const float2* gb = gs + j;
#pragma unroll 8
        for (int row = 0; row < nr; row++) {  // conj(x) g
          const float2 a = xa[row * ni], b = gb[row * nj];
          sr = fmaf(a.x, b.x, sr); sr = fmaf(a.y, b.y, sr);
          si = fmaf(a.x, b.y, si); si = fmaf(-a.y, b.x, si);
        }
        accr[p] = sr;
        acci[p] = si;
      }
    }
    __syncthreads();  // the tiles may be overwritten by the copy after next
  }
#pragma unroll
  for (int p = 0; p < kPairs; p++) {
    const int pair = threadIdx.x + 256 * p;
    if (pair < npairs) {
      atomicAdd(Wg + 2 * pair, accr[p]);
      atomicAdd(Wg + 2 * pair + 1, acci[p]);
    }
  }
}

}  // namespace

int launch_mix(float* r, const float* x, const float* W, long long rows, int n_in, int n_out, int mode, cudaStream_t s) {
  static const char* fn = "SO3part_mix";
  if (n_in < 1 || n_out < 1 || n_in > kMixMaxN || n_out > kMixMaxN) return fail(GELIB_SKIPPED, fn, "more than 64 channels");
  if (rows <= 0) return GELIB_OK;
  const int nk = mode == 0 ? n_in : n_out, nj = mode == 0 ? n_out : n_in;  // contraction length, output channels
  const size_t smem = ((size_t)nk * (nj + 1) + (size_t)kTileRows * nk) * sizeof(float2);
  const unsigned blocks = (unsigned)std::min<long long>((rows + kTileRows - 1) / kTileRows, 148LL * 16);
  cudaError_t e;
  const bool pow2 = (nj & (nj - 1)) == 0 && nj <= 32;
  if (pow2 && (nk == 16 || nk == 32)) {
    const size_t smem_r = (size_t)2 * kTileRows * nk * sizeof(float2);
    float2* rp = reinterpret_cast<float2*>(r);
    const float2 *xp = reinterpret_cast<const float2*>(x), *wp = reinterpret_cast<const float2*>(W);
    if (mode == 0 && nk == 16) mix_reg_kernel<0, 16><<<blocks, 256, smem_r, s>>>(rp, xp, wp, rows, nj, n_out);
    else if (mode == 0) mix_reg_kernel<0, 32><<<blocks, 256, smem_r, s>>>(rp, xp, wp, rows, nj, n_out);
    else if (nk == 16) mix_reg_kernel<1, 16><<<blocks, 256, smem_r, s>>>(rp, xp, wp, rows, nj, n_out);
    else mix_reg_kernel<1, 32><<<blocks, 256, smem_r, s>>>(rp, xp, wp, rows, nj, n_out);
    e = cudaSuccess;
  } else if (mode == 0) {
    e = cudaFuncSetAttribute(mix_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      mix_kernel<0><<<blocks, 256, smem, s>>>(reinterpret_cast<float2*>(r), reinterpret_cast<const float2*>(x),
                                              reinterpret_cast<const float2*>(W), rows, nk, nj, n_out);
  } else {
    e = cudaFuncSetAttribute(mix_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      mix_kernel<1><<<blocks, 256, smem, s>>>(reinterpret_cast<float2*>(r), reinterpret_cast<const float2*>(x),
                                              reinterpret_cast<const float2*>(W), rows, nk, nj, n_out);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "mixing kernel launch");
  count_launch();
  return GELIB_OK;
}

int launch_mix_back_w(float* Wg, const float* x, const float* g, long long rows, int n_in, int n_out, cudaStream_t s) {
  static const char* fn = "SO3part_mix_back_w";
  if (n_in < 1 || n_out < 1 || n_in > kMixMaxN || n_out > kMixMaxN) return fail(GELIB_SKIPPED, fn, "more than 64 channels");
  if (rows <= 0) return GELIB_OK;
  const long long want_blocks = std::min<long long>((rows + kTileRows - 1) / kTileRows, 148LL * 8);
  long long rpb = (rows + want_blocks - 1) / want_blocks;
  rpb = (rpb + kTileRows - 1) / kTileRows * kTileRows;
  const unsigned blocks = (unsigned)((rows + rpb - 1) / rpb);
  const size_t smem = (size_t)2 * kTileRows * (n_in + n_out) * sizeof(float2);
  cudaError_t e = cudaFuncSetAttribute(mix_back_w_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess)
    mix_back_w_kernel<<<blocks, 256, smem, s>>>(Wg, reinterpret_cast<const float2*>(x), reinterpret_cast<const float2*>(g), rows,
                                                n_in, n_out, rpb);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return check_cuda(e, fn, "weight gradient kernel launch");
  count_launch();
  return GELIB_OK;
}

}  // namespace gelib_b200
