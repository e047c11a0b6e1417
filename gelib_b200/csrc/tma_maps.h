// Tensor maps (cuTensorMapEncodeTiled) for the 32 x 32 channel tiles of the parts of an SO3vec, shared by the kernels
// that move such tiles with cp.async.bulk.tensor (the pair backward loads them, the tensor-core forward stores them).
#pragma once
#include <cuda.h>

#include <array>
#include <vector>

#include "plan.h"

namespace gelib_b200 {

constexpr int kMaxMaps = 16;  // tensor maps per call: one per (part, N2)

struct TmaMaps {
  CUtensorMap m[kMaxMaps];
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// The tensor maps of one call: for every slot (part ri, N2, rows) a rank-5 view
//   {2*N2 floats of a row of N2 channels, rows of N2 channels, m rows, inner cell dimension, outer cell dimension}
// of the part, box 32 floats x 32 rows, 128-byte swizzle.  The cells (b, g0, g1) of the part become at most two
// dimensions (extent-1 and broadcast dimensions drop out, neighbours that are contiguous merge); tk[ri] receives the
// multipliers that turn (b, g0, g1) into the outer and the inner coordinate.  False when the views cannot be described
// that way (strides not multiples of 16 bytes, three independent cell dimensions, ...).
inline bool encode_part_maps(const std::vector<PartView>& parts, const CellGrid& cg, int offs_extra, int nslots,
                             const int* slot_info /* nslots x {ri, N2, rows} */, unsigned (*tk)[6], TmaMaps& maps) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc || nslots > kMaxMaps) return false;
  struct Dim {
    unsigned long long ext;
    long long stride;  // floats
    unsigned k[3];
  };
  std::vector<std::array<Dim, 2>> cell_dims(parts.size());
  for (size_t ri = 0; ri < parts.size(); ri++) {
    const PartView& p = parts[ri];
    std::vector<Dim> L;
    const long long ext[3] = {cg.B, cg.G0, cg.G1}, str[3] = {p.sb, p.sg0, p.sg1};
    for (int i = 0; i < 3; i++) {
      if (ext[i] <= 1 || str[i] == 0) continue;
      if (str[i] < 0) return false;
      Dim d = {(unsigned long long)ext[i], str[i], {0, 0, 0}};
      d.k[i] = 1;
      L.push_back(d);
    }
    while (L.size() > 2) {  // merge an outer dimension with its inner neighbour when they are contiguous
      bool merged = false;
      for (size_t i = 0; i + 1 < L.size() && !merged; i++) {
        if (L[i].stride == (long long)L[i + 1].ext * L[i + 1].stride) {
          Dim d = L[i + 1];
          for (int j = 0; j < 3; j++) d.k[j] = L[i].k[j] * (unsigned)L[i + 1].ext + L[i + 1].k[j];
          d.ext = L[i].ext * L[i + 1].ext;
          L[i] = d;
          L.erase(L.begin() + i + 1);
          merged = true;
        }
      }
      if (!merged) return false;
    }
    const Dim none = {1, 0, {0, 0, 0}};
    cell_dims[ri][0] = L.size() == 2 ? L[0] : none;             // outer
    cell_dims[ri][1] = L.empty() ? none : L.back();             // inner
    for (int j = 0; j < 3; j++) {
      tk[ri][j] = cell_dims[ri][0].k[j];
      tk[ri][3 + j] = cell_dims[ri][1].k[j];
    }
  }
  for (int sl = 0; sl < nslots; sl++) {
    const int ri = slot_info[3 * sl], n2 = slot_info[3 * sl + 1], rows = slot_info[3 * sl + 2];
    const PartView& p = parts[ri];
    float* base = p.base + 2LL * offs_extra;
    if (reinterpret_cast<uintptr_t>(base) % 16) return false;
    cuuint64_t dims[5] = {(cuuint64_t)2 * n2, (cuuint64_t)rows, (cuuint64_t)(2 * p.l + 1), cell_dims[ri][1].ext, cell_dims[ri][0].ext};
    long long str[4] = {(long long)n2 * 8, p.sm * 4, cell_dims[ri][1].stride * 4, cell_dims[ri][0].stride * 4};
    cuuint64_t strides[4];
    for (int i = 0; i < 4; i++) {
      if (dims[i + 1] == 1) str[i] = i == 0 ? 16 : (long long)strides[i - 1] * (long long)dims[i];  // never used: any valid value
      if (str[i] <= 0 || str[i] % 16 || str[i] >= (1LL << 40)) return false;
      strides[i] = (cuuint64_t)str[i];
    }
    for (int i = 0; i < 5; i++)
      if (dims[i] == 0 || dims[i] > 0xffffffffULL) return false;
    const cuuint32_t box[5] = {32, 32, 1, 1, 1}, one[5] = {1, 1, 1, 1, 1};
    if (enc(&maps.m[sl], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, base, dims, strides, box, one, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  return true;
}

}  // namespace gelib_b200
