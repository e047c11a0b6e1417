// Measures the FP32 multiply-add rate of the current device: the second roof of the Clebsch-Gordan kernels (the first
// is HBM bandwidth).  The reference publishes no such figure; its benchmark counts 4 flops per band term on the CPU
// (benchmarking/benchmark_CGproduct.cpp:31-37,70).  Every thread runs 16 independent chains of dependent FFMAs, enough
// warps are resident to cover the pipeline latency, and the rate is what CUDA events see around one launch.
#include <algorithm>

#include "plan.h"

namespace gelib_b200 {

namespace {

__global__ void __launch_bounds__(256) ffma_probe_kernel(float* out, int iters, float a, float b) {
  float x[16];
#pragma unroll
  for (int i = 0; i < 16; i++) x[i] = (float)(threadIdx.x + i);
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int i = 0; i < 16; i++) x[i] = fmaf(x[i], a, b);
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 16; i++) s += x[i];
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

}  // namespace

// TFLOP/s (2 flops per FFMA) of the current device, best of `reps` launches; <= 0 on failure.  `scratch` must hold
// ctas * 256 floats of device memory (the caller's: nothing is allocated here).
double probe_fp32_tflops(float* scratch, int ctas, int reps, cudaStream_t s) {
  if (!scratch || ctas <= 0) return -1.0;
  const int iters = 4096;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -1.0;
  double best = -1.0;
  for (int r = 0; r < reps + 1; r++) {  // the first launch warms up
    cudaEventRecord(e0, s);
    ffma_probe_kernel<<<ctas, 256, 0, s>>>(scratch, iters, 1.0001f, 0.5f);
    cudaEventRecord(e1, s);
    if (cudaEventSynchronize(e1) != cudaSuccess) break;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    count_launch();
    if (r > 0 && ms > 0.f) best = std::max(best, 2.0 * 16 * iters * 256.0 * ctas / (ms * 1e-3) / 1e12);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return best;
}

}  // namespace gelib_b200
