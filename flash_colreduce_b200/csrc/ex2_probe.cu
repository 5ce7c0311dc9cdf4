// Measurement helper of the benchmark, built as a library of its own
// (libfcr_ex2_probe.so): the rate at which this GPU evaluates
// ex2.approx.ftz.f32, the instruction the softmax folds of the operator use for
// one exponential per attention score.  The benchmark divides the number of
// scores by this rate to get the exponential-unit bound of the roofline.  Not
// part of the operator library and not needed to use it.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

namespace {

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Eight independent dependency chains per thread, registers only.
__global__ void ex2_probe_kernel(float* sink, int iters) {
  float v[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) v[u] = -1.0f - 0.001f * (float)(threadIdx.x + u);
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = ex2(v[u]) - 1.5f;
  }
  float s = 0.f;
#pragma unroll
  for (int u = 0; u < 8; ++u) s += v[u];
  if (s == 123.456f) sink[0] = s;
}

}  // namespace

// Exponentials per second sustained by the current device (best of `repeats` runs);
// synchronises the device; 0 on any error.
extern "C" double fcr_probe_ex2_rate(int32_t repeats) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0.0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0.0;
  float* sink = nullptr;
  if (cudaMalloc(&sink, 256) != cudaSuccess) return 0.0;
  const int iters = 4096, threads = 1024, blocks = sms * 2;
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  ex2_probe_kernel<<<blocks, threads>>>(sink, iters);
  double best = 0.0;
  for (int r = 0; r < std::max(repeats, 1); ++r) {
    cudaEventRecord(a);
    ex2_probe_kernel<<<blocks, threads>>>(sink, iters);
    cudaEventRecord(b);
    if (cudaEventSynchronize(b) != cudaSuccess) break;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, a, b);
    best = std::max(best, (double)blocks * threads * 8.0 * iters / (ms * 1e-3));
  }
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  cudaFree(sink);
  return best;
}
