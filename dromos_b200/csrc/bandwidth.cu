// lx_bandwidth_probe: the read-only DRAM bandwidth of the current device, the ceiling a weight-streaming kernel is
// measured against (ABI: lernex/dromos engine/cuda/kernels.h:373). A buffer far larger than L2 is read with 16-byte
// loads, eight in flight per thread; the best of `reps` timed passes is reported.
#include <algorithm>

#include "launch.cuh"

namespace b200 {
namespace {

template <int kUnroll>
__global__ void __launch_bounds__(256) read_kernel(const uint4* __restrict__ src, int64_t n16, uint32_t* sink) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  uint32_t acc = 0;
  for (; i + (kUnroll - 1) * stride < n16; i += kUnroll * stride) {
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) v[u] = __ldcs(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  for (; i < n16; i += stride) {
    const uint4 v = __ldcs(src + i);
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  if (acc == 0x9e3779b9u) *sink = acc;  // keeps the loads alive; practically never true
}

__global__ void __launch_bounds__(256) fill_kernel(uint4* dst, int64_t n16) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint32_t h = static_cast<uint32_t>(i) * 2654435761u;
    dst[i] = make_uint4(h, h ^ 0x5bd1e995u, h + 0x27d4eb2fu, ~h);
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int lx_bandwidth_probe(int64_t bytes, int reps, double* read_gbps, double* spec_gbps, void* stream) {
  if (bytes < 65536 || bytes % 16 != 0 || reps <= 0 || !read_gbps) return kInvalid;
  auto s = static_cast<cudaStream_t>(stream);
  uint4* buf = nullptr;
  uint32_t* sink = nullptr;
  if (cudaMalloc(&buf, bytes) != cudaSuccess) return static_cast<int>(cudaGetLastError());
  if (cudaMalloc(&sink, 4) != cudaSuccess) {
    const int e = static_cast<int>(cudaGetLastError());
    cudaFree(buf);
    return e;
  }
  int dev = 0, sms = 148, mem_khz = 0, bus_bits = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&mem_khz, cudaDevAttrMemoryClockRate, dev);
  cudaDeviceGetAttribute(&bus_bits, cudaDevAttrGlobalMemoryBusWidth, dev);
  if (spec_gbps) *spec_gbps = 2.0 * mem_khz * 1e3 * (bus_bits / 8.0) / 1e9;
  const int64_t n16 = bytes / 16;
  cudaEvent_t t0, t1;
  cudaEventCreate(&t0);
  cudaEventCreate(&t1);
  int e = launch_kernel(fill_kernel, dim3(sms * 8), dim3(256), 0, s, buf, n16);
  double best = 0.0;
  for (int r = 0; r < reps + 1 && !e; ++r) {  // the first pass is a warm-up
    cudaEventRecord(t0, s);
    e = launch_kernel(read_kernel<8>, dim3(sms * 8), dim3(256), 0, s, static_cast<const uint4*>(buf), n16, sink);
    cudaEventRecord(t1, s);
    if (cudaEventSynchronize(t1) != cudaSuccess) e = static_cast<int>(cudaGetLastError());
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, t0, t1);
    if (r > 0 && ms > 0.0f) best = std::max(best, bytes / (ms * 1e-3) / 1e9);
  }
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  cudaFree(buf);
  cudaFree(sink);
  *read_gbps = best;
  return e;
}
