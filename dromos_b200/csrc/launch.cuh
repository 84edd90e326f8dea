// Host-side launch helpers: every kernel of the library is launched through launch_kernel, which counts the launch,
// marks it for programmatic dependent launch (the kernel may start while its predecessor in the stream drains; it
// calls griddepcontrol.wait before reading anything the predecessor wrote) and returns the launch status.
#pragma once

#include <cstdlib>
#include <mutex>

#include "stream.cuh"

namespace b200 {

// LX_PDL=0 turns programmatic dependent launch off (plain stream order), as in the reference's common.cuh switch.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LX_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

// LX_B200_FORCE_SCALAR=1 sends every dense product down the scalar kernel (a second implementation to test against).
inline bool force_scalar() {
  const char* v = std::getenv("LX_B200_FORCE_SCALAR");
  return v && v[0] == '1';
}

template <typename... KArgs, typename... Args>
int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(e);
  }
  return kOk;
}

template <int F, int RT, int WR, int NT, int U, int S, int MODE>
int launch_stream(const StreamParams& P, dim3 grid, cudaStream_t stream) {
  auto kernel = stream_kernel<F, RT, WR, NT, U, S, MODE>;
  const size_t smem = stream_smem_bytes<F, RT, WR, NT, U, S>(P.K);
  // The opt-in to more than 48 KB of dynamic shared memory is per device and per kernel; set it once per device.
  static std::mutex mu;
  static unsigned long long done_mask = 0;  // bit per device ordinal (< 64)
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!(done_mask >> (dev & 63) & 1ull)) {
      const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
      if (e != cudaSuccess) {
        cudaGetLastError();
        return static_cast<int>(e);
      }
      done_mask |= 1ull << (dev & 63);
    }
  }
  if (smem > 220 * 1024) return kNotSupported;
  return launch_kernel(kernel, grid, dim3(kThreads), smem, stream, P);
}

struct ActLayout {
  int64_t ld_q, ld_bs;
  int64_t q_off, scale_off, bs_off, total;
};
ActLayout act_layout(int M, int K, int math);

}  // namespace b200
