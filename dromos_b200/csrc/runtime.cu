// Process-wide state of the library: launch counter, per-device status word, architecture query / override, the
// variant table (tunable.h of the reference ABI) and the two runtime entry points the reference's loader probes.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "launch.cuh"
#include "variants.h"

namespace b200 {

std::atomic<int64_t> g_launches{0};

int* status_word() {
  static std::mutex mu;
  static int* words[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::lock_guard<std::mutex> lock(mu);
  if (!words[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    cudaMemset(p, 0, sizeof(int));
    words[dev] = p;
  }
  return words[dev];
}

int split_scratch(float** partials, int** flags) {
  static std::mutex mu;
  static uint8_t* base[64] = {};
  static unsigned next[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::lock_guard<std::mutex> lock(mu);
  const size_t region = static_cast<size_t>(kSplitMaxCtas) * (kSplitBytesPerCta + sizeof(int));
  if (!base[dev]) {
    void* p = nullptr;
    if (cudaMalloc(&p, region * kSplitRegions) != cudaSuccess) {
      cudaGetLastError();
      return kNotSupported;
    }
    cudaMemset(p, 0, region * kSplitRegions);
    base[dev] = static_cast<uint8_t*>(p);
  }
  uint8_t* r = base[dev] + region * (next[dev]++ % kSplitRegions);
  *partials = reinterpret_cast<float*>(r);
  *flags = reinterpret_cast<int*>(r + static_cast<size_t>(kSplitMaxCtas) * kSplitBytesPerCta);
  return kOk;
}

TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<TensorMapEncodeFn>(p);
  }();
  return fn;
}

namespace {

std::mutex g_mu;
int g_arch_override = -1;  // -1: LX_ARCH_OVERRIDE not read yet

struct TableKey {
  std::string kernel;
  int m_bucket, N, K;
  bool operator<(const TableKey& o) const {
    return std::tie(kernel, m_bucket, N, K) < std::tie(o.kernel, o.m_bucket, o.N, o.K);
  }
};
std::map<TableKey, int>& table() {
  static std::map<TableKey, int> t;
  return t;
}

// M is bucketed to the next power of two, so one entry covers a range of batch sizes (tunable.h:47-49).
int m_bucket(int m) {
  int b = 1;
  while (b < m) b <<= 1;
  return b;
}

int real_arch() {
  int dev = 0, major = 0, minor = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
  return 10 * major + minor;
}

const VariantList* find_kernel(const char* name) {
  if (!name) return nullptr;
  for (int i = 0; i < kVariantKernels; ++i)
    if (std::strcmp(kVariantTable[i].kernel, name) == 0) return &kVariantTable[i];
  return nullptr;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int lx_arch(void) {
  const int real = real_arch();
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_arch_override < 0) {
    const char* env = std::getenv("LX_ARCH_OVERRIDE");
    g_arch_override = env ? std::max(0, std::atoi(env)) : 0;
  }
  return g_arch_override > 0 && g_arch_override < real ? g_arch_override : real;
}

int lx_set_arch_override(int arch) {
  {
    std::lock_guard<std::mutex> lock(g_mu);
    g_arch_override = arch > 0 ? arch : 0;
  }
  return lx_arch();
}

int lx_tune_get(const char* kernel, int M, int N, int K) {
  if (!kernel) return -1;
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = table().find(TableKey{kernel, m_bucket(M), N, K});
  return it == table().end() ? -1 : it->second;
}

// The admission rule of the decode GEMV kernels (the reference's order-class rule, engine/cuda/tunable.cu:104-118): a
// variant is stored only if it adds a row's products in the same order as what runs by default for that format and K,
// because a row's bits must not depend on the M bucket the table is keyed on, and the BF16X kernel must keep the bits of
// the bf16 kernel. The default is the tcgen05 product for INT8 weights wide enough for it (class 2), else the decode
// GEMV where the shape admits it (class 0), else the TMA-ring kernel (class 1); a GEMV variant named for a shape the
// GEMV cannot take changes nothing and is admitted.
int lx_tune_set(const char* kernel, int M, int N, int K, int variant) {
  if (!kernel) return kInvalid;
  const VariantList* v = find_kernel(kernel);
  if (v && (variant < 0 || variant >= v->count)) return LX_ERR_TUNE_VARIANT;
  const int wtype = gemv_kernel_wtype(kernel);
  if (wtype >= 0) {
    const bool eligible = gemv_shape_ok(wtype, K, true);
    const bool wide_int8 = wtype == LX_W_INT8 && tc_rows_shape_ok(wtype, N, K);
    const int cls = gemv_order_class(wtype == LX_W_BF16X ? x16_variant(variant) : variant), default_cls = wide_int8 ? 2 : eligible ? 0 : 1;
    if (cls != default_cls && !(cls == 0 && !eligible && !wide_int8)) return LX_ERR_TUNE_REJECTED;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  table()[TableKey{kernel, m_bucket(M), N, K}] = variant;
  return kOk;
}

// Stores a variant with no admission check (tunable.h:50-52): for tests and benchmarks that run every variant.
int lx_tune_force(const char* kernel, int M, int N, int K, int variant) {
  if (!kernel) return kInvalid;
  const VariantList* v = find_kernel(kernel);
  if (v && (variant < 0 || variant >= v->count)) return LX_ERR_TUNE_VARIANT;
  std::lock_guard<std::mutex> lock(g_mu);
  table()[TableKey{kernel, m_bucket(M), N, K}] = variant;
  return kOk;
}

void lx_tune_clear(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  table().clear();
}

int lx_tune_kernels(const char** names, int capacity) {
  for (int i = 0; i < kVariantKernels && i < capacity; ++i) names[i] = kVariantTable[i].kernel;
  return kVariantKernels;
}

int lx_tune_variants(const char* kernel) {
  const VariantList* v = find_kernel(kernel);
  return v ? v->count : 0;
}

const char* lx_tune_variant_name(const char* kernel, int variant) {
  const VariantList* v = find_kernel(kernel);
  return v && variant >= 0 && variant < v->count ? v->names[variant] : nullptr;
}

// The autotuner's timing hook: this library's callers time variants through the product entry points themselves
// (lx_tune_force + lx_gemv_w), so no kernel registers a runner.
int lx_tune_run(const char*, int, const lx_tune_problem*, float*, void*) { return kNotSupported; }
int lx_tune_runnable(const char*) { return 0; }

// The key of a problem in the table: the kernel name, then "@w<format>m<math>" and "@e<experts>" when they are not
// the defaults (tunable.h:71-75).
int lx_tune_key(const char* kernel, const lx_tune_problem* problem, char* out, int capacity) {
  if (!kernel || !problem) return 0;
  std::string key = kernel;
  if (problem->weight != 0 || problem->math != 0)
    key += "@w" + std::to_string(problem->weight) + "m" + std::to_string(problem->math);
  if (problem->experts != 1) key += "@e" + std::to_string(problem->experts);
  if (out && capacity > 0) {
    const size_t n = std::min(key.size(), static_cast<size_t>(capacity - 1));
    std::memcpy(out, key.data(), n);
    out[n] = '\0';
  }
  return static_cast<int>(key.size());
}

int lx_rt_backend(void) { return LX_BACKEND_CUDA; }

int lx_rt_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int64_t lx_b200_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

int lx_b200_last_error(void) {
  int* w = status_word();
  if (!w) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -static_cast<int>(cudaGetLastError());
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -static_cast<int>(cudaGetLastError());
  if (v) cudaMemset(w, 0, sizeof(int));
  // the entry point that allocates nothing keeps its kernels' status in the first word of its own array
  if (int* sw = static_scratch_status()) {
    int sv = 0;
    if (cudaMemcpy(&sv, sw, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -static_cast<int>(cudaGetLastError());
    if (sv) cudaMemset(sw, 0, sizeof(int));
    if (!v) v = sv;
  }
  return v;
}

}  // extern "C"
