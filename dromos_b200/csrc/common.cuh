// Shared device and host helpers of libdromos_b200: error codes, launch accounting, the device status word,
// mbarrier / bulk-copy (TMA) wrappers with bounded waits, number-format conversions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "dromos_b200.h"

namespace b200 {

constexpr int kOk = 0;
constexpr int kInvalid = 1;  // cudaErrorInvalidValue
constexpr int kNotSupported = LX_ERR_NOT_SUPPORTED;

// Codes a kernel leaves in the device status word when one of its bounded waits gives up.
constexpr int kStatusFullWait = 1;   // a consumer waited for a weight stage that never arrived
constexpr int kStatusEmptyWait = 2;  // the producer waited for a ring slot that was never released
constexpr int kStatusDrainWait = 3;  // the final drain of in-flight copies ran out
constexpr int kStatusPartWait = 4;   // a CTA waited for another CTA's partial sums that never came

// ---- host: launch accounting and status -----------------------------------------------------------------
extern std::atomic<int64_t> g_launches;
// The device status word of the current device (allocated on first use, one per device, never freed).
int* status_word();
// The status word of the entry point that works in the library's own static array (its first word), once that entry
// point has looked the array up on the current device; null before.
int* static_scratch_status();

inline int launch_status() {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return static_cast<int>(cudaGetLastError());
}

inline bool valid_dtype(int d) { return d == LX_F32 || d == LX_BF16; }
inline bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// ---- device: numbers ------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
}
__device__ __forceinline__ float load_f32(const void* p, int dtype, int64_t i) {
  return dtype == LX_BF16 ? bf16_bits_to_f32(static_cast<const uint16_t*>(p)[i]) : static_cast<const float*>(p)[i];
}
__device__ __forceinline__ void store_from_f32(void* p, int dtype, int64_t i, float v) {
  if (dtype == LX_BF16) static_cast<uint16_t*>(p)[i] = static_cast<uint16_t>(f32_to_bf16_bits(v));
  else static_cast<float*>(p)[i] = v;
}
// One e4m3 byte as f32, exact (the byte's 7 magnitude bits placed at f32 bits 20..26 and rebased by 2^120;
// subnormals come out right because f32 subnormals scale the same way).
// Nearest e4m3 (ties to even), magnitudes beyond 448 saturate.
__device__ __forceinline__ uint32_t e4m3_encode(float v) {
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
  const float mag = __uint_as_float((b & 0x7fu) << 20) * 0x1p120f;
  return (b & 0x80u) ? -mag : mag;
}
// One e2m1 code (low 4 bits) as f32, exact.
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  const float mag = __uint_as_float((code & 7u) << 22) * 0x1p126f;
  return (code & 8u) ? -mag : mag;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- device: mbarrier + bulk copies ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Waits for the barrier's phase with the given parity, for at most kWaitBudgetNs. On a timeout writes `code`
// to the status word and returns false; the caller carries on (its results are then garbage, but nothing hangs).
constexpr uint64_t kWaitBudgetNs = 2000000000ull;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > kWaitBudgetNs) {
      if (status) atomicExch(status, code);
      return false;
    }
  }
}
// 1-D bulk copy global -> this CTA's shared memory, completing `bytes` on the mbarrier. Both addresses 16-byte
// aligned, bytes a multiple of 16. No multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// 2-D tile copy global -> this CTA's shared memory through a tensor map: the box the map was encoded with, from
// element x of row y. x times the element size must be a multiple of 16 bytes. No multicast.
__device__ __forceinline__ void tile_g2s(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// Asks L2 to fetch the box of a tensor map at (x, y); nothing lands in shared memory.
__device__ __forceinline__ void tile_prefetch_l2(const void* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y) : "memory");
}
// Release store / acquire load on a flag another CTA polls, and a bounded wait for it to become nonzero.
__device__ __forceinline__ void st_release(int* p, int v) { asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_cg(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ bool flag_wait(const int* flag, int* status) {
  if (ld_acquire(flag)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (ld_acquire(flag)) return true;
    if (global_timer_ns() - t0 > kWaitBudgetNs) {
      if (status) atomicExch(status, kStatusPartWait);
      return false;
    }
  }
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Programmatic dependent launch: a kernel launched with the attribute may start before its predecessor in the
// stream has finished; it must wait here before it reads anything the predecessor wrote.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- device: tensor-core fragments ----------------------------------------------------------------------
// D += A (16x16, row) * B (16x8, col), f32 accumulate. kHalf: f16 operands, else bf16.
template <bool kHalf>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kHalf) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

}  // namespace b200
