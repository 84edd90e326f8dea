// What the tcgen05 / TMEM kernels of this library share: the instruction wrappers, bounded waits, ring positions, and
// the functions that turn activations into B-operand blocks (digits, planes, the K-major core-matrix order).
#pragma once

#include <algorithm>
#include <cstring>
#include <mutex>

#include "launch.cuh"

namespace b200 {
namespace {

constexpr int kBM = 128;          // rows the tensor core multiplies = TMEM lanes; a tile uses the first R of them
constexpr int kTmemColumns = 512;
constexpr int kMinTileRows = 32;  // below this the instruction rate of the tensor pipe, not HBM, would bound a stage
constexpr int kMaxRows = 64;      // activation rows per pass
constexpr int kStatusTcWait = 5;  // a bounded wait of this kernel gave up

// How activations become B-operand columns.
enum ActMath { kActBf16 = 0, kActF16 = 1, kActE4m3 = 2, kActS8 = 3 };
constexpr int act_elem(int act) { return act == kActBf16 || act == kActF16 ? 2 : 1; }
// Values of K per stage. (512 for the 8-bit formats halves the per-stage bookkeeping but was no faster, and the
// activation blocks of 32 rows and more no longer fit beside a useful weight ring.)
constexpr int ks_of(int) { return 256; }

template <int F>
struct TcFmt;
template <>
struct TcFmt<LX_W_BF16> {
  static constexpr int kRowBytes = 512;  // bytes per weight row per stage
  static constexpr int kAct = kActBf16;
};
template <>
struct TcFmt<LX_W_INT8> {
  static constexpr int kRowBytes = 256;
  static constexpr int kAct = kActS8;
};
template <>
struct TcFmt<LX_W_FP8> {
  static constexpr int kRowBytes = 256;
  static constexpr int kAct = kActE4m3;
};
template <>
struct TcFmt<LX_W_NVFP4> {
  static constexpr int kRowBytes = 128;
  static constexpr int kAct = kActF16;
};
inline int act_planes(int act, bool x_bf16) {
  return act == kActS8 ? 3 : act == kActE4m3 ? (x_bf16 ? 2 : 3) : (x_bf16 ? 1 : 2);
}

// ---- tcgen05 wrappers ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// No memory clobber: the store touches tensor memory only, so the compiler may move the shared-memory loads of later
// chunks above it. tcgen05.wait::st (volatile, with a clobber) still orders the stores before the mbarrier arrival.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]));
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[smem descriptor] * B[smem descriptor], one CTA.
template <int kAct>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (kAct == kActE4m3) {
    asm volatile(
        "{ .reg .pred p; setp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if constexpr (kAct == kActS8) {
    asm volatile(
        "{ .reg .pred p; setp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{ .reg .pred p; setp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// D[tmem] (+)= A[tmem] * B[smem descriptor], one CTA, f16 operands.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.u32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every tcgen05.mma issued so far by this thread has completed.
// The same with the two descriptors given as 32-bit halves: the issuing thread is one thread whose own instruction
// stream bounds a stage (measured: ~1200 cycles per stage of eight products), so the 64-bit descriptor arithmetic is
// kept out of it; per product the low words move by a constant.
template <int kAct>
__device__ __forceinline__ void umma_ss_halves(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t accumulate) {
  if constexpr (kAct == kActE4m3) {
    asm volatile(
        "{ .reg .pred p; .reg .b64 da, db; setp.ne.u32 p, %6, 0; mov.b64 da, {%1, %2}; mov.b64 db, {%3, %4};\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %5, p; }" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if constexpr (kAct == kActS8) {
    asm volatile(
        "{ .reg .pred p; .reg .b64 da, db; setp.ne.u32 p, %6, 0; mov.b64 da, {%1, %2}; mov.b64 db, {%3, %4};\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p; }" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{ .reg .pred p; .reg .b64 da, db; setp.ne.u32 p, %6, 0; mov.b64 da, {%1, %2}; mov.b64 db, {%3, %4};\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p; }" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Shared-memory operand descriptor: K-major, no swizzle; core matrices are 8 rows x 16 bytes (128 contiguous bytes),
// lbo = bytes between core matrices next to each other along K, sbo = along the row dimension.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((addr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(lbo >> 4) << 16) |
         (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46);
}

// The same for a tile that a 2-D TMA copy wrote with the 128-byte swizzle (rows of 128 bytes, groups of 8 rows 1024
// bytes apart); K advances inside the 128 bytes by moving the start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return static_cast<uint64_t>((addr & 0x3ffffu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

// A wait of this kernel: at most 0.25 s. A role whose wait gives up records it and leaves its loops at once (each of the
// other roles then gives up on its own next wait), so the CTA still reaches the end and frees its tensor memory.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > 250000000ull) {
      if (status) atomicExch(status, kStatusTcWait);
      return false;
    }
  }
}

// Position in a ring of `depth` slots: the slot and the parity of the ring's current lap (no division in the loops:
// an integer division by a run-time depth costs more than the eight products of a stage).
struct Ring {
  int slot = 0;
  uint32_t lap = 0;
  __device__ __forceinline__ void advance(int depth) {
    if (++slot == depth) {
      slot = 0;
      lap ^= 1u;
    }
  }
};

// ---- activation preparation ----------------------------------------------------------------------------------------
// The same functions serve the preparation kernel (more than 8 activation rows) and the CTAs that prepare their own
// activations (up to 8 rows), so a row's digits, and with them its sums, are the same bits on either way.

// V consecutive activations of a row starting at k0, as f32; zero past K.
template <bool XBF, int V>
__device__ __forceinline__ void load_values(const void* __restrict__ x, int64_t row, int k0, int K, bool aligned16, float (&v)[V]) {
  if (aligned16 && k0 + V <= K) {
    if constexpr (XBF) {
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + row + k0);
#pragma unroll
      for (int q = 0; q < V / 8; ++q) {
        const uint4 t = src[q];
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int z = 0; z < 4; ++z) {
          v[8 * q + 2 * z] = __uint_as_float(w[z] << 16);
          v[8 * q + 2 * z + 1] = __uint_as_float(w[z] & 0xffff0000u);
        }
      }
    } else {
      const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(x) + row + k0);
#pragma unroll
      for (int q = 0; q < V / 4; ++q) {
        const float4 t = src[q];
        v[4 * q] = t.x, v[4 * q + 1] = t.y, v[4 * q + 2] = t.z, v[4 * q + 3] = t.w;
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) v[i] = k0 + i < K ? load_f32(x, XBF ? LX_BF16 : LX_F32, row + k0 + i) : 0.0f;
  }
}

// Thread t of n: the largest magnitude among its share of a row (the callers reduce over the n threads).
template <bool XBF>
__device__ __forceinline__ float row_max_share(const void* __restrict__ x, int64_t row, int K, bool aligned16, int t, int n) {
  float a = 0.0f;
  if (XBF && aligned16) {
    const uint4* xr = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + row);
    uint32_t m = 0;  // bf16 magnitudes compare as integers
    for (int i = t; i < K / 8; i += n) {
      const uint4 q = xr[i];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int z = 0; z < 4; ++z) {
        m = max(m, (w[z] & 0x7fffu) << 16);
        m = max(m, w[z] & 0x7fff0000u);
      }
    }
    a = __uint_as_float(m);
    for (int k = K / 8 * 8 + t; k < K; k += n) a = fmaxf(a, fabsf(load_f32(x, LX_BF16, row + k)));
  } else if (!XBF && aligned16) {
    const float4* xr = reinterpret_cast<const float4*>(static_cast<const float*>(x) + row);
    for (int i = t; i < K / 4; i += n) {
      const float4 q = xr[i];
      a = fmaxf(fmaxf(a, fabsf(q.x)), fmaxf(fabsf(q.y), fmaxf(fabsf(q.z), fabsf(q.w))));
    }
    for (int k = K / 4 * 4 + t; k < K; k += n) a = fmaxf(a, fabsf(load_f32(x, LX_F32, row + k)));
  } else {
    for (int k = t; k < K; k += n) a = fmaxf(a, fabsf(load_f32(x, XBF ? LX_BF16 : LX_F32, row + k)));
  }
  return a;
}

// The power of two that brings a row's largest magnitude into the math's top binade: 2^14 for f16 (below 65504),
// 2^7 for e4m3 (below 448), 2^5 for the first int8 digit (at most 64); 1 for bf16 (no scaling).
template <int ACT>
__device__ __forceinline__ float scale_of(float a) {
  if constexpr (ACT == kActBf16) return 1.0f;
  constexpr int kTop = ACT == kActF16 ? 14 : ACT == kActE4m3 ? 7 : 5;
  int ex = static_cast<int>((__float_as_uint(a) >> 23) & 0xffu);
  ex = a > 0.0f ? min(max(ex, 30), 230) : 127 + kTop;
  return __uint_as_float(static_cast<uint32_t>(254 + kTop - ex) << 23);
}

// The low-precision maths (INT8 weights x int8 activations, FP8 x e4m3): a row is quantized once as lx_quantize_act
// quantizes it (lernex/dromos engine/cuda/quant.cu; kernels.h "lx_quantize_act"): scale = max|x| / top with top = 127 or
// 448 (1 for an all-zero row), values x * (top / max|x|) rounded to nearest even and clamped.
template <int ACT>
__device__ __forceinline__ void quant_scales(float a, float& to_q, float& back) {
  constexpr float kTop = ACT == kActS8 ? 127.0f : 448.0f;
  to_q = a > 0.0f ? __fdiv_rn(kTop, a) : 0.0f;
  back = a > 0.0f ? __fdiv_rn(a, kTop) : 1.0f;
}
template <int ACT>
__device__ __forceinline__ void quantize_plane(const float (&v)[16], float to_q, uint32_t (&w)[4]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) w[q] = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float r = v[i] * to_q;
    uint32_t b;
    if constexpr (ACT == kActS8) b = static_cast<uint32_t>(static_cast<int>(fminf(fmaxf(rintf(r), -127.0f), 127.0f))) & 0xffu;
    else b = e4m3_encode(r) & 0xffu;
    w[i / 4] |= b << ((i % 4) * 8);
  }
}

// V = 16 / element size scaled values to the 16 bytes of each plane.
template <int ACT, bool XBF, int V>
__device__ __forceinline__ void make_planes(const float (&v)[V], float sc, uint32_t (&w)[3][4]) {
#pragma unroll
  for (int j = 0; j < 3; ++j)
#pragma unroll
    for (int q = 0; q < 4; ++q) w[j][q] = 0;
  if constexpr (ACT == kActBf16 || ACT == kActF16) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float r = v[i] * sc;
      uint32_t hi, lo = 0;
      if constexpr (ACT == kActBf16) {
        hi = f32_to_bf16_bits(r);
        if (!XBF) lo = f32_to_bf16_bits(r - bf16_bits_to_f32(hi));
      } else {
        const __half h = __float2half_rn(r);
        hi = __half_as_ushort(h);
        if (!XBF) lo = __half_as_ushort(__float2half_rn(r - __half2float(h)));
      }
      w[0][i / 2] |= (hi & 0xffffu) << ((i % 2) * 16);
      w[1][i / 2] |= (lo & 0xffffu) << ((i % 2) * 16);
    }
  } else if constexpr (ACT == kActE4m3) {
    // Digits in base 16 of the scaled value: each e4m3 takes the next four significant bits. Two values per
    // conversion instruction (saturating, round to nearest even); the digit's value comes back through f16, exactly.
#pragma unroll
    for (int i = 0; i < V; i += 2) {
      float r0 = v[i] * sc, r1 = v[i + 1] * sc;
#pragma unroll
      for (int j = 0; j < (XBF ? 2 : 3); ++j) {
        uint32_t pair;  // bits 0-7: the digit of r0, bits 8-15: of r1
        asm("{ .reg .b16 p; cvt.rn.satfinite.e4m3x2.f32 p, %2, %1; cvt.u32.u16 %0, p; }" : "=r"(pair) : "f"(r0), "f"(r1));
        uint32_t h2;
        asm("{ .reg .b16 p; cvt.u16.u32 p, %1; cvt.rn.f16x2.e4m3x2 %0, p; }" : "=r"(h2) : "r"(pair));
        const __half2 back = *reinterpret_cast<const __half2*>(&h2);
        r0 = (r0 - __low2float(back)) * 16.0f;
        r1 = (r1 - __high2float(back)) * 16.0f;
        w[j][i / 4] |= pair << ((i % 4) * 8);
      }
    }
  } else {
    // Digits in base 128 of the scaled value (below 64 in magnitude), each in [-64, 64): the value is rounded once to
    // 14 binary places and the integer split exactly.
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int q = __float2int_rn(v[i] * sc * 16384.0f);
      const int d2 = ((q + 64) & 127) - 64;
      const int q1 = (q - d2) >> 7;
      const int d1 = ((q1 + 64) & 127) - 64;
      const int d0 = (q1 - d1) >> 7;
      w[0][i / 4] |= (static_cast<uint32_t>(d0) & 0xffu) << ((i % 4) * 8);
      w[1][i / 4] |= (static_cast<uint32_t>(d1) & 0xffu) << ((i % 4) * 8);
      w[2][i / 4] |= (static_cast<uint32_t>(d2) & 0xffu) << ((i % 4) * 8);
    }
  }
}

// Where the 16 bytes at byte offset kb (a multiple of 16) along K of column c sit inside a stage's block: the K-major
// core-matrix order of the B operand (8 columns x 16 bytes per core matrix).
__device__ __forceinline__ int block_offset(int NC, int kb, int c) { return ((kb >> 4) * (NC >> 3) + (c >> 3)) * 128 + (c & 7) * 16; }

// ---- host side ---------------------------------------------------------------------------------------------------------
inline int sm_count() {
  static std::mutex mu;
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::lock_guard<std::mutex> lock(mu);
  if (!sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    sms[dev] = n;
  }
  return sms[dev];
}

// Tag: one flag set per kernel (the instantiations of a kernel template share a function type).
template <int Tag, typename Kernel>
int allow_big_smem(Kernel kernel) {
  static std::mutex mu;
  static bool done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::lock_guard<std::mutex> lock(mu);
  if (!done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    // all of the SM's L1 as shared memory, so that two CTAs of half an SM each fit side by side
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    done[dev] = true;
  }
  return kOk;
}

// The same opt-in without the carve-out preference: a kernel that reads through L1 (plain loads, many in flight) wants
// the driver to leave L1 everything its shared memory does not need. Measured: with the whole of L1 carved out as shared
// memory the decode GEMV streamed at 2.4 TB/s instead of 6.
template <int Tag, typename Kernel>
int allow_dynamic_smem(Kernel kernel) {
  static std::mutex mu;
  static bool done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::lock_guard<std::mutex> lock(mu);
  if (!done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    done[dev] = true;
  }
  return kOk;
}

inline int act_of(int wtype) {
  return wtype == LX_W_BF16 ? kActBf16 : wtype == LX_W_INT8 ? kActS8 : wtype == LX_W_FP8 ? kActE4m3 : kActF16;
}

}  // namespace
}  // namespace b200
