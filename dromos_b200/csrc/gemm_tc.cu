// The batched-decode product on the 5th-generation tensor cores: y[m, n] = sum_k x[m, k] * w[n, k] for 9..64 activation
// rows per pass, weights streamed once in their stored format.
//
// The weight tile is the A operand of tcgen05.mma (128 weight rows = the 128 lanes of the accumulator in tensor memory),
// the activations are the B operand (one accumulator column per activation row and digit), K advances 32 bytes per
// instruction. An instruction costs the tensor pipe at least ~46 cycles whatever the column count, so what matters is
// instructions per byte of weights, and that decides the math per format:
//
//   BF16   kind::f16, A = the bf16 weights as they land in shared memory (128-byte swizzled TMA boxes, read through a
//          shared-memory descriptor), B = bf16 activations; f32 activations as a high and a low bf16 column.
//   FP8    kind::f8f6f4, A = the e4m3 weights as they land, B = the scaled activations as two (bf16 x) or three (f32 x)
//          e4m3 digits in base 16; the digit columns are recombined in the epilogue.
//   INT8   kind::i8, A = the int8 weights as they land, B = the scaled activations as three int8 digits in base 128;
//          the s32 sums are exact.
//   NVFP4  no kind multiplies e2m1 * e4m3-block-scale weights by wider activations, so eight converter warps expand each
//          stage to f16 in registers (exact) and write it with tcgen05.st into tensor memory as the A operand of
//          kind::f16 (K = 16 per instruction); B = activations as f16 after a per-row power-of-two scaling.
//
// Roles (one CTA per SM): a weight producer thread (2-D TMA tile copies, no multicast, ring of stages with one mbarrier
// each), an activation producer thread (1-D bulk copies of prepared blocks through a second, shallower ring), one MMA
// issuer thread, and the epilogue warps (tcgen05.ld, lane = weight row; row factor, activation scale, bias, alpha /
// beta, store). The direct formats keep two accumulators in tensor memory so that the next tile's products run while
// the epilogue of the last one is still reading.
//
// Work is split by STAGE, not by tile: the n_tiles * n_stages stages are dealt out in equal contiguous ranges, one per
// CTA, so every SM streams the same number of bytes whatever N is. A tile whose stages fall to several CTAs is summed
// without any CTA waiting for another: each contributor writes its partial accumulator to the workspace and counts
// itself on the tile's counter; the one that arrives last adds the partials in the fixed order of the ranges (its own
// included, read back from the workspace) and finishes the tile. The sum therefore does not depend on arrival order.
//
// Activations are prepared once per call by a small kernel into the caller's workspace, in the K-major core-matrix
// order the B descriptor reads. The same kernel clears the tile counters.
//
// Every wait is bounded; a wait that gives up writes a code to the status word and the kernel still frees its TMEM.
#include <algorithm>
#include <cstring>

#include "launch.cuh"

namespace b200 {
namespace {

constexpr int kBM = 128;          // weight rows per tile = TMEM lanes
constexpr int kKS = 256;          // values of K per stage
constexpr int kTmemColumns = 512;
constexpr int kMaxCtas = 160;     // bound on the grid (one CTA per SM), sizes the counters and the partial slots
constexpr int kMinStagesPerCta = 4;
constexpr int kMaxRows = 64;      // activation rows per pass
constexpr int kStatusTcWait = 5;  // a bounded wait of this kernel gave up

// How activations become B-operand columns.
enum ActMath { kActBf16 = 0, kActF16 = 1, kActE4m3 = 2, kActS8 = 3 };

struct TcParams {
  const uint8_t* scale;   // f32 [N] (INT8 / FP8); NVFP4 block scales come through the tensor map
  float global;
  int N, K, M;            // M: activation rows of this pass
  int NC;                 // accumulator columns, a multiple of 16: column j * Mp + m is digit j of row m
  int Mp;                 // M rounded up to 8
  int planes;             // digits (or halves) per activation row
  float digit;            // weight of a plane relative to the one before it
  const uint8_t* xprep;   // prepared activations: n_stages blocks of x_bytes
  int x_bytes;            // NC * 256 * bytes per element
  const float* inv_scales;  // M f32: what each row's sum is multiplied by
  int* counters;          // kMaxCtas tile counters, zero when the kernel starts
  uint32_t* partials;     // 2 slots of 128 * NC words per CTA
  const void* bias;
  int bias_dtype;
  void* y;
  int y_dtype, ld_y;
  float alpha, beta;
  int* status;
  int SW, SX;             // depth of the weight ring and of the activation ring
};

// Where the parts of the workspace begin, for a pass of NC columns of `elem` bytes over n_stages stages.
struct TcLayout {
  int64_t scales, counters, partials, total;
  TcLayout(int NC, int elem, int64_t n_stages) {
    scales = n_stages * NC * kKS * elem;
    counters = scales + 256;
    partials = counters + ((kMaxCtas * 4 + 255) / 256) * 256;
    total = partials + 2ll * kMaxCtas * kBM * NC * 4;
  }
};

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
constexpr int act_elem(int act) { return act == kActBf16 || act == kActF16 ? 2 : 1; }
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

// ---- activation preparation ----------------------------------------------------------------------------------------
// Block (chunk, u): 128 threads, each 16 bytes of K of every plane of activation row u. The row's largest magnitude
// is found by every block of the row again (the row is a few KB, from L2), which saves a second kernel. With kb the
// byte offset of k inside its stage (k % 256 times the element size), plane j of row u is column c = j * Mp + u and
// goes to
//   stage * x_bytes + ((kb / 16) * (NC / 8) + c / 8) * 128 + (c % 8) * 16 + kb % 16,
// the K-major core-matrix order of the B operand. k past K is written as zero up to the end of the last stage; columns
// that no row owns are never written (their accumulator columns are never read).
template <int ACT, bool XBF>
__global__ void __launch_bounds__(128) tc_prep_kernel(const void* __restrict__ x, int ld_x, int rows, int K, int NC, int Mp, int planes,
                                                      uint8_t* __restrict__ out, float* __restrict__ inv_scales, int* __restrict__ counters,
                                                      int n_stages) {
  constexpr int kElem = act_elem(ACT), V = 16 / kElem;
  constexpr int kXDtype = XBF ? LX_BF16 : LX_F32;
  pdl_trigger();
  pdl_wait();  // the kernel before this one may still be reading the workspace
  __shared__ float part[4];
  const int u = blockIdx.y, tid = threadIdx.x;
  if (blockIdx.x == 0 && u == 0)
    for (int i = tid; i < kMaxCtas; i += 128) counters[i] = 0;
  const int k0 = (blockIdx.x * 128 + tid) * V;
  const bool in_range = k0 < n_stages * kKS;
  const int kb = (k0 % kKS) * kElem;
  const size_t x_bytes = static_cast<size_t>(NC) * kKS * kElem;
  auto address = [&](int c) {
    return out + static_cast<size_t>(k0 / kKS) * x_bytes + (static_cast<size_t>(kb / 16) * (NC / 8) + c / 8) * 128 + (c % 8) * 16;
  };
  const int64_t row = static_cast<int64_t>(u) * ld_x;
  const bool aligned16 = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ld_x % (XBF ? 8 : 4) == 0;
  // this thread's values first (the loads are in flight while the row's largest magnitude is found)
  float v[V];
  if (in_range && aligned16 && k0 + V <= K) {
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
    for (int i = 0; i < V; ++i) v[i] = (in_range && k0 + i < K) ? load_f32(x, kXDtype, row + k0 + i) : 0.0f;
  }
  float sc = 1.0f;
  if constexpr (ACT != kActBf16) {
    float a = 0.0f;
    if (XBF && aligned16) {
      const uint4* xr = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + row);
      uint32_t m = 0;  // bf16 magnitudes compare as integers
      for (int i = tid; i < K / 8; i += 128) {
        const uint4 q = xr[i];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          m = max(m, (w[t] & 0x7fffu) << 16);
          m = max(m, w[t] & 0x7fff0000u);
        }
      }
      a = __uint_as_float(m);
      for (int k = K / 8 * 8 + tid; k < K; k += 128) a = fmaxf(a, fabsf(load_f32(x, kXDtype, row + k)));
    } else if (!XBF && aligned16) {
      const float4* xr = reinterpret_cast<const float4*>(static_cast<const float*>(x) + row);
      for (int i = tid; i < K / 4; i += 128) {
        const float4 q = xr[i];
        a = fmaxf(fmaxf(a, fabsf(q.x)), fmaxf(fabsf(q.y), fmaxf(fabsf(q.z), fabsf(q.w))));
      }
      for (int k = K / 4 * 4 + tid; k < K; k += 128) a = fmaxf(a, fabsf(load_f32(x, kXDtype, row + k)));
    } else {
      for (int k = tid; k < K; k += 128) a = fmaxf(a, fabsf(load_f32(x, kXDtype, row + k)));
    }
    a = warp_max(a);
    if ((tid & 31) == 0) part[tid >> 5] = a;
    __syncthreads();
    a = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
    // The power of two that brings the largest magnitude into the math's top binade: 2^14 for f16 (below 65504),
    // 2^7 for e4m3 (below 448), 2^5 for the first int8 digit (at most 64).
    constexpr int kTop = ACT == kActF16 ? 14 : ACT == kActE4m3 ? 7 : 5;
    int ex = static_cast<int>((__float_as_uint(a) >> 23) & 0xffu);
    ex = a > 0.0f ? min(max(ex, 30), 230) : 127 + kTop;
    sc = __uint_as_float(static_cast<uint32_t>(254 + kTop - ex) << 23);
  }
  if (blockIdx.x == 0 && tid == 0) inv_scales[u] = 1.0f / sc;
  if (!in_range) return;
  uint32_t w[3][4] = {};
#pragma unroll
  for (int i = 0; i < V; ++i) {
    float r = v[i] * sc;
    uint32_t d[3] = {0, 0, 0};
    if constexpr (ACT == kActBf16) {
      d[0] = f32_to_bf16_bits(r);
      if (!XBF) d[1] = f32_to_bf16_bits(r - bf16_bits_to_f32(d[0]));
    } else if constexpr (ACT == kActF16) {
      const __half h = __float2half_rn(r);
      d[0] = __half_as_ushort(h);
      if (!XBF) d[1] = __half_as_ushort(__float2half_rn(r - __half2float(h)));
    } else if constexpr (ACT == kActE4m3) {
      // digits in base 16 of the scaled value: each e4m3 takes the next four significant bits
#pragma unroll
      for (int j = 0; j < (XBF ? 2 : 3); ++j) {
        d[j] = __nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
        r = (r - e4m3_to_f32(d[j])) * 16.0f;
      }
    } else {
      // digits in base 128 of the scaled value, each in [-64, 64]
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const float q = rintf(r);
        d[j] = static_cast<uint32_t>(static_cast<int>(q)) & 0xffu;
        r = (r - q) * 128.0f;
      }
    }
    constexpr uint32_t kMask = kElem == 2 ? 0xffffu : 0xffu;
#pragma unroll
    for (int j = 0; j < 3; ++j) w[j][i * kElem / 4] |= (d[j] & kMask) << ((i * kElem % 4) * 8);
  }
  for (int j = 0; j < planes; ++j) *reinterpret_cast<uint4*>(address(j * Mp + u)) = make_uint4(w[j][0], w[j][1], w[j][2], w[j][3]);
}

// ---- expanding NVFP4 -------------------------------------------------------------------------------------------------
// 16 e2m1 values (8 bytes) times one e4m3 block scale
__device__ __forceinline__ void expand_nvfp4(uint32_t w0, uint32_t w1, uint32_t scale_byte, uint32_t (&p)[8]) {
  uint32_t s2;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(s2) : "r"(scale_byte & 0xffu));
  const uint32_t s = __byte_perm(s2, s2, 0x1010);
  const uint32_t w[2] = {w0, w1};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t v0, v1, v2, v3;
    asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0; cvt.rn.f16x2.e2m1x2 %1, b1; cvt.rn.f16x2.e2m1x2 %2, b2; cvt.rn.f16x2.e2m1x2 %3, b3; }"
        : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
        : "r"(w[i]));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v0) : "r"(s));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v1) : "r"(s));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v2) : "r"(s));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v3) : "r"(s));
    p[4 * i] = v0, p[4 * i + 1] = v1, p[4 * i + 2] = v2, p[4 * i + 3] = v3;
  }
}

// ---- dealing stages to CTAs ----------------------------------------------------------------------------------------
// First stage of CTA b's range when `total` stages are dealt to `ctas` CTAs.
__host__ __device__ __forceinline__ int range_begin(int total, int ctas, int b) {
  return static_cast<int>(static_cast<int64_t>(total) * b / ctas);
}
// The CTA whose range holds stage g.
__device__ __forceinline__ int owner_of(int total, int ctas, int g) {
  int b = static_cast<int>(static_cast<int64_t>(g) * ctas / total);
  while (b + 1 < ctas && range_begin(total, ctas, b + 1) <= g) ++b;
  while (b > 0 && range_begin(total, ctas, b) > g) --b;
  return b;
}

// ---- finishing a segment (this CTA's stages of one tile) --------------------------------------------------------------
// The epilogue warps of a CTA: `warps` of them meet on group_bar; the calling thread owns weight row r of the tile
// (accumulator lane r, its warp's lane quarter already in d_addr) and the 8-row chunks chunk0, chunk0 + chunk_step, ...
struct Epilogue {
  uint32_t group_bar;
  int warps;
  int meetings;
  volatile int* flags;  // two words, used alternately, so that a flag is not rewritten while a slow warp still reads it
  bool leader;
  int lane;
  int chunk0, chunk_step;
  // All epilogue warps meet (a bounded wait, unlike bar.sync); what they wrote before is visible after.
  __device__ __forceinline__ bool meet(int* status) {
    __syncwarp();
    if (lane == 0) mbar_arrive(group_bar);
    return tc_wait(group_bar, (meetings++) & 1, status);
  }
};

__device__ __forceinline__ uint4 ld_cg_u128(const uint32_t* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int kAct>
__device__ __forceinline__ void combine_and_store(const TcParams& P, const uint32_t (&raw)[3][8], int m0, int n, float rf, float bias) {
  if (n >= P.N) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int m = m0 + j;
    if (m >= P.M) continue;
    float sum = 0.0f, digit = 1.0f;
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      if (p >= P.planes) break;
      const float v = kAct == kActS8 ? static_cast<float>(static_cast<int>(raw[p][j])) : __uint_as_float(raw[p][j]);
      sum += v * digit;
      digit *= P.digit;
    }
    sum *= P.inv_scales[m];
    float out = P.alpha * (rf * sum + bias);
    const int64_t at = static_cast<int64_t>(m) * P.ld_y + n;
    if (P.beta != 0.0f) out = fmaf(P.beta, load_f32(P.y, P.y_dtype, at), out);
    store_from_f32(P.y, P.y_dtype, at, out);
  }
}

template <int kAct>
__device__ __forceinline__ uint32_t add_raw(uint32_t a, uint32_t b) {
  if constexpr (kAct == kActS8) return a + b;  // two's complement: the s32 sums add exactly
  else return __float_as_uint(__uint_as_float(a) + __uint_as_float(b));
}

// A partial accumulator in the workspace: word (column c, row r) at ((c / 4) * 128 + r) * 4 + c % 4, so that a thread
// moves four columns of its row with one 16-byte access and a warp's accesses are contiguous.
__device__ __forceinline__ uint32_t* partial_at(uint32_t* slot, int column, int r) { return slot + ((column >> 2) * kBM + r) * 4; }

// Returns false when a bounded wait gave up. release_bar (0 = none) gets one arrival per warp as soon as the
// accumulator has been read.
//
// A tile shared by CTAs b_lo .. b_hi is finished by whichever of them comes last, and the sum always runs in the order
// b_lo, b_lo + 1, ...: a contributor first looks at the tile's counter; if all the others have counted themselves it
// adds their partials (from the workspace) and its own (from tensor memory, at its place in the order) and stores the
// result. Otherwise it writes its partial, counts itself, and only if the others arrived in between does it finish
// the tile after all, now reading every part from the workspace. Nobody waits for anybody.
template <int F>
__device__ __forceinline__ bool finish_segment(const TcParams& P, Epilogue& E, uint32_t d_addr, int tile, int r, bool whole, bool first_of_range,
                                               int total, int ctas, int n_stages, uint32_t release_bar) {
  constexpr int kAct = TcFmt<F>::kAct;
  const int n = tile * kBM + r;
  const int Mp = P.Mp, chunks = Mp / 8;
  float rf = 1.0f, bias = 0.0f;
  if (n < P.N) {
    if constexpr (F == LX_W_INT8 || F == LX_W_FP8) rf = reinterpret_cast<const float*>(P.scale)[n];
    if constexpr (F == LX_W_NVFP4) rf = P.global;
    if (P.bias) bias = load_f32(P.bias, P.bias_dtype, n);
  }
  auto release = [&]() {
    tc_fence_before();
    __syncwarp();
    if (release_bar && E.lane == 0) mbar_arrive(release_bar);
  };
  auto slot_of = [&](int b) {
    return P.partials + (2 * static_cast<size_t>(b) + (range_begin(total, ctas, b) / n_stages == tile ? 0 : 1)) * (kBM * P.NC);
  };
  uint32_t raw[3][8];
  if (whole) {
    for (int c = E.chunk0; c < chunks; c += E.chunk_step) {
#pragma unroll
      for (int p = 0; p < 3; ++p)
        if (p < P.planes) tmem_ld8(d_addr + p * Mp + c * 8, raw[p]);
      tmem_wait_ld();
      if (c + E.chunk_step >= chunks) release();
      combine_and_store<kAct>(P, raw, c * 8, n, rf, bias);
    }
    if (E.chunk0 >= chunks) release();
    return true;
  }
  const int me = blockIdx.x;
  const int b_lo = owner_of(total, ctas, tile * n_stages), b_hi = owner_of(total, ctas, tile * n_stages + n_stages - 1);
  // Have all the others counted themselves already?
  volatile int* flag = E.flags + (E.meetings & 1);
  if (E.leader) *flag = ld_acquire(P.counters + b_lo) == b_hi - b_lo ? 1 : 0;
  if (!E.meet(P.status)) return false;
  if (*flag) {
    __threadfence();
    for (int c = E.chunk0; c < chunks; c += E.chunk_step) {
      uint32_t own[3][8];
#pragma unroll
      for (int p = 0; p < 3; ++p)
        if (p < P.planes) tmem_ld8(d_addr + p * Mp + c * 8, own[p]);
      bool started = false;
      for (int b = b_lo; b <= b_hi; ++b) {
        uint32_t part[3][8];
        if (b == me) {
          tmem_wait_ld();
          if (c + E.chunk_step >= chunks) release();
#pragma unroll
          for (int p = 0; p < 3; ++p)
#pragma unroll
            for (int j = 0; j < 8; ++j) part[p][j] = own[p][j];
        } else {
          uint32_t* theirs = slot_of(b);
#pragma unroll
          for (int p = 0; p < 3; ++p) {
            if (p >= P.planes) break;
            const uint4 lo = ld_cg_u128(partial_at(theirs, p * Mp + c * 8, r)), hi = ld_cg_u128(partial_at(theirs, p * Mp + c * 8 + 4, r));
            part[p][0] = lo.x, part[p][1] = lo.y, part[p][2] = lo.z, part[p][3] = lo.w;
            part[p][4] = hi.x, part[p][5] = hi.y, part[p][6] = hi.z, part[p][7] = hi.w;
          }
        }
#pragma unroll
        for (int p = 0; p < 3; ++p)
#pragma unroll
          for (int j = 0; j < 8; ++j) raw[p][j] = started ? add_raw<kAct>(raw[p][j], part[p][j]) : add_raw<kAct>(0u, part[p][j]);
        started = true;
      }
      combine_and_store<kAct>(P, raw, c * 8, n, rf, bias);
    }
    if (E.chunk0 >= chunks) release();
    return true;
  }
  // Not the last one (as far as it could tell): the partial goes to this CTA's slot (0 when the segment is the first
  // of its range, else 1), then the CTA counts itself.
  uint32_t* mine = P.partials + (2 * static_cast<size_t>(me) + (first_of_range ? 0 : 1)) * (kBM * P.NC);
  for (int c = E.chunk0; c < chunks; c += E.chunk_step) {
#pragma unroll
    for (int p = 0; p < 3; ++p)
      if (p < P.planes) tmem_ld8(d_addr + p * Mp + c * 8, raw[p]);
    tmem_wait_ld();
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      if (p >= P.planes) break;
      *reinterpret_cast<uint4*>(partial_at(mine, p * Mp + c * 8, r)) = make_uint4(raw[p][0], raw[p][1], raw[p][2], raw[p][3]);
      *reinterpret_cast<uint4*>(partial_at(mine, p * Mp + c * 8 + 4, r)) = make_uint4(raw[p][4], raw[p][5], raw[p][6], raw[p][7]);
    }
  }
  release();
  __threadfence();
  if (!E.meet(P.status)) return false;
  flag = E.flags + (E.meetings & 1);
  if (E.leader) *flag = atomicAdd(P.counters + b_lo, 1) == b_hi - b_lo ? 1 : 0;
  if (!E.meet(P.status)) return false;
  if (!*flag) return true;
  // The others arrived in between: every part is in the workspace now, this CTA's too.
  __threadfence();
  for (int c = E.chunk0; c < chunks; c += E.chunk_step) {
    for (int b = b_lo; b <= b_hi; ++b) {
      uint32_t* theirs = slot_of(b);
#pragma unroll
      for (int p = 0; p < 3; ++p) {
        if (p >= P.planes) break;
        const uint4 lo = ld_cg_u128(partial_at(theirs, p * Mp + c * 8, r)), hi = ld_cg_u128(partial_at(theirs, p * Mp + c * 8 + 4, r));
        const uint32_t part[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) raw[p][j] = b == b_lo ? add_raw<kAct>(0u, part[j]) : add_raw<kAct>(raw[p][j], part[j]);
      }
    }
    combine_and_store<kAct>(P, raw, c * 8, n, rf, bias);
  }
  return true;
}

// ---- BF16 / FP8 / INT8: weights go from shared memory straight into the tensor core ------------------------------------
constexpr int kDirectThreads = 192;   // warps 0-3 epilogue, warp 4 producers, warp 5 MMA issuer
constexpr int kDBufColumns = 256;     // two accumulators, 256 TMEM columns apart

template <int F>
__global__ void __launch_bounds__(kDirectThreads, 1) tc_direct_kernel(const __grid_constant__ CUtensorMap wmap, const TcParams P) {
  using Fm = TcFmt<F>;
  constexpr int kAct = Fm::kAct;
  constexpr int kWStage = kBM * Fm::kRowBytes;   // weight bytes per stage, a multiple of 1024
  constexpr int kBoxes = Fm::kRowBytes / 128;    // 128-byte-wide tile copies per stage
  extern __shared__ __align__(1024) uint8_t smem[];
  const int NC = P.NC, SW = P.SW, SX = P.SX;
  const int x_bytes = P.x_bytes;
  uint8_t* const xring = smem + static_cast<size_t>(SW) * kWStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(xring + static_cast<size_t>(SX) * x_bytes);
  const uint32_t bar0 = smem_u32(bars);
  auto w_full = [&](int s) { return bar0 + 8u * s; };                     // weight stage landed
  auto w_empty = [&](int s) { return bar0 + 8u * (SW + s); };             // its products are done
  auto x_full = [&](int s) { return bar0 + 8u * (2 * SW + s); };          // activation block landed
  auto x_empty = [&](int s) { return bar0 + 8u * (2 * SW + SX + s); };    // its products are done
  auto d_full = [&](int b) { return bar0 + 8u * (2 * SW + 2 * SX + b); };       // accumulator b is complete
  auto d_empty = [&](int b) { return bar0 + 8u * (2 * SW + 2 * SX + 2 + b); };  // accumulator b has been read
  const uint32_t group_bar = bar0 + 8u * (2 * SW + 2 * SX + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SW + 2 * SX + 5);
  int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_stages = (P.K + kKS - 1) / kKS;
  const int n_tiles = (P.N + kBM - 1) / kBM;
  const int total = n_tiles * n_stages, ctas = gridDim.x;
  const int g_begin = range_begin(total, ctas, blockIdx.x), g_end = range_begin(total, ctas, blockIdx.x + 1);

  if (tid == 0) {
    for (int s = 0; s < SW; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), 1);
    }
    for (int s = 0; s < SX; ++s) {
      mbar_init(x_full(s), 1);
      mbar_init(x_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(d_full(b), 1);
      mbar_init(d_empty(b), 4);
    }
    mbar_init(group_bar, 4);
    mbar_init_fence();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(tmem_slot), kTmemColumns);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ================================ producers ================================
    pdl_trigger();
    if (lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
    // Everything earlier in the stream is complete after this: the preparation kernel (activations, counters) and
    // whatever wrote the weights before it.
    pdl_wait();
    if (lane == 0) {
      for (int g = g_begin; g < g_end; ++g) {
        const int i = g - g_begin, slot = i % SW;
        const int tile = g / n_stages, s = g % n_stages;
        if (i >= SW && !tc_wait(w_empty(slot), ((i / SW) - 1) & 1, P.status)) break;
        const uint32_t dst = smem_u32(smem) + static_cast<uint32_t>(slot) * kWStage;
        mbar_arrive_expect_tx(w_full(slot), kWStage);
#pragma unroll
        for (int b = 0; b < kBoxes; ++b)
          tile_g2s(dst + b * (kBM * 128), &wmap, (s * Fm::kRowBytes + b * 128) / 4, tile * kBM, w_full(slot));
      }
    } else if (lane == 1) {
      for (int g = g_begin; g < g_end; ++g) {
        const int i = g - g_begin, slot = i % SX;
        if (i >= SX && !tc_wait(x_empty(slot), ((i / SX) - 1) & 1, P.status)) break;
        mbar_arrive_expect_tx(x_full(slot), x_bytes);
        bulk_g2s(smem_u32(xring) + static_cast<uint32_t>(slot) * x_bytes, P.xprep + static_cast<size_t>(g % n_stages) * x_bytes, x_bytes,
                 x_full(slot));
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      // c format (f32 = 1, s32 = 2), a / b format (bf16 = 1 in kind::f16, e4m3 = 0 in kind::f8f6f4, signed = 1 in
      // kind::i8), both operands K-major, N / 8, M / 16
      const uint32_t cfmt = kAct == kActS8 ? 2u : 1u, abfmt = kAct == kActE4m3 ? 0u : 1u;
      const uint32_t idesc = (cfmt << 4) | (abfmt << 7) | (abfmt << 10) | (static_cast<uint32_t>(NC >> 3) << 17) |
                             (static_cast<uint32_t>(kBM >> 4) << 24);
      const uint32_t lbo = static_cast<uint32_t>(NC / 8) * 128, sbo = 128;
      int seg = 0;
      uint32_t d_tmem = tmem_base;
      for (int g = g_begin; g < g_end; ++g) {
        const int i = g - g_begin, slot = i % SW, xs = i % SX;
        const int s = g % n_stages;
        const bool first = (g == g_begin) || s == 0;  // the first stage of a segment starts the sum anew
        if (first) {
          d_tmem = tmem_base + (seg & 1) * kDBufColumns;
          if (seg >= 2) {  // the epilogue of the segment before last has read this accumulator
            if (!tc_wait(d_empty(seg & 1), ((seg >> 1) - 1) & 1, P.status)) break;
            tc_fence_after();
          }
        }
        if (!tc_wait(w_full(slot), (i / SW) & 1, P.status) || !tc_wait(x_full(xs), (i / SX) & 1, P.status)) break;
        tc_fence_after();
        const uint32_t wb = smem_u32(smem) + static_cast<uint32_t>(slot) * kWStage;
        const uint32_t xb = smem_u32(xring) + static_cast<uint32_t>(xs) * x_bytes;
#pragma unroll
        for (int b = 0; b < kBoxes; ++b) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const int c = b * 4 + ks;  // 32 bytes of K per instruction
            const uint64_t adesc = smem_desc_sw128(wb + b * (kBM * 128) + ks * 32);
            const uint64_t bdesc = smem_desc(xb + static_cast<uint32_t>(2 * c) * lbo, lbo, sbo);
            umma_ss<kAct>(d_tmem, adesc, bdesc, idesc, (!first || c) ? 1u : 0u);
          }
        }
        umma_commit(w_empty(slot));
        umma_commit(x_empty(xs));
        if (s == n_stages - 1 || g == g_end - 1) {
          umma_commit(d_full(seg & 1));
          ++seg;
        }
      }
    }
  } else {
    // ================================ epilogue ================================
    const int r = tid;  // weight row of the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    Epilogue E{group_bar, 4, 0, last_flag, tid == 0, lane, 0, 1};
    int seg = 0;
    for (int g = g_begin; g < g_end; ++seg) {
      const int tile = g / n_stages;
      const int seg_end = min(g_end, (tile + 1) * n_stages);
      if (!tc_wait(d_full(seg & 1), (seg >> 1) & 1, P.status)) break;
      tc_fence_after();
      pdl_wait();  // bias, y and the activation scales may come from earlier kernels
      const bool whole = g == tile * n_stages && seg_end == (tile + 1) * n_stages;
      if (!finish_segment<F>(P, E, lane_addr + (seg & 1) * kDBufColumns, tile, r, whole, g == g_begin, total, ctas, n_stages, d_empty(seg & 1)))
        break;
      g = seg_end;
    }
  }
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, kTmemColumns);
}

// ---- NVFP4: converter warps expand the stage into tensor memory ---------------------------------------------------------
constexpr int kChunks = kKS / 16;  // tcgen05.mma instructions per stage (K = 16 each)
constexpr int kASlots = 3;         // A-operand slots in TMEM, one stage each (kKS / 2 columns)
constexpr int kAColumns = kKS / 2;
constexpr int kDColumn = kASlots * kAColumns;  // the accumulator's first TMEM column (128 columns remain for it)
constexpr int kConvWarps = 8, kConvThreads = 320;  // warps 0-7 convert, warp 8 produces, warp 9 issues

__global__ void __launch_bounds__(kConvThreads, 1)
    tc_nvfp4_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap, const TcParams P) {
  constexpr int F = LX_W_NVFP4;
  using Fm = TcFmt<F>;
  constexpr int kRawBytes = kBM * Fm::kRowBytes;   // weight bytes per stage: one 128-byte-wide box
  constexpr int kScaleBytes = kBM * 16;            // 16 block scales per row per stage
  constexpr int kWStage = kRawBytes + kScaleBytes; // a multiple of 1024
  extern __shared__ __align__(1024) uint8_t smem[];
  const int NC = P.NC, SW = P.SW, SX = P.SX;
  const int x_bytes = P.x_bytes;
  uint8_t* const xring = smem + static_cast<size_t>(SW) * kWStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(xring + static_cast<size_t>(SX) * x_bytes);
  const uint32_t bar0 = smem_u32(bars);
  auto w_full = [&](int s) { return bar0 + 8u * s; };                               // weight stage landed
  auto w_empty = [&](int s) { return bar0 + 8u * (SW + s); };                       // read by all converter warps
  auto x_full = [&](int s) { return bar0 + 8u * (2 * SW + s); };                    // activation block landed
  auto x_empty = [&](int s) { return bar0 + 8u * (2 * SW + SX + s); };              // its products are done
  auto a_full = [&](int a) { return bar0 + 8u * (2 * SW + 2 * SX + a); };           // A slot written
  auto a_empty = [&](int a) { return bar0 + 8u * (2 * SW + 2 * SX + kASlots + a); };// A slot consumed
  const uint32_t d_full = bar0 + 8u * (2 * SW + 2 * SX + 2 * kASlots);              // the segment's accumulator is complete
  const uint32_t group_bar = d_full + 8u;                                           // the converter warps meet here
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SW + 2 * SX + 2 * kASlots + 2);
  int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_stages = (P.K + kKS - 1) / kKS;
  const int n_tiles = (P.N + kBM - 1) / kBM;
  const int total = n_tiles * n_stages, ctas = gridDim.x;
  const int g_begin = range_begin(total, ctas, blockIdx.x), g_end = range_begin(total, ctas, blockIdx.x + 1);

  if (tid == 0) {
    for (int s = 0; s < SW; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), kConvWarps);
    }
    for (int s = 0; s < SX; ++s) {
      mbar_init(x_full(s), 1);
      mbar_init(x_empty(s), 1);
    }
    for (int a = 0; a < kASlots; ++a) {
      mbar_init(a_full(a), kConvWarps);
      mbar_init(a_empty(a), 1);
    }
    mbar_init(d_full, 1);
    mbar_init(group_bar, kConvWarps);
    mbar_init_fence();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), kTmemColumns);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ================================ producers ================================
    pdl_trigger();
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&smap) : "memory");
    }
    pdl_wait();  // everything earlier in the stream is complete: prepared activations, counters, weights
    if (lane == 0) {
      for (int g = g_begin; g < g_end; ++g) {
        const int i = g - g_begin, slot = i % SW;
        const int tile = g / n_stages, s = g % n_stages;
        if (i >= SW && !tc_wait(w_empty(slot), ((i / SW) - 1) & 1, P.status)) break;
        const uint32_t dst = smem_u32(smem) + static_cast<uint32_t>(slot) * kWStage;
        mbar_arrive_expect_tx(w_full(slot), kWStage);
        tile_g2s(dst, &wmap, (s * Fm::kRowBytes) / 4, tile * kBM, w_full(slot));
        tile_g2s(dst + kRawBytes, &smap, s * 16, tile * kBM, w_full(slot));
      }
    } else if (lane == 1) {
      for (int g = g_begin; g < g_end; ++g) {
        const int i = g - g_begin, slot = i % SX;
        if (i >= SX && !tc_wait(x_empty(slot), ((i / SX) - 1) & 1, P.status)) break;
        mbar_arrive_expect_tx(x_full(slot), x_bytes);
        bulk_g2s(smem_u32(xring) + static_cast<uint32_t>(slot) * x_bytes, P.xprep + static_cast<size_t>(g % n_stages) * x_bytes, x_bytes,
                 x_full(slot));
      }
    }
  } else if (warp == 9) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(NC >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);  // f16 x f16 -> f32
      const uint32_t lbo = static_cast<uint32_t>(NC / 8) * 128, sbo = 128;
      for (int g = g_begin; g < g_end; ++g) {
        const int i = g - g_begin, xs = i % SX, a = i % kASlots;
        const int s = g % n_stages;
        // the activations of this stage are in shared memory, the converted weights in tensor memory
        if (!tc_wait(x_full(xs), (i / SX) & 1, P.status) || !tc_wait(a_full(a), (i / kASlots) & 1, P.status)) break;
        tc_fence_after();
        const uint32_t xb = smem_u32(xring) + static_cast<uint32_t>(xs) * x_bytes;
        const bool first = (g == g_begin) || s == 0;  // the first stage of a segment starts the sum anew
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          const uint64_t bdesc = smem_desc(xb + static_cast<uint32_t>(2 * c) * lbo, lbo, sbo);
          umma_ts(tmem_base + kDColumn, tmem_base + a * kAColumns + c * 8, bdesc, idesc, (!first || c) ? 1u : 0u);
        }
        umma_commit(a_empty(a));    // the A slot may be overwritten once these products are done
        umma_commit(x_empty(xs));   // and so may the activation block
        // A segment ends here: its accumulator is complete when everything issued so far is. The next segment's first
        // product overwrites it, but waits for an A slot the converters fill only after they have read the accumulator.
        if (s == n_stages - 1 || g == g_end - 1) umma_commit(d_full);
      }
    }
  } else {
    // ================================ converters, then epilogue ================================
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;  // weight row of the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    Epilogue E{group_bar, kConvWarps, 0, last_flag, tid == 0, lane, half, 2};
    int segment = 0;
    for (int g = g_begin; g < g_end; ++g) {
      const int i = g - g_begin, slot = i % SW, a = i % kASlots;
      const int tile = g / n_stages, s = g % n_stages;
      if (!tc_wait(w_full(slot), (i / SW) & 1, P.status) || (i >= kASlots && !tc_wait(a_empty(a), ((i / kASlots) - 1) & 1, P.status))) break;
      tc_fence_after();
      const uint8_t* stage = smem + static_cast<size_t>(slot) * kWStage;
      const uint32_t a_addr = lane_addr + a * kAColumns + half * (kAColumns / 2);
      const int sw = r & 7;
      // this half's 128 values = 64 bytes = pieces 4 half .. 4 half + 3 of the row's 128 bytes; 8 block scales
      const uint8_t* box = stage + r * 128;
      uint4 q[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = *reinterpret_cast<const uint4*>(box + (((4 * half + j) ^ sw) << 4));
      const uint2 sc = *reinterpret_cast<const uint2*>(stage + kRawBytes + r * 16 + half * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t p[8];
        const uint32_t sword = j < 2 ? sc.x : sc.y;
        expand_nvfp4(q[j].x, q[j].y, sword >> (16 * (j & 1)), p);
        tmem_st8(a_addr + (2 * j) * 8, p);
        expand_nvfp4(q[j].z, q[j].w, sword >> (16 * (j & 1) + 8), p);
        tmem_st8(a_addr + (2 * j + 1) * 8, p);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(w_empty(slot));  // the bytes are in registers / tensor memory: the stage may be refilled
        mbar_arrive(a_full(a));
      }
      if (s != n_stages - 1 && g != g_end - 1) continue;
      // ---- the segment is over ----
      if (!tc_wait(d_full, segment & 1, P.status)) break;
      ++segment;
      tc_fence_after();
      pdl_wait();  // bias, y and the activation scales may come from earlier kernels
      const int seg_first = max(g_begin, tile * n_stages);  // the segment is stages seg_first .. g of the tile
      const bool whole = seg_first == tile * n_stages && s == n_stages - 1;
      if (!finish_segment<F>(P, E, lane_addr + kDColumn, tile, r, whole, seg_first == g_begin, total, ctas, n_stages, 0u)) break;
    }
  }
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, kTmemColumns);
}

// ---- launching -------------------------------------------------------------------------------------------------------
int sm_count() {
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
    done[dev] = true;
  }
  return kOk;
}

template <int F>
int tc_launch(const lx_weight& w, TcParams P, cudaStream_t stream) {
  using Fm = TcFmt<F>;
  constexpr int kWStage = kBM * Fm::kRowBytes + (F == LX_W_NVFP4 ? kBM * 16 : 0);
  constexpr int kBudget = 220 * 1024;
  P.SX = P.x_bytes > 24 * 1024 ? 2 : 3;
  P.SW = std::min(8, (kBudget - P.SX * P.x_bytes) / kWStage);
  if (P.SW < 2) return kNotSupported;
  const int sms = sm_count();
  if (!sms) return kInvalid;
  // Tensor memory is taken whole (512 columns), so exactly one CTA may live on an SM: ask for more than half of its
  // shared memory whatever the rings need.
  const size_t smem = std::max<size_t>(static_cast<size_t>(P.SW) * kWStage + static_cast<size_t>(P.SX) * P.x_bytes + 1024, 120 * 1024);
  alignas(64) CUtensorMap wmap, smap;
  memset(&wmap, 0, sizeof(wmap));
  memset(&smap, 0, sizeof(smap));
  const int64_t row_bytes = F == LX_W_BF16 ? 2ll * P.K : F == LX_W_NVFP4 ? P.K / 2 : P.K;
  if (int e = make_tile_map(&wmap, w.data, row_bytes, P.N, 128, kBM, 4, true)) return e;
  const int tiles = (P.N + kBM - 1) / kBM, n_stages = (P.K + kKS - 1) / kKS;
  const int total = tiles * n_stages;
  const int grid = std::min(total, std::max(1, std::min({sms, kMaxCtas, std::max(tiles, total / kMinStagesPerCta)})));
  if constexpr (F == LX_W_NVFP4) {
    if (int e = make_tile_map(&smap, w.scale, P.K / 16, P.N, 16, kBM, 1, false)) return e;
    if (int e = allow_big_smem<F>(tc_nvfp4_kernel)) return e;
    return launch_kernel(tc_nvfp4_kernel, dim3(grid), dim3(kConvThreads), smem, stream, wmap, smap, P);
  } else {
    if (int e = allow_big_smem<F>(tc_direct_kernel<F>)) return e;
    return launch_kernel(tc_direct_kernel<F>, dim3(grid), dim3(kDirectThreads), smem, stream, wmap, P);
  }
}

int act_of(int wtype) {
  return wtype == LX_W_BF16 ? kActBf16 : wtype == LX_W_INT8 ? kActS8 : wtype == LX_W_FP8 ? kActE4m3 : kActF16;
}
// Activation rows one pass takes: the block of one stage stays within 48 KB.
int rows_per_pass(int act, bool x_bf16) { return (act == kActBf16 && !x_bf16) ? 32 : kMaxRows; }

}  // namespace

// The product, in passes of at most 64 activation rows. workspace: at least tc_workspace_bytes.
int tc_product(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype, void* y, int y_dtype,
               int ld_y, int M, int N, int K, float alpha, float beta, void* workspace, cudaStream_t stream) {
  const bool x_bf16 = x_dtype == LX_BF16;
  const int act = act_of(w.type), elem = act_elem(act);
  const int per_pass = rows_per_pass(act, x_bf16);
  const int n_stages = (K + kKS - 1) / kKS;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  for (int m0 = 0; m0 < M; m0 += per_pass) {
    const int rows = std::min(per_pass, M - m0);
    TcParams P{};
    P.scale = static_cast<const uint8_t*>(w.scale);
    P.global = w.global;
    P.N = N, P.K = K, P.M = rows;
    P.planes = act_planes(act, x_bf16);
    P.digit = act == kActS8 ? 0.0078125f : act == kActE4m3 ? 0.0625f : 1.0f;
    P.Mp = (rows + 7) / 8 * 8;
    P.NC = (P.planes * P.Mp + 15) / 16 * 16;
    P.x_bytes = P.NC * kKS * elem;
    const TcLayout L(P.NC, elem, n_stages);
    P.xprep = ws;
    P.inv_scales = reinterpret_cast<const float*>(ws + L.scales);
    P.counters = reinterpret_cast<int*>(ws + L.counters);
    P.partials = reinterpret_cast<uint32_t*>(ws + L.partials);
    P.bias = bias, P.bias_dtype = bias_dtype;
    P.y = static_cast<uint8_t*>(y) + static_cast<int64_t>(m0) * ld_y * (y_dtype == LX_BF16 ? 2 : 4);
    P.y_dtype = y_dtype, P.ld_y = ld_y;
    P.alpha = alpha, P.beta = beta;
    P.status = status_word();
    const uint8_t* xrow = static_cast<const uint8_t*>(x) + static_cast<int64_t>(m0) * ld_x * (x_bf16 ? 2 : 4);
    const int per_block = 128 * 16 / elem;
    const dim3 prep_grid((n_stages * kKS + per_block - 1) / per_block, rows);
    auto prep = [&](auto kernel) {
      return launch_kernel(kernel, prep_grid, dim3(128), 0, stream, static_cast<const void*>(xrow), ld_x, rows, K, P.NC, P.Mp, P.planes, ws,
                           reinterpret_cast<float*>(ws + L.scales), reinterpret_cast<int*>(ws + L.counters), n_stages);
    };
    int pe;
    switch (act * 2 + (x_bf16 ? 1 : 0)) {
      case kActBf16 * 2: pe = prep(tc_prep_kernel<kActBf16, false>); break;
      case kActBf16 * 2 + 1: pe = prep(tc_prep_kernel<kActBf16, true>); break;
      case kActF16 * 2: pe = prep(tc_prep_kernel<kActF16, false>); break;
      case kActF16 * 2 + 1: pe = prep(tc_prep_kernel<kActF16, true>); break;
      case kActE4m3 * 2: pe = prep(tc_prep_kernel<kActE4m3, false>); break;
      case kActE4m3 * 2 + 1: pe = prep(tc_prep_kernel<kActE4m3, true>); break;
      case kActS8 * 2: pe = prep(tc_prep_kernel<kActS8, false>); break;
      default: pe = prep(tc_prep_kernel<kActS8, true>); break;
    }
    if (pe) return pe;
    int e;
    switch (w.type) {
      case LX_W_BF16: e = tc_launch<LX_W_BF16>(w, P, stream); break;
      case LX_W_INT8: e = tc_launch<LX_W_INT8>(w, P, stream); break;
      case LX_W_FP8: e = tc_launch<LX_W_FP8>(w, P, stream); break;
      case LX_W_NVFP4: e = tc_launch<LX_W_NVFP4>(w, P, stream); break;
      default: e = kNotSupported;
    }
    if (e) return e;
  }
  return kOk;
}

// Bytes of workspace the product needs for M activation rows, whatever the weight format and activation dtype.
int64_t tc_workspace_bytes(int M, int K) {
  const int rows = std::min(M, kMaxRows);
  const int Mp = (rows + 7) / 8 * 8;
  const int64_t n_stages = (K + kKS - 1) / kKS;
  int64_t need = 0;
  for (int act = 0; act < 4; ++act)
    for (int bf = 0; bf < 2; ++bf) {
      const int r = std::min(rows, rows_per_pass(act, bf != 0));
      const int mp = std::min(Mp, (r + 7) / 8 * 8);
      const int NC = (act_planes(act, bf != 0) * mp + 15) / 16 * 16;
      need = std::max(need, TcLayout(NC, act_elem(act), n_stages).total);
    }
  return need;
}

}  // namespace b200
