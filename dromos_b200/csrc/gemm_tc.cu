// The batched-decode product on the 5th-generation tensor cores: y[m, n] = sum_k x[m, k] * w[n, k] for 9..64 activation
// rows (more rows run as passes of 64), weights streamed once in their stored format.
//
// At these row counts the product is a real contraction (up to ~1 PFLOP/s would be needed to keep up with HBM at
// M = 64), so it runs on tcgen05.mma with the accumulator in tensor memory:
//
//   D[128 weight rows, NC columns] (TMEM, f32) += A[128, 16] (TMEM, f16 or bf16) * B[16, NC] (shared memory)
//
//   * producer warp   streams 128-row x 256-value weight stages through a shared-memory ring with 2-D TMA tile copies
//                     (128-byte-swizzled boxes, no multicast), and with each stage the matching block of prepared
//                     activations (1-D bulk copy); one mbarrier per stage.
//   * converter warps four warps, thread r owns weight row r of the tile: it reads its row's bytes from the stage
//                     (conflict-free thanks to the swizzle), expands them in registers to f16 pairs (int8, e4m3 and
//                     e2m1 * e4m3 block scale are all exact in f16; bf16 weights pass through as bf16) and writes them
//                     with tcgen05.st into the A operand region of tensor memory, lane r. The weight bytes never go
//                     back to shared memory.
//   * MMA warp        one thread issues 16 tcgen05.mma per stage (K = 16 each; A from TMEM, B through a shared-memory
//                     descriptor) and commits them to the mbarrier that frees the A slot.
//   * epilogue        the converter warps read the tile's accumulator (tcgen05.ld, lane = weight row), apply the row
//                     factor, the activation scale, bias, alpha / beta and store y.
//
// Activations are prepared once per call by a small kernel into the caller's workspace: f16 after a per-row
// power-of-two scaling (bf16 as they are for bf16 weights), f32 inputs as a high and a low half in two columns, laid
// out in the K-major core-matrix order the B descriptor reads.
//
// Every wait is bounded; a wait that gives up writes a code to the status word and the kernel still frees its TMEM.
#include <algorithm>
#include <cstring>

#include "launch.cuh"

namespace b200 {
namespace {

constexpr int kBM = 128;          // weight rows per tile = TMEM lanes
constexpr int kKS = 256;          // values of K per stage
constexpr int kChunks = kKS / 16; // tcgen05.mma instructions per stage (K = 16 each)
constexpr int kASlots = 2;        // A-operand slots in TMEM, one stage each (kKS / 2 columns)
constexpr int kAColumns = kKS / 2;
constexpr int kDColumn = kASlots * kAColumns;  // the accumulator's first TMEM column
constexpr int kTmemColumns = 512;
constexpr int kConverterThreads = 128, kTcThreads = 192;  // warps 0-3 convert, warp 4 produces, warp 5 issues

constexpr int kStatusTcWait = 5;  // a bounded wait of this kernel gave up

struct TcParams {
  const uint8_t* scale;   // f32 [N] (INT8 / FP8); NVFP4 block scales come through the tensor map
  float global;
  int N, K, M;            // M: activation rows of this pass
  int NC;                 // columns (16, 32, 48 or 64): M rows, or 2 M for f32 activations
  int split;              // activations are f32: column 2 m is the high half, 2 m + 1 the low half
  const uint8_t* xprep;   // prepared activations: n_stages blocks of NC * 512 bytes, then NC f32 inverse scales
  const void* bias;
  int bias_dtype;
  void* y;
  int y_dtype, ld_y;
  float alpha, beta;
  int* status;
};

template <int F>
struct TcFmt;
template <>
struct TcFmt<LX_W_BF16> {
  static constexpr int kRowBytes = 512;  // bytes per weight row per stage
  static constexpr bool kBf16 = true;
};
template <>
struct TcFmt<LX_W_INT8> {
  static constexpr int kRowBytes = 256;
  static constexpr bool kBf16 = false;
};
template <>
struct TcFmt<LX_W_FP8> {
  static constexpr int kRowBytes = 256;
  static constexpr bool kBf16 = false;
};
template <>
struct TcFmt<LX_W_NVFP4> {
  static constexpr int kRowBytes = 128;
  static constexpr bool kBf16 = false;
};

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
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem descriptor], one CTA, f16 / bf16 operands.
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
// One CTA per activation row m: its largest magnitude, its power-of-two scale, then its values as 16-bit floats in
// the block layout of the B operand: element (column c, k) of stage s sits at
//   s * NC * 512 + ((k % 256) / 8 * (NC / 8) + c / 8) * 128 + (c % 8) * 16 + (k % 8) * 2.
// Columns past the live ones and k past K are zero (the whole buffer is cleared first by the caller's memset).
__global__ void __launch_bounds__(256) tc_prep_kernel(const void* __restrict__ x, int x_dtype, int ld_x, int M, int K, int NC, int split,
                                                      int bf16_math, uint8_t* __restrict__ out, int n_stages) {
  pdl_trigger();
  pdl_wait();
  __shared__ float part[8];
  const int m = blockIdx.x;
  float* inv_scales = reinterpret_cast<float*>(out + static_cast<size_t>(n_stages) * NC * 512);
  float sc = 1.0f;
  if (!bf16_math) {
    float a = 0.0f;
    for (int k = threadIdx.x; k < K; k += 256) a = fmaxf(a, fabsf(load_f32(x, x_dtype, static_cast<int64_t>(m) * ld_x + k)));
    a = warp_max(a);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = a;
    __syncthreads();
    a = 0.0f;
    for (int i = 0; i < 8; ++i) a = fmaxf(a, part[i]);
    int ex = static_cast<int>((__float_as_uint(a) >> 23) & 0xffu);
    ex = a > 0.0f ? min(max(ex, 30), 230) : 141;
    sc = __uint_as_float(static_cast<uint32_t>(268 - ex) << 23);  // largest magnitude into [2^14, 2^15)
  }
  const int ncols = split ? 2 : 1;
  if (threadIdx.x < ncols) inv_scales[m * ncols + threadIdx.x] = 1.0f / sc;
  for (int k = threadIdx.x; k < K; k += 256) {
    const float v = load_f32(x, x_dtype, static_cast<int64_t>(m) * ld_x + k) * sc;
    uint16_t hi, lo = 0;
    if (bf16_math) {
      hi = static_cast<uint16_t>(f32_to_bf16_bits(v));
      if (split) lo = static_cast<uint16_t>(f32_to_bf16_bits(v - bf16_bits_to_f32(hi)));
    } else {
      const __half h = __float2half_rn(v);
      hi = __half_as_ushort(h);
      if (split) lo = __half_as_ushort(__float2half_rn(v - __half2float(h)));
    }
    const int s = k / kKS, kin = k % kKS;
    for (int t = 0; t < ncols; ++t) {
      const int c = m * ncols + t;
      const size_t at = static_cast<size_t>(s) * NC * 512 + (static_cast<size_t>(kin / 8) * (NC / 8) + c / 8) * 128 + (c % 8) * 16 +
                        (kin % 8) * 2;
      *reinterpret_cast<uint16_t*>(out + at) = t ? lo : hi;
    }
  }
}

// ---- expanding 16 weight values to eight 16-bit pairs ---------------------------------------------------------------
__device__ __forceinline__ void expand_fp8(uint4 q, uint32_t (&p)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.rn.f16x2.e4m3x2 %0, lo; cvt.rn.f16x2.e4m3x2 %1, hi; }"
        : "=r"(p[2 * i]), "=r"(p[2 * i + 1])
        : "r"(w[i]));
  }
}
__device__ __forceinline__ void expand_int8(uint4 q, uint32_t (&p)[8]) {
  // (v ^ 0x80) is v + 128; 0x6400 | u is the f16 1024 + u; minus 1152 leaves v exactly
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t u = w[i] ^ 0x80808080u;
    uint32_t lo = __byte_perm(u, 0x64646464u, 0x5140), hi = __byte_perm(u, 0x64646464u, 0x5342);
    asm("sub.rn.f16x2 %0, %0, %1;" : "+r"(lo) : "r"(0x64806480u));
    asm("sub.rn.f16x2 %0, %0, %1;" : "+r"(hi) : "r"(0x64806480u));
    p[2 * i] = lo, p[2 * i + 1] = hi;
  }
}
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

template <int F>
constexpr int tc_stage_bytes(int NC) {
  return kBM * TcFmt<F>::kRowBytes + (F == LX_W_NVFP4 ? kBM * 16 : 0) + NC * 512;
}

template <int F>
__global__ void __launch_bounds__(kTcThreads, 1)
    tc_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap, const TcParams P, int S) {
  using Fm = TcFmt<F>;
  constexpr int kRawBytes = kBM * Fm::kRowBytes;           // weight bytes per stage
  constexpr int kBoxes = Fm::kRowBytes / 128;              // 128-byte-wide tile copies per stage
  constexpr int kScaleBytes = F == LX_W_NVFP4 ? kBM * 16 : 0;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int NC = P.NC;
  const int x_bytes = NC * 512;
  const int stage_bytes = kRawBytes + kScaleBytes + x_bytes;  // a multiple of 1024 (every part is)
  // barriers live after the ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(S) * stage_bytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 2 * kASlots + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };                        // stage landed (TMA bytes)
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };                 // stage read (converters and MMA done with it)
  auto a_full = [&](int a) { return bar0 + 8u * (2 * S + a); };                // A slot written (4 converter warps)
  auto a_empty = [&](int a) { return bar0 + 8u * (2 * S + kASlots + a); };     // A slot consumed (tcgen05.commit)
  const uint32_t d_full = bar0 + 8u * (2 * S + 2 * kASlots);                   // the tile's accumulator is complete

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_stages = (P.K + kKS - 1) / kKS;
  const int n_tiles = (P.N + kBM - 1) / kBM;
  const int tile_begin = static_cast<int>(static_cast<int64_t>(n_tiles) * blockIdx.x / gridDim.x);
  const int tile_end = static_cast<int>(static_cast<int64_t>(n_tiles) * (blockIdx.x + 1) / gridDim.x);

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 5);  // four converter warps + the commit of the stage's products
    }
    for (int a = 0; a < kASlots; ++a) {
      mbar_init(a_full(a), 4);
      mbar_init(a_empty(a), 1);
    }
    mbar_init(d_full, 1);
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
    // ================================ producer ================================
    pdl_trigger();
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
      pdl_wait();  // the prepared activations come from the kernel before this one
      int gs = 0;
      bool ok = true;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        for (int s = 0; s < n_stages && ok; ++s, ++gs) {
          const int slot = gs % S;
          if (gs >= S && !tc_wait(empty_bar(slot), ((gs / S) - 1) & 1, P.status)) {
            ok = false;
            break;
          }
          const uint32_t dst = smem_u32(smem) + static_cast<uint32_t>(slot) * stage_bytes;
          mbar_arrive_expect_tx(full_bar(slot), stage_bytes);
#pragma unroll
          for (int b = 0; b < kBoxes; ++b)
            tile_g2s(dst + b * (kBM * 128), &wmap, (s * Fm::kRowBytes + b * 128) / 4, tile * kBM, full_bar(slot));
          if constexpr (F == LX_W_NVFP4) tile_g2s(dst + kRawBytes, &smap, s * 16, tile * kBM, full_bar(slot));
          bulk_g2s(dst + kRawBytes + kScaleBytes, P.xprep + static_cast<size_t>(s) * x_bytes, x_bytes, full_bar(slot));
        }
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t fmt = Fm::kBf16 ? 1u : 0u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(NC >> 3) << 17) |
                             (static_cast<uint32_t>(kBM >> 4) << 24);
      const uint32_t lbo = static_cast<uint32_t>(NC / 8) * 128, sbo = 128;
      int gs = 0;
      bool ok = true;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        for (int s = 0; s < n_stages && ok; ++s, ++gs) {
          const int slot = gs % S, a = gs % kASlots;
          // the activations of this stage are in shared memory, the converted weights in tensor memory
          if (!tc_wait(full_bar(slot), (gs / S) & 1, P.status) || !tc_wait(a_full(a), (gs / kASlots) & 1, P.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t xb = smem_u32(smem) + static_cast<uint32_t>(slot) * stage_bytes + kRawBytes + kScaleBytes;
#pragma unroll
          for (int c = 0; c < kChunks; ++c) {
            const uint64_t bdesc = smem_desc(xb + static_cast<uint32_t>(2 * c) * lbo, lbo, sbo);
            umma_ts(tmem_base + kDColumn, tmem_base + a * kAColumns + c * 8, bdesc, idesc, (s | c) ? 1u : 0u);
          }
          umma_commit(a_empty(a));        // the A slot may be overwritten once these products are done
          umma_commit(empty_bar(slot));   // and so may the stage (its activations)
        }
        // The tile's accumulator is complete when everything issued so far is. The next tile's first product (which
        // overwrites it) waits for that tile's first A slot, and the converters write it only after their epilogue.
        umma_commit(d_full);
      }
    }
  } else {
    // ================================ converters, then epilogue ================================
    const int r = tid;  // weight row of the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float* inv_scales = reinterpret_cast<const float*>(P.xprep + static_cast<size_t>(n_stages) * x_bytes);
    pdl_wait();
    int gs = 0;
    bool ok = true;
    for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
      for (int s = 0; s < n_stages && ok; ++s, ++gs) {
        const int slot = gs % S, a = gs % kASlots;
        if (!tc_wait(full_bar(slot), (gs / S) & 1, P.status) ||
            (gs >= kASlots && !tc_wait(a_empty(a), ((gs / kASlots) - 1) & 1, P.status))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint8_t* stage = smem + static_cast<size_t>(slot) * stage_bytes;
        const uint32_t a_addr = lane_addr + a * kAColumns;
        uint4 scales = make_uint4(0, 0, 0, 0);
        if constexpr (F == LX_W_NVFP4) scales = *reinterpret_cast<const uint4*>(stage + kRawBytes + r * 16);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          uint32_t p[8];
          if constexpr (F == LX_W_BF16) {
            // 16 values = 32 bytes = two 16-byte pieces of box c / 4
            const uint8_t* box = stage + (c / 4) * (kBM * 128) + r * 128;
            const int piece = (c % 4) * 2;
            const uint4 q0 = *reinterpret_cast<const uint4*>(box + (((piece) ^ (r & 7)) << 4));
            const uint4 q1 = *reinterpret_cast<const uint4*>(box + (((piece + 1) ^ (r & 7)) << 4));
            p[0] = q0.x, p[1] = q0.y, p[2] = q0.z, p[3] = q0.w, p[4] = q1.x, p[5] = q1.y, p[6] = q1.z, p[7] = q1.w;
          } else if constexpr (F == LX_W_NVFP4) {
            // 16 values = 8 bytes = half of piece c / 2 of the single box
            const uint8_t* box = stage + r * 128;
            const uint2 q = *reinterpret_cast<const uint2*>(box + ((((c / 2)) ^ (r & 7)) << 4) + (c & 1) * 8);
            const uint32_t sw[4] = {scales.x, scales.y, scales.z, scales.w};
            expand_nvfp4(q.x, q.y, sw[c / 4] >> (8 * (c % 4)), p);
          } else {
            const uint8_t* box = stage + (c / 8) * (kBM * 128) + r * 128;
            const uint4 q = *reinterpret_cast<const uint4*>(box + (((c % 8) ^ (r & 7)) << 4));
            if constexpr (F == LX_W_FP8) expand_fp8(q, p);
            else expand_int8(q, p);
          }
          tmem_st8(a_addr + c * 8, p);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(a_full(a));
          mbar_arrive(empty_bar(slot));
        }
      }
      // ---- epilogue: this thread's weight row against every activation row ----
      if (!ok || !tc_wait(d_full, (tile - tile_begin) & 1, P.status)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int n = tile * kBM + r;
      float rf = 1.0f;
      if (n < P.N) {
        if constexpr (F == LX_W_INT8 || F == LX_W_FP8) rf = reinterpret_cast<const float*>(P.scale)[n];
        if constexpr (F == LX_W_NVFP4) rf = P.global;
      }
      const float bias = (P.bias && n < P.N) ? load_f32(P.bias, P.bias_dtype, n) : 0.0f;
      for (int c0 = 0; c0 < NC; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(lane_addr + kDColumn + c0, v);
        tmem_wait_ld();
        if (n < P.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int col = c0 + j;
            int m;
            float sum;
            if (P.split) {
              if (col & 1) continue;
              m = col >> 1;
              if (m >= P.M) continue;
              sum = __uint_as_float(v[j]) * inv_scales[col] + __uint_as_float(v[(j + 1) & 15]) * inv_scales[col + 1];
            } else {
              m = col;
              if (m >= P.M) continue;
              sum = __uint_as_float(v[j]) * inv_scales[col];
            }
            float t = rf * sum + bias;
            float out = P.alpha * t;
            const int64_t at = static_cast<int64_t>(m) * P.ld_y + n;
            if (P.beta != 0.0f) out = fmaf(P.beta, load_f32(P.y, P.y_dtype, at), out);
            store_from_f32(P.y, P.y_dtype, at, out);
          }
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, kTmemColumns);
}



template <int F>
int tc_launch(const lx_weight& w, TcParams P, cudaStream_t stream) {
  const int stage = tc_stage_bytes<F>(P.NC);
  int S = std::min(6, (200 * 1024) / stage);
  if (S < 2) return kNotSupported;
  // Tensor memory is taken whole (512 columns), so exactly one CTA may live on an SM: ask for more than half of its
  // shared memory whatever the ring needs.
  const size_t smem = std::max<size_t>(static_cast<size_t>(S) * stage + 256, 120 * 1024);
  auto kernel = tc_kernel<F>;
  static std::mutex mu;
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!sms[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
      int n = 0;
      if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) {
        cudaGetLastError();
        return static_cast<int>(e);
      }
      sms[dev] = n;
    }
  }
  alignas(64) CUtensorMap wmap, smap;
  memset(&wmap, 0, sizeof(wmap));
  memset(&smap, 0, sizeof(smap));
  const int64_t row_bytes = F == LX_W_BF16 ? 2ll * P.K : F == LX_W_NVFP4 ? P.K / 2 : P.K;
  if (int e = make_tile_map(&wmap, w.data, row_bytes, P.N, 128, kBM, 4, true)) return e;
  if constexpr (F == LX_W_NVFP4)
    if (int e = make_tile_map(&smap, w.scale, P.K / 16, P.N, 16, kBM, 1, false)) return e;
  const int tiles = (P.N + kBM - 1) / kBM;
  return launch_kernel(kernel, dim3(std::min(tiles, sms[dev])), dim3(kTcThreads), smem, stream, wmap, smap, P, S);
}

}  // namespace

// The product for one pass of at most 64 columns. xprep: workspace of at least tc_prep_bytes.
int tc_product(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype, void* y, int y_dtype,
               int ld_y, int M, int N, int K, float alpha, float beta, void* workspace, cudaStream_t stream) {
  const bool x_bf16 = x_dtype == LX_BF16;
  const int per_pass = x_bf16 ? 64 : 32;
  const int n_stages = (K + kKS - 1) / kKS;
  for (int m0 = 0; m0 < M; m0 += per_pass) {
    const int rows = std::min(per_pass, M - m0);
    TcParams P{};
    P.scale = static_cast<const uint8_t*>(w.scale);
    P.global = w.global;
    P.N = N, P.K = K, P.M = rows;
    P.split = x_bf16 ? 0 : 1;
    P.NC = ((x_bf16 ? rows : 2 * rows) + 15) / 16 * 16;
    P.xprep = static_cast<const uint8_t*>(workspace);
    P.bias = bias, P.bias_dtype = bias_dtype;
    P.y = static_cast<uint8_t*>(y) + static_cast<int64_t>(m0) * ld_y * (y_dtype == LX_BF16 ? 2 : 4);
    P.y_dtype = y_dtype, P.ld_y = ld_y;
    P.alpha = alpha, P.beta = beta;
    P.status = status_word();
    const size_t blocks = static_cast<size_t>(n_stages) * P.NC * 512;
    if (cudaMemsetAsync(workspace, 0, blocks + 64 * 4, stream) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    const uint8_t* xrow = static_cast<const uint8_t*>(x) + static_cast<int64_t>(m0) * ld_x * (x_bf16 ? 2 : 4);
    if (int e = launch_kernel(tc_prep_kernel, dim3(rows), dim3(256), 0, stream, static_cast<const void*>(xrow), x_dtype, ld_x, rows, K,
                              P.NC, P.split, w.type == LX_W_BF16 ? 1 : 0, static_cast<uint8_t*>(workspace), n_stages))
      return e;
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

// Bytes of prepared activations for a pass of M rows.
int64_t tc_prep_bytes(int M, int K, bool x_bf16) {
  const int cols = x_bf16 ? M : 2 * M;
  const int NC = (cols + 15) / 16 * 16;
  const int64_t n_stages = (K + kKS - 1) / kKS;
  return n_stages * NC * 512 + 64 * 4 + 256;
}

}  // namespace b200
