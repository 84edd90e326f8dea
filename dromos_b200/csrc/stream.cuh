// The weight-streaming product kernel: y[m, n] = sum_k x[m, k] * w[n, k] for a few activation rows (1..64) against
// a weight matrix that is read exactly once, at DRAM speed, in its stored format.
//
// Shape of the kernel
//   * A CTA owns R consecutive weight rows (16 * RT * WR) and all of K. Eight consumer warps and one producer warp.
//   * The producer streams the rows through a ring of S shared-memory stages with 1-D bulk copies (TMA,
//     cp.async.bulk, no multicast): one copy per row per stage (SEG contiguous bytes of that row), all of a stage's
//     copies completing on the stage's "full" mbarrier. Consumers release a stage on its "empty" mbarrier.
//   * The weight tile is the A operand of mma.sync m16n8k16 (16 weight rows x 16 k), the activations are the B
//     operand (16 k x 8 activation rows), so one instruction covers 8 activation rows and NT of them cover 8 * NT.
//     A lane takes 16 contiguous bytes of a weight row from shared memory and uses them as the k-slots the
//     instruction assigns to it; since a dot product does not care about the order of k, the activations are laid
//     out in shared memory in the matching order ("fragment order") and no weight byte is ever shuffled.
//   * Quantized weights are expanded in registers to f16 pairs (exact: int8, e4m3 and e2m1 * e4m3 all fit f16) and
//     multiplied by activations converted to f16 after a per-row power-of-two scaling (exact up to values 2^-29
//     below the row's largest); bf16 and BF16X weights go in as bf16 against the bf16 activations as they are.
//     f32 activations are split into a high and a low half (two columns), so they keep ~16 bits more than one half.
//   * WK = 8 / WR warps split the K range of every stage between them; their partial sums meet in shared memory
//     and are added in a fixed order, so results are deterministic and a row's bits do not depend on M.
//   * Every wait is bounded (common.cuh mbar_wait): a stage that never arrives ends the kernel with a status code.
#pragma once

#include <cuda.h>
#include <cuda_fp4.h>

#include "common.cuh"

namespace b200 {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = 32 * kConsumerWarps;
constexpr int kThreads = kConsumerThreads + 32;

enum StreamMode { kDense = 0, kGateUp = 1, kDown = 2 };

struct StreamParams {
  // the weight: one matrix, or a stack of experts each `N` rows
  const uint8_t* w;
  const uint8_t* scale;       // f32 [N] (INT8 / FP8) or e4m3 [N, K / 16] (NVFP4), stacked like w
  float global;               // NVFP4
  const float* expert_global; // NVFP4 stacks, or null
  int64_t row_bytes;          // bytes of one weight row (BF16X: of one record)
  int N, K;
  // the activations
  const void* x;
  int x_dtype, ld_x, M;
  int x_vec;                  // bf16 activation rows all start on 16-byte boundaries
  // dense epilogue
  const void* bias;
  int bias_dtype;
  void* y;
  int y_dtype, ld_y;
  float alpha, beta;
  // experts: grouping tables and the routed rows
  const int32_t* offsets;  // [groups + 1]: where each group's pairs start in `pairs`
  const int32_t* group_expert;  // [groups] the expert of each group, or null when group g is expert g
  const int32_t* pairs;    // [P] pair index t * top_k + k, grouped by expert
  const float* route_w;    // [P] by pair index
  int top_k, I;
  void* moe_out;           // gate_up: bf16 [P, I] in grouped order; down: f32 [P, L] by pair index
  int* status;
  int tiled;               // the weight rows come as 2-D tile copies through the tensor maps (else row by row)
};

template <int F>
struct Fmt;
template <>
struct Fmt<LX_W_BF16> {
  static constexpr bool kHalf = false;
  static constexpr int kStepValues = 32;  // values a warp step covers per row (64 bytes)
};
template <>
struct Fmt<LX_W_INT8> {
  static constexpr bool kHalf = true;
  static constexpr int kStepValues = 64;
};
template <>
struct Fmt<LX_W_FP8> {
  static constexpr bool kHalf = true;
  static constexpr int kStepValues = 64;
};
template <>
struct Fmt<LX_W_NVFP4> {
  static constexpr bool kHalf = true;
  static constexpr int kStepValues = 128;
};
template <>
struct Fmt<LX_W_BF16X> {
  static constexpr bool kHalf = false;
  static constexpr int kStepValues = 32;  // 32 sign|mantissa bytes + 16 bytes of codes
};

// BF16X layout constants (the format: u32 patch slots, one base exponent byte per 128 values, padding to 8 bytes,
// then per 128 values a 192-byte block of 128 sign|mantissa bytes and 64 bytes of 4-bit exponent codes).
namespace x16 {
constexpr uint32_t kNoPatch = 0xffffffffu;
__host__ __device__ constexpr int blocks(int K) { return (K + 127) / 128; }
__host__ __device__ constexpr int header_bytes(int K) { return (4 * (2 + K / 2048) + blocks(K) + 7) / 8 * 8; }
__host__ __device__ constexpr int patch_slots(int K) { return (header_bytes(K) - blocks(K)) / 4; }
__host__ __device__ constexpr int64_t row_bytes(int K) { return header_bytes(K) + 192ll * blocks(K); }
}  // namespace x16

template <int F, int RT, int WR, int NT, int U, int S>
struct StreamCfg {
  static constexpr int WK = kConsumerWarps / WR;
  static constexpr int R = 16 * RT * WR;
  static constexpr int kStepValues = Fmt<F>::kStepValues;
  static constexpr int VPT = kStepValues / 4;          // values a lane holds per row per step
  static constexpr int J = VPT / 4;                     // mma instructions per step per (row tile, n tile)
  static constexpr int JJ2 = VPT / 8;                   // 16-byte activation fragments per step per n tile
  static constexpr int STEPS = WK * U;                  // steps in a stage
  static constexpr int KSTAGE = STEPS * kStepValues;    // values of K in a stage
  static constexpr bool kX16 = F == LX_W_BF16X;
  static constexpr int SEG = kX16 ? (KSTAGE / 128) * 192 : STEPS * 64;  // weight bytes per row per stage
  // Row pitch in the stage: a tile copy lands its rows back to back (pitch SEG). BF16X records that are not
  // 16-byte aligned come row by row instead, each with 16 bytes of slack for the 8 bytes it may start late.
  static constexpr int PITCH_ROWWISE = SEG + 16;
  static constexpr int SCALE_SEG = F == LX_W_NVFP4 ? KSTAGE / 16 : 0;
  static constexpr int STAGE_BYTES = (R * ((kX16 ? PITCH_ROWWISE : SEG) + SCALE_SEG) + 127) / 128 * 128;
  static constexpr int XSTAGE_BYTES = STEPS * NT * JJ2 * 512;  // activation fragments for one stage, all 8 columns
  // Activations are staged into two halves (one chunk of K each); a half holds at least one stage's fragments.
  static constexpr int XHALF = XSTAGE_BYTES > 16384 ? XSTAGE_BYTES : 16384;
  static constexpr int XBYTES = 2 * XHALF;
  static constexpr int COLS = 8 * NT;
  static constexpr int RED_BYTES = WK * R * COLS * 4;
  static constexpr int RING_BYTES = S * STAGE_BYTES;
  static constexpr int MAIN_BYTES = RING_BYTES + RED_BYTES;  // the reduction buffer follows the ring
  static constexpr int HDR_PITCH = 0;  // BF16X headers are sized at run time (they depend on K)
  static_assert(!kX16 || STEPS % 4 == 0, "a BF16X stage is whole 128-value blocks");
  static_assert(R <= 256, "row bookkeeping assumes at most 256 rows per CTA");
};

// ---- expanding a lane's 16 bytes into mma operand pairs -----------------------------------------------------
// pairs[i] holds values (2i, 2i + 1) of the lane's chunk as two 16-bit floats; mma j of the step takes pairs 2j (its
// k-slots 2t, 2t + 1) and 2j + 1 (k-slots 2t + 8, 2t + 9).
template <int F>
struct Expand;

template <>
struct Expand<LX_W_BF16> {
  __device__ __forceinline__ static void run(uint4 q, uint32_t, uint32_t (&p)[4]) {
    p[0] = q.x, p[1] = q.y, p[2] = q.z, p[3] = q.w;
  }
};

template <>
struct Expand<LX_W_INT8> {
  // int8 v -> f16: (v ^ 0x80) is v + 128 in [1, 255]; 0x6400 | u is the f16 1024 + u; minus 1152 leaves v exactly.
  __device__ __forceinline__ static void run(uint4 q, uint32_t, uint32_t (&p)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t u = w[i] ^ 0x80808080u;
      uint32_t lo = __byte_perm(u, 0x64646464u, 0x5140);
      uint32_t hi = __byte_perm(u, 0x64646464u, 0x5342);
      __half2 l = __hsub2(*reinterpret_cast<__half2*>(&lo), bias);
      __half2 h = __hsub2(*reinterpret_cast<__half2*>(&hi), bias);
      p[2 * i] = *reinterpret_cast<uint32_t*>(&l);
      p[2 * i + 1] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
};

template <>
struct Expand<LX_W_FP8> {
  __device__ __forceinline__ static void run(uint4 q, uint32_t, uint32_t (&p)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2_raw l = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffffu), __NV_E4M3);
      const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3);
      p[2 * i] = static_cast<uint32_t>(l.x) | (static_cast<uint32_t>(l.y) << 16);
      p[2 * i + 1] = static_cast<uint32_t>(h.x) | (static_cast<uint32_t>(h.y) << 16);
    }
  }
};

template <>
struct Expand<LX_W_NVFP4> {
  // sc: the lane's two e4m3 block scales (values 0..15 and 16..31 of the chunk) in its low 16 bits.
  __device__ __forceinline__ static void run(uint4 q, uint32_t sc, uint32_t (&p)[16]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    const __half2_raw s = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(sc & 0xffffu), __NV_E4M3);
    const __half2 s0 = __halves2half2(__ushort_as_half(s.x), __ushort_as_half(s.x));
    const __half2 s1 = __halves2half2(__ushort_as_half(s.y), __ushort_as_half(s.y));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const __half2_raw r =
            __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>((w[i] >> (8 * b)) & 0xffu), __NV_E2M1);
        __half2 v = __halves2half2(__ushort_as_half(r.x), __ushort_as_half(r.y));
        v = __hmul2(v, i < 2 ? s0 : s1);
        p[4 * i + b] = *reinterpret_cast<uint32_t*>(&v);
      }
    }
  }
};

// BF16X: four bf16 from four sign|mantissa bytes and their four exponents (one per byte).
__device__ __forceinline__ uint2 x16_assemble(uint32_t sm, uint32_t e) {
  const uint32_t hi = (sm & 0x80808080u) | ((e >> 1) & 0x7f7f7f7fu);
  const uint32_t lo = (sm & 0x7f7f7f7fu) | ((e << 7) & 0x80808080u);
  return make_uint2(__byte_perm(lo, hi, 0x5140), __byte_perm(lo, hi, 0x7362));
}

// A row's patches, walked forward in k. `next` is the next patch not yet passed (kNoPatch once there are none).
struct PatchCursor {
  const uint32_t* p;
  int left;
  uint32_t next;
  // slots: the row's header slots (shared memory); rec: the row's record in global memory (for an overflow record).
  __device__ __forceinline__ void start(const uint32_t* slots, int n_slots, const uint8_t* rec) {
    p = slots;
    next = p[0];
    int n = n_slots;
    if (next != x16::kNoPatch && (next & 0x80000000u)) {
      const uint32_t* r = reinterpret_cast<const uint32_t*>(rec + static_cast<int64_t>(next & 0x7fffffffu) * 8);
      n = static_cast<int>(r[0]) + 1;  // the patches and their terminator
      p = r + 1;
      next = p[0];
    }
    ++p;
    left = n - 1;
  }
  __device__ __forceinline__ void advance() {
    next = left > 0 ? *p : x16::kNoPatch;
    ++p;
    --left;
  }
  // Applies the patches that fall in [k0, k0 + 8) to the exponent bytes of values k0..k0+3 (e_lo), k0+4..k0+7 (e_hi).
  __device__ __forceinline__ void apply(uint32_t k0, uint32_t& e_lo, uint32_t& e_hi) {
    while ((next >> 8) < k0) advance();
    while ((next >> 8) < k0 + 8) {
      const uint32_t d = (next >> 8) - k0;
      const uint32_t sh = 8 * (d & 3), v = (next & 0xffu) << sh, m = ~(0xffu << sh);
      if (d < 4) e_lo = (e_lo & m) | v;
      else e_hi = (e_hi & m) | v;
      advance();
    }
  }
};

template <int F, int RT, int WR, int NT, int U, int S>
size_t stream_smem_bytes(int K) {
  using C = StreamCfg<F, RT, WR, NT, U, S>;
  size_t b = C::MAIN_BYTES + C::XBYTES + 2 * S * 8 + 64 * (8 + 4 + 8) /* row pointers, maxima, chunk scales */ + 128;
  if (C::kX16) b += static_cast<size_t>(C::R) * ((x16::header_bytes(K) + 15) / 16 * 16);
  return b;
}

template <int F, int RT, int WR, int NT, int U, int S, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    stream_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap, const StreamParams P) {
  using C = StreamCfg<F, RT, WR, NT, U, S>;
  constexpr bool kHalf = Fmt<F>::kHalf;
  constexpr int R = C::R, WK = C::WK, COLS = C::COLS;

  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;                                      // S stages, then the reduction buffer
  uint8_t* xs = smem + C::MAIN_BYTES;                        // activation fragments of the current chunk
  uint64_t* bars = reinterpret_cast<uint64_t*>(xs + C::XBYTES);  // full[S], empty[S]
  const uint8_t** xrow = reinterpret_cast<const uint8_t**>(bars + 2 * S);  // [64] this pass's activation rows
  uint32_t* runmax = reinterpret_cast<uint32_t*>(xrow + 64);  // [64] bits of each row's largest magnitude so far
  float* bufscale = reinterpret_cast<float*>(runmax + 64);    // [2][64] the scale each half's columns were stored in
  uint8_t* hdr = reinterpret_cast<uint8_t*>(bufscale + 128);  // BF16X: R headers

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K = P.K;

  // ---- which rows, which weight, which activation rows ----------------------------------------------------
  int e = 0;          // expert
  int row0;           // first weight row of this CTA inside its matrix
  int n_cols_total;   // activation rows (columns of the product) this CTA serves
  int col_base0 = 0;  // experts: first grouped pair of the expert
  const uint8_t* wbase = P.w;
  const uint8_t* sbase = P.scale;
  float global = P.global;
  if constexpr (MODE == kDense) {
    row0 = blockIdx.x * R;
    n_cols_total = P.M;
  } else {
    const int group = blockIdx.y;
    col_base0 = P.offsets[group];
    n_cols_total = P.offsets[group + 1] - col_base0;
    if (n_cols_total <= 0) return;
    e = P.group_expert ? P.group_expert[group] : group;
    // gate_up: half of the CTA's rows are gate rows, the other half the matching up rows
    row0 = MODE == kGateUp ? blockIdx.x * (R / 2) : blockIdx.x * R;
    const int64_t rows = P.N;
    wbase += static_cast<int64_t>(e) * rows * P.row_bytes;
    if constexpr (F == LX_W_INT8 || F == LX_W_FP8) sbase += static_cast<int64_t>(e) * rows * 4;
    if constexpr (F == LX_W_NVFP4) {
      sbase += static_cast<int64_t>(e) * rows * (K / 16);
      if (P.expert_global) global = P.expert_global[e];
    }
  }
  // local row r of the CTA -> row of the matrix (clamped to the last row past the end)
  auto matrix_row = [&](int r) -> int {
    int n;
    if constexpr (MODE == kGateUp) {
      const int i = row0 + (r < R / 2 ? r : r - R / 2);
      n = i < P.I ? (r < R / 2 ? i : P.I + i) : P.N - 1;
    } else {
      n = row0 + r;
    }
    return n < P.N ? n : P.N - 1;
  };

  const int n_stages = (K + C::KSTAGE - 1) / C::KSTAGE;
  // f32 activations take two columns each (a high and a low half). More rows than the columns hold are served in
  // further passes over the weights (the host sizes NT so that decode-sized calls need one pass).
  const bool split = MODE == kDense && P.x_dtype != LX_BF16;
  const int cap = split ? COLS / 2 : COLS;
  const int col_chunks = (n_cols_total + cap - 1) / cap;
  const int total_stages = n_stages * col_chunks;

  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kConsumerWarps);
    }
    mbar_init_fence();
  }
  __syncthreads();

  // =========================================================================================================
  // Producer warp
  // =========================================================================================================
  if (warp == kConsumerWarps) {
    pdl_trigger();
    const int hb = C::kX16 ? x16::header_bytes(K) : 0;
    // first row of this CTA in the (stacked) weight, as the tile copies address it
    const int64_t stack_row0 = static_cast<int64_t>(e) * P.N + row0;
    if (P.tiled && lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
      if constexpr (F == LX_W_NVFP4) asm volatile("prefetch.tensormap [%0];" ::"l"(&smap) : "memory");
    }
    for (int gs = 0; gs < total_stages; ++gs) {
      const int s = gs % n_stages, slot = gs % S;
      if (gs >= S) mbar_wait(empty_bar(slot), ((gs / S) - 1) & 1, P.status, kStatusEmptyWait);
      const uint32_t stage = smem_u32(ring) + static_cast<uint32_t>(slot) * C::STAGE_BYTES;
      if (P.tiled) {
        // One tile copy per stage: R rows x SEG bytes (rows and bytes past the matrix read as zero). gate_up takes
        // two half-height tiles, the gate rows and the up rows.
        if (lane == 0) {
          mbar_arrive_expect_tx(full_bar(slot), R * (C::SEG + C::SCALE_SEG));
          const int x0 = (hb + s * C::SEG) / 4;  // the maps count the row in 4-byte elements
          if constexpr (MODE == kGateUp) {
            tile_g2s(stage, &wmap, x0, static_cast<int>(stack_row0), full_bar(slot));
            tile_g2s(stage + (R / 2) * C::SEG, &wmap, x0, static_cast<int>(stack_row0 + P.I), full_bar(slot));
          } else {
            tile_g2s(stage, &wmap, x0, static_cast<int>(stack_row0), full_bar(slot));
          }
          if constexpr (F == LX_W_NVFP4) {
            const uint32_t sdst = stage + R * C::SEG;
            if constexpr (MODE == kGateUp) {
              tile_g2s(sdst, &smap, s * C::SCALE_SEG, static_cast<int>(stack_row0), full_bar(slot));
              tile_g2s(sdst + (R / 2) * C::SCALE_SEG, &smap, s * C::SCALE_SEG, static_cast<int>(stack_row0 + P.I), full_bar(slot));
            } else {
              tile_g2s(sdst, &smap, s * C::SCALE_SEG, static_cast<int>(stack_row0), full_bar(slot));
            }
          }
        }
        continue;
      }
      if constexpr (C::kX16) {
        // Row by row. Records are 8-byte aligned: copy from the 16-byte boundary at or below the data, and if the
        // rounded-up end would pass the end of the rows, bring the last 8 bytes with an ordinary load instead.
        const int b0 = s * (C::KSTAGE / 128);
        const uint32_t bytes = min(C::KSTAGE / 128, x16::blocks(K) - b0) * 192;
        const uint8_t* end_all = wbase + static_cast<int64_t>(P.N) * P.row_bytes;
        uint32_t tx = 0;
        for (int r = lane; r < R; r += 32) {
          const uint8_t* src = wbase + matrix_row(r) * P.row_bytes + hb + static_cast<int64_t>(s) * C::SEG;
          const uint32_t sh = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & 15);
          uint32_t len = (bytes + sh + 15) & ~15u;
          if (src - sh + len > end_all) {
            len -= 16;
            *reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(slot) * C::STAGE_BYTES + r * C::PITCH_ROWWISE + len) =
                *reinterpret_cast<const uint64_t*>(src - sh + len);
          }
          tx += len;
        }
        tx = __reduce_add_sync(0xffffffffu, tx);
        if (lane == 0) mbar_arrive_expect_tx(full_bar(slot), tx);
        __syncwarp();
        for (int r = lane; r < R; r += 32) {
          const uint8_t* src = wbase + matrix_row(r) * P.row_bytes + hb + static_cast<int64_t>(s) * C::SEG;
          const uint32_t sh = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & 15);
          uint32_t len = (bytes + sh + 15) & ~15u;
          if (src - sh + len > end_all) len -= 16;
          if (len) bulk_g2s(stage + r * C::PITCH_ROWWISE, src - sh, len, full_bar(slot));
        }
      }
    }
    return;
  }

  // =========================================================================================================
  // Consumer warps
  // =========================================================================================================
  const int g = lane >> 2, t = lane & 3;
  const int wr = warp / WK, wk = warp % WK;

  // BF16X: bring the CTA's row headers (patch slots, base exponents) into shared memory.
  int hpitch = 0;
  if constexpr (C::kX16) {
    const int hb = x16::header_bytes(K);
    hpitch = (hb + 15) / 16 * 16;
    for (int i = tid; i < R * (hb / 8); i += kConsumerThreads) {
      const int r = i / (hb / 8), c = i % (hb / 8);
      *reinterpret_cast<uint64_t*>(hdr + r * hpitch + 8 * c) =
          *reinterpret_cast<const uint64_t*>(wbase + matrix_row(r) * P.row_bytes + 8 * c);
    }
  }
  // Everything below reads activations, which the previous kernel in the stream may have written.
  pdl_wait();

  float acc[RT][NT][4];
  const bool x_bf16 = P.x_dtype == LX_BF16;
  const int hdr_slots = C::kX16 ? x16::patch_slots(K) : 0;
  const int x_elem = x_bf16 ? 2 : 4;
  const int pitch = P.tiled ? C::SEG : C::PITCH_ROWWISE;  // BF16X only (the other formats always come as tiles)

  for (int cc = 0; cc < col_chunks; ++cc) {
    const int col0 = cc * cap;
    const int n_real = min(cap, n_cols_total - col0);  // activation rows of this pass
    const int n_cols = split ? 2 * n_real : n_real;    // columns they occupy
    // Fragment buffers hold 8-column tiles; a single tile is stored compactly (only its live columns).
    const int ncp = NT == 1 ? n_cols : 8;
    const int xs_stage = 2 * C::KSTAGE * NT * ncp;  // bytes of activations per weight stage
    // Stages per activation chunk: as many as fit one half of the fragment buffer.
    const int xg = max(1, C::XHALF / xs_stage);
    const int n_xchunks = (n_stages + xg - 1) / xg;

    named_bar_sync(1, kConsumerThreads);  // the previous pass's epilogue is done with the shared tables
    // activation row pointers of this pass's rows, and the running |max| of each
    for (int j = tid; j < n_real; j += kConsumerThreads) {
      int64_t row;
      if constexpr (MODE == kDense) row = col0 + j;
      else if constexpr (MODE == kGateUp) row = P.pairs[col_base0 + col0 + j] / P.top_k;
      else row = col_base0 + col0 + j;
      xrow[j] = static_cast<const uint8_t*>(P.x) + row * P.ld_x * x_elem;
      runmax[j] = 0u;
    }
#pragma unroll
    for (int a = 0; a < RT; ++a)
#pragma unroll
      for (int b = 0; b < NT; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.0f;

    PatchCursor cur[RT][2];
    uint32_t x16_shift[RT][2];  // BF16X row by row: how far the row's data sits past the 16-byte boundary of its copy
    named_bar_sync(1, kConsumerThreads);
    if constexpr (C::kX16) {
#pragma unroll
      for (int a = 0; a < RT; ++a)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = (wr * RT + a) * 16 + g + 8 * h;
          const uint8_t* rec = wbase + matrix_row(r) * P.row_bytes;
          cur[a][h].start(reinterpret_cast<const uint32_t*>(hdr + r * hpitch), hdr_slots, rec);
          x16_shift[a][h] = P.tiled ? 0u : static_cast<uint32_t>(reinterpret_cast<uintptr_t>(rec + x16::header_bytes(K)) & 15);
        }
    }

    // ---- activation staging --------------------------------------------------------------------------------
    // Chunk c covers stages [c * xg, (c + 1) * xg) and goes into half c & 1 of the fragment buffer. Its 8-value
    // groups are the items; item i is column i / groups, group i % groups, so consecutive threads read consecutive
    // 16 bytes of one activation row. A thread owns items tid, tid + 256, ... (at most kItems: a half holds 256 *
    // kItems groups). bf16 rows that are 16-byte aligned are prefetched: a chunk's loads are issued one chunk ahead
    // and sit in registers while the chunk before it is multiplied.
    constexpr int kItems = C::XHALF / 16 / kConsumerThreads;
    const bool x_fast = x_bf16 && P.x_vec;
    uint4 pre[kItems];
    auto chunk_groups = [&](int c) { return (min(K, (c + 1) * xg * C::KSTAGE) - c * xg * C::KSTAGE) / 8; };
    auto prefetch = [&](int c) {
      const int groups = chunk_groups(c), items = n_cols * groups, k0 = c * xg * C::KSTAGE;
#pragma unroll
      for (int q = 0; q < kItems; ++q) {
        const int i = tid + q * kConsumerThreads;
        if (i < items) pre[q] = *reinterpret_cast<const uint4*>(xrow[i / groups] + 2 * (k0 + 8 * (i % groups)));
      }
    };
    // The eight values of item i of chunk c, widened to f32.
    auto values = [&](int c, int q, int i, int groups, float (&v)[8]) {
      if (x_fast) {
        const uint32_t w4[4] = {pre[q].x, pre[q].y, pre[q].z, pre[q].w};
#pragma unroll
        for (int z = 0; z < 4; ++z) {
          v[2 * z] = __uint_as_float(w4[z] << 16);
          v[2 * z + 1] = __uint_as_float(w4[z] & 0xffff0000u);
        }
      } else {
        const int col = i / groups, k = c * xg * C::KSTAGE + 8 * (i % groups);
        const uint8_t* xr = xrow[split ? col >> 1 : col];
#pragma unroll
        for (int z = 0; z < 8; ++z)
          v[z] = x_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(xr)[k + z]) : reinterpret_cast<const float*>(xr)[k + z];
      }
    };
    // Power-of-two scale that brings a row whose largest magnitude has the bits `m` into [2^14, 2^15).
    auto scale_for = [](uint32_t m) -> float {
      int ex = static_cast<int>((m >> 23) & 0xffu);
      ex = m ? min(max(ex, 30), 240) : 141;
      return __uint_as_float(static_cast<uint32_t>(268 - ex) << 23);
    };
    // Converts the chunk (from the prefetched registers, or from memory) and stores it in fragment order.
    auto commit = [&](int c) {
      const int groups = chunk_groups(c), items = n_cols * groups, buf = c & 1;
      if constexpr (kHalf) {
#pragma unroll
        for (int q = 0; q < kItems; ++q) {
          const int i = tid + q * kConsumerThreads;
          if (i < items) {
            float v[8], m = 0.0f;
            values(c, q, i, groups, v);
#pragma unroll
            for (int z = 0; z < 8; ++z) m = fmaxf(m, fabsf(v[z]));
            const int col = i / groups;
            atomicMax(&runmax[split ? col >> 1 : col], __float_as_uint(m));
          }
        }
        named_bar_sync(1, kConsumerThreads);
      }
#pragma unroll
      for (int q = 0; q < kItems; ++q) {
        const int i = tid + q * kConsumerThreads;
        if (i >= items) continue;
        float v[8];
        values(c, q, i, groups, v);
        const int col = i / groups;
        uint32_t out[4];
        if constexpr (kHalf) {
          const float sc = scale_for(runmax[split ? col >> 1 : col]);
#pragma unroll
          for (int z = 0; z < 4; ++z) {
            const float a0 = v[2 * z] * sc, a1 = v[2 * z + 1] * sc;
            __half h0 = __float2half_rn(a0), h1 = __float2half_rn(a1);
            if (split && (col & 1)) {
              h0 = __float2half_rn(a0 - __half2float(h0));
              h1 = __float2half_rn(a1 - __half2float(h1));
            }
            out[z] = static_cast<uint32_t>(__half_as_ushort(h0)) | (static_cast<uint32_t>(__half_as_ushort(h1)) << 16);
          }
          if (i % groups == 0) bufscale[buf * 64 + col] = sc;
        } else if (x_fast) {
          out[0] = pre[q].x, out[1] = pre[q].y, out[2] = pre[q].z, out[3] = pre[q].w;
        } else {
#pragma unroll
          for (int z = 0; z < 4; ++z) {
            uint32_t b0 = f32_to_bf16_bits(v[2 * z]), b1 = f32_to_bf16_bits(v[2 * z + 1]);
            if (split && (col & 1)) {
              b0 = f32_to_bf16_bits(v[2 * z] - bf16_bits_to_f32(b0));
              b1 = f32_to_bf16_bits(v[2 * z + 1] - bf16_bits_to_f32(b1));
            }
            out[z] = b0 | (b1 << 16);
          }
        }
        const int kin = 8 * (i % groups);
        const int step = kin / C::kStepValues, within = kin % C::kStepValues;
        const int tt = within / C::VPT, jj2 = (within % C::VPT) / 8;
        const int unit = (((step * C::JJ2 + jj2) * NT + (NT == 1 ? 0 : col >> 3)) * 4 + tt) * ncp + (NT == 1 ? col : col & 7);
        *reinterpret_cast<uint4*>(xs + buf * C::XHALF + unit * 16) = make_uint4(out[0], out[1], out[2], out[3]);
      }
      named_bar_sync(1, kConsumerThreads);
    };

    float cur_scale[NT][2];  // the scale the accumulators of this lane's two columns of each tile are in
#pragma unroll
    for (int b = 0; b < NT; ++b) cur_scale[b][0] = cur_scale[b][1] = 0.0f;

    if (x_fast) prefetch(0);
    commit(0);
    if (x_fast && n_xchunks > 1) prefetch(1);
    for (int s = 0; s < n_stages; ++s) {
      const int gs = cc * n_stages + s, slot = gs % S;
      const int xc = s / xg, xbuf = xc & 1;
      if (s % xg == 0) {
        if (xc > 0) {
          // This chunk's activations: converted from the registers its loads landed in while the previous chunk was
          // multiplied. The half they go to was last read two chunks ago, behind the barriers since.
          commit(xc);
          if (x_fast && xc + 1 < n_xchunks) prefetch(xc + 1);
        }
        if constexpr (kHalf) {
          // accumulators move to this chunk's scale (scales only shrink, so nothing overflows)
#pragma unroll
          for (int b = 0; b < NT; ++b)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int col = 8 * b + 2 * t + h;
              const float ns = col < n_cols ? bufscale[xbuf * 64 + col] : 1.0f;
              if (cur_scale[b][h] != ns) {
                const float ratio = cur_scale[b][h] != 0.0f ? ns / cur_scale[b][h] : 1.0f;
#pragma unroll
                for (int a = 0; a < RT; ++a) acc[a][b][h] *= ratio, acc[a][b][2 + h] *= ratio;
                cur_scale[b][h] = ns;
              }
            }
        }
      }

      mbar_wait(full_bar(slot), (gs / S) & 1, P.status, kStatusFullWait);
      const uint8_t* stage = ring + static_cast<size_t>(slot) * C::STAGE_BYTES;
      const int k_stage0 = s * C::KSTAGE;
      const uint8_t* xbase = xs + xbuf * C::XHALF;

#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int st = wk * U + u;  // step inside the stage
        const int k_step0 = k_stage0 + st * C::kStepValues;
        if (k_step0 >= K) break;
        // weight operands
        uint32_t A[RT][C::J][4];
#pragma unroll
        for (int a = 0; a < RT; ++a) {
          const int r_lo = (wr * RT + a) * 16 + g, r_hi = r_lo + 8;
          uint32_t plo[C::VPT / 2], phi[C::VPT / 2];
          if constexpr (C::kX16) {
            const int blk = st >> 2, quarter = st & 3;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int r = h ? r_hi : r_lo;
              const uint8_t* b = stage + r * pitch + x16_shift[a][h] + blk * 192;
              const uint2 sm = *reinterpret_cast<const uint2*>(b + 32 * quarter + 8 * t);
              const uint32_t codes = *reinterpret_cast<const uint32_t*>(b + 128 + 4 * (4 * quarter + t));
              const uint32_t base = hdr[r * hpitch + 4 * hdr_slots + (k_step0 >> 7)];
              uint32_t e_lo = base * 0x01010101u - (codes & 0x0f0f0f0fu);
              uint32_t e_hi = base * 0x01010101u - ((codes >> 4) & 0x0f0f0f0fu);
              cur[a][h].apply(static_cast<uint32_t>(k_step0 + 8 * t), e_lo, e_hi);
              const uint2 v0 = x16_assemble(sm.x, e_lo), v1 = x16_assemble(sm.y, e_hi);
              uint32_t* dst = h ? phi : plo;
              dst[0] = v0.x, dst[1] = v0.y, dst[2] = v1.x, dst[3] = v1.y;
            }
          } else {
            const uint4 qlo = *reinterpret_cast<const uint4*>(stage + r_lo * C::SEG + st * 64 + t * 16);
            const uint4 qhi = *reinterpret_cast<const uint4*>(stage + r_hi * C::SEG + st * 64 + t * 16);
            uint32_t sc_lo = 0, sc_hi = 0;
            if constexpr (F == LX_W_NVFP4) {
              const uint8_t* sc = stage + R * C::SEG + st * 8 + t * 2;
              sc_lo = *reinterpret_cast<const uint16_t*>(sc + r_lo * C::SCALE_SEG);
              sc_hi = *reinterpret_cast<const uint16_t*>(sc + r_hi * C::SCALE_SEG);
            }
            Expand<F>::run(qlo, sc_lo, plo);
            Expand<F>::run(qhi, sc_hi, phi);
          }
#pragma unroll
          for (int j = 0; j < C::J; ++j) {
            A[a][j][0] = plo[2 * j];
            A[a][j][1] = phi[2 * j];
            A[a][j][2] = plo[2 * j + 1];
            A[a][j][3] = phi[2 * j + 1];
          }
        }
        // activation operands and the products
        const int xstep = (s - xc * xg) * C::STEPS + st;
#pragma unroll
        for (int b = 0; b < NT; ++b) {
#pragma unroll
          for (int jj = 0; jj < C::JJ2; ++jj) {
            uint4 xb = make_uint4(0, 0, 0, 0);
            if (NT > 1 || g < ncp)
              xb = *reinterpret_cast<const uint4*>(xbase + ((((xstep * C::JJ2 + jj) * NT + b) * 4 + t) * ncp + g) * 16);
#pragma unroll
            for (int a = 0; a < RT; ++a) {
              mma16816<kHalf>(acc[a][b], A[a][2 * jj], xb.x, xb.y);
              mma16816<kHalf>(acc[a][b], A[a][2 * jj + 1], xb.z, xb.w);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(slot));
    }

    // ---- the K-split partial sums meet in shared memory, added in warp order -------------------------------
    float* red = reinterpret_cast<float*>(ring + C::RING_BYTES);  // [WK][R][COLS]
#pragma unroll
    for (int a = 0; a < RT; ++a)
#pragma unroll
      for (int b = 0; b < NT; ++b) {
        const int r = (wr * RT + a) * 16 + g, c = 8 * b + 2 * t;
        float* o = red + (static_cast<size_t>(wk) * R + r) * COLS + c;
        float i0 = 1.0f, i1 = 1.0f;  // back from the lane's column scales to plain units
        if constexpr (kHalf) {
          i0 = cur_scale[b][0] != 0.0f ? 1.0f / cur_scale[b][0] : 1.0f;
          i1 = cur_scale[b][1] != 0.0f ? 1.0f / cur_scale[b][1] : 1.0f;
        }
        o[0] = acc[a][b][0] * i0, o[1] = acc[a][b][1] * i1;
        o[8 * COLS] = acc[a][b][2] * i0, o[8 * COLS + 1] = acc[a][b][3] * i1;
      }
    named_bar_sync(1, kConsumerThreads);
    auto total = [&](int r, int j) -> float {
      float sum = 0.0f;
      if (split) {
#pragma unroll
        for (int q = 0; q < WK; ++q)
          sum += red[(static_cast<size_t>(q) * R + r) * COLS + 2 * j] + red[(static_cast<size_t>(q) * R + r) * COLS + 2 * j + 1];
      } else {
#pragma unroll
        for (int q = 0; q < WK; ++q) sum += red[(static_cast<size_t>(q) * R + r) * COLS + j];
      }
      return sum;
    };
    auto row_factor = [&](int n) -> float {
      if constexpr (F == LX_W_INT8 || F == LX_W_FP8) return reinterpret_cast<const float*>(sbase)[n];
      else if constexpr (F == LX_W_NVFP4) return global;
      else return 1.0f;
    };
    if constexpr (MODE == kDense) {
      for (int i = tid; i < R * n_real; i += kConsumerThreads) {
        const int j = i / R, r = i % R, n = row0 + r;
        if (n >= P.N) continue;
        float tval = row_factor(n) * total(r, j);
        if (P.bias) tval += load_f32(P.bias, P.bias_dtype, n);
        float v = P.alpha * tval;
        const int64_t at = static_cast<int64_t>(col0 + j) * P.ld_y + n;
        if (P.beta != 0.0f) v = fmaf(P.beta, load_f32(P.y, P.y_dtype, at), v);
        store_from_f32(P.y, P.y_dtype, at, v);
      }
    } else if constexpr (MODE == kGateUp) {
      // mid[pair, i] = bf16(silu(s_g * gate . x) * (s_u * up . x)), rows in grouped order
      uint16_t* mid = static_cast<uint16_t*>(P.moe_out);
      for (int i = tid; i < (R / 2) * n_real; i += kConsumerThreads) {
        const int j = i / (R / 2), r = i % (R / 2), row = row0 + r;
        if (row >= P.I) continue;
        const float gv = row_factor(row) * total(r, j);
        const float uv = row_factor(P.I + row) * total(R / 2 + r, j);
        const float act = gv / (1.0f + expf(-gv)) * uv;
        mid[static_cast<int64_t>(col_base0 + col0 + j) * P.I + row] = static_cast<uint16_t>(f32_to_bf16_bits(act));
      }
    } else {
      // rows[pair, l] = weight[pair] * (s_l * down . mid), by pair index
      float* rows = static_cast<float*>(P.moe_out);
      for (int i = tid; i < R * n_real; i += kConsumerThreads) {
        const int j = i / R, r = i % R, n = row0 + r;
        if (n >= P.N) continue;
        const int pair = P.pairs[col_base0 + col0 + j];
        rows[static_cast<int64_t>(pair) * P.N + n] = P.route_w[pair] * (row_factor(n) * total(r, j));
      }
    }
  }
}

}  // namespace b200
