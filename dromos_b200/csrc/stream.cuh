// The weight-streaming product kernel: y[m, n] = sum_k x[m, k] * w[n, k] for a few activation rows (1..64) against
// a weight matrix that is read exactly once, at DRAM speed, in its stored format.
//
// Shape of the kernel
//   * Persistent CTAs (as many as fit the GPU at once), each walking a contiguous range of tiles. A tile is R
//     consecutive weight rows (16 * RT * WR) and all of K. NW consumer warps and one producer warp per CTA.
//   * The producer streams tiles through a ring of S shared-memory stages with 2-D TMA tile copies
//     (cp.async.bulk.tensor, no multicast): one copy per stage brings R rows x SEG bytes and completes on the stage's
//     "full" mbarrier; consumers release a stage on its "empty" mbarrier. The ring never drains between tiles.
//   * The weight tile is the A operand of mma.sync (16 weight rows x one k-group), the activations are the B operand
//     (k-group x 8 columns). A lane takes 16 contiguous bytes of a weight row from shared memory and uses them as the
//     k-slots the instruction assigns to it; since a dot product does not care about the order of k, the activations
//     are laid out in shared memory in the matching order ("fragment order") and no weight byte is ever shuffled.
//   * Math per format, chosen so that the weight bytes need as little work as possible:
//       BF16, BF16X  bf16 x bf16 (m16n8k16); BF16X rows are decoded in registers to the very bf16 bits they encode.
//       INT8         s8 x s8 -> s32 (m16n8k32) on the stored bytes. An activation is scaled by a power of two per
//                    row and written as three int8 digits in base 128 (three columns), 21 bits below the row's
//                    largest magnitude; the integer sums are exact and the digits are recombined in the epilogue.
//       FP8          e4m3 x e4m3 (m16n8k32) on the stored bytes. A scaled bf16 activation is the exact sum of two e4m3
//                    numbers (4 + 4 significant bits), so it takes two columns; f32 activations take three.
//       NVFP4        expanded in registers to f16 pairs times the block scale (exact), f16 x f16 (m16n8k16) against
//                    activations converted to f16 after a per-row power-of-two scaling.
//     f32 activations on the 16-bit paths are split into a high and a low half (two columns).
//   * WK = NW / WR warps split the K range of every stage between them; their partial sums meet in shared memory
//     and are added in a fixed order, so results are deterministic and a row's bits do not depend on M.
//   * Every wait is bounded (common.cuh mbar_wait): a stage that never arrives ends the kernel with a status code.
#pragma once

#include <cuda.h>
#include <cuda_fp4.h>

#include "common.cuh"

namespace b200 {

enum StreamMode { kDense = 0, kGateUp = 1, kDown = 2 };
enum MmaKind { kMmaBf16 = 0, kMmaF16 = 1, kMmaE4m3 = 2, kMmaS8 = 3 };

struct StreamParams {
  // the weight: one matrix, or a stack of experts each `N` rows
  const uint8_t* w;
  const uint8_t* scale;        // f32 [N] (INT8 / FP8) or e4m3 [N, K / 16] (NVFP4), stacked like w
  float global;                // NVFP4
  const float* expert_global;  // NVFP4 stacks, or null
  int64_t row_bytes;           // bytes of one weight row (BF16X: of one record)
  int N, K;
  // the activations
  const void* x;
  int x_dtype, ld_x, M;
  int x_vec;  // bf16 activation rows all start on 16-byte boundaries
  // dense epilogue
  const void* bias;
  int bias_dtype;
  void* y;
  int y_dtype, ld_y;
  float alpha, beta;
  // experts: grouping tables and the routed rows
  int groups;                   // expert groups the grid walks
  const int32_t* offsets;       // [groups + 1]: where each group's pairs start in `pairs`
  const int32_t* group_expert;  // [groups] the expert of each group, or null when group g is expert g
  const int32_t* pairs;         // [P] pair index t * top_k + k, grouped by expert
  const float* route_w;         // [P] by pair index
  int top_k, I;
  void* moe_out;  // gate_up: bf16 [P, I] in grouped order; down: f32 [P, L] by pair index
  int* status;
  int tiled;  // the weight rows come as 2-D tile copies through the tensor maps (else row by row)
  // Dense products may cut the work between CTAs at stage granularity instead of tile granularity (split_k): a tile
  // whose stages end up in several CTAs is finished by the last of them, which adds the others' partial sums (left in
  // `partials`, announced through `flags`) in CTA order.
  int split_k;
  float* partials;  // [grid][R * COLS]
  int* flags;       // [grid], zero between launches
};

template <int F>
struct Fmt;
template <>
struct Fmt<LX_W_BF16> {
  static constexpr int kMma = kMmaBf16;
  static constexpr int kStepValues = 32;  // values a warp step covers per row (64 bytes)
};
template <>
struct Fmt<LX_W_INT8> {
  static constexpr int kMma = kMmaS8;
  static constexpr int kStepValues = 64;
};
template <>
struct Fmt<LX_W_FP8> {
  static constexpr int kMma = kMmaE4m3;
  static constexpr int kStepValues = 64;
};
template <>
struct Fmt<LX_W_NVFP4> {
  static constexpr int kMma = kMmaF16;
  static constexpr int kStepValues = 128;
};
template <>
struct Fmt<LX_W_BF16X> {
  static constexpr int kMma = kMmaBf16;
  static constexpr int kStepValues = 32;  // 32 sign|mantissa bytes + 16 bytes of codes
};

// Columns one activation row takes under a math: its digits / halves.
__host__ __device__ constexpr int terms_for(int mma, bool x_bf16) {
  return mma == kMmaS8 ? 3 : mma == kMmaE4m3 ? (x_bf16 ? 2 : 3) : (x_bf16 ? 1 : 2);
}

// BF16X layout constants (the format: u32 patch slots, one base exponent byte per 128 values, padding to 8 bytes,
// then per 128 values a 192-byte block of 128 sign|mantissa bytes and 64 bytes of 4-bit exponent codes).
namespace x16 {
constexpr uint32_t kNoPatch = 0xffffffffu;
__host__ __device__ constexpr int blocks(int K) { return (K + 127) / 128; }
__host__ __device__ constexpr int header_bytes(int K) { return (4 * (2 + K / 2048) + blocks(K) + 7) / 8 * 8; }
__host__ __device__ constexpr int patch_slots(int K) { return (header_bytes(K) - blocks(K)) / 4; }
__host__ __device__ constexpr int64_t row_bytes(int K) { return header_bytes(K) + 192ll * blocks(K); }
}  // namespace x16

// F format, NW consumer warps, RT row tiles per warp, WR warp rows, NT column tiles, U steps per warp per stage,
// S ring stages, XKB kilobytes per activation half-buffer.
template <int F, int NW, int RT, int WR, int NT, int U, int S, int XKB>
struct StreamCfg {
  static constexpr int kMma = Fmt<F>::kMma;
  static constexpr bool k8bit = kMma == kMmaE4m3 || kMma == kMmaS8;
  static constexpr int kConsumerThreads = 32 * NW;
  static constexpr int kThreads = kConsumerThreads + 32;
  static constexpr int WK = NW / WR;
  static constexpr int R = 16 * RT * WR;
  static constexpr int kStepValues = Fmt<F>::kStepValues;
  static constexpr int VPT = kStepValues / 4;         // values a lane holds per row per step
  static constexpr int GV = k8bit ? 16 : 8;           // values in one 16-byte activation unit
  static constexpr int NREG = k8bit ? 4 : VPT / 2;    // operand registers a lane holds per row per step
  static constexpr int XU = NREG / 4;                 // 16-byte activation units per step per column tile
  static constexpr int STEPS = WK * U;                // steps in a stage
  static constexpr int KSTAGE = STEPS * kStepValues;  // values of K in a stage
  static constexpr bool kX16 = F == LX_W_BF16X;
  static constexpr int SEG = kX16 ? (KSTAGE / 128) * 192 : STEPS * 64;  // weight bytes per row per stage
  // A tile copy is at most 256 four-byte elements wide, so a stage is NBOX copies of R rows x BOXW bytes, laid out
  // one box after the other (BF16X boxes are whole 192-byte blocks).
  static constexpr int BOXW = kX16 ? (SEG <= 768 ? SEG : 768) : (SEG <= 1024 ? SEG : 1024);
  static constexpr int NBOX = SEG / BOXW;
  static constexpr int BOX_STEPS = kX16 ? BOXW / 48 : BOXW / 64;  // warp steps one box holds
  // Row pitch in the stage: a tile copy lands its rows back to back (pitch SEG). BF16X records that are not
  // 16-byte aligned come row by row instead, each with 16 bytes of slack for the 8 bytes it may start late.
  static constexpr int PITCH_ROWWISE = SEG + 16;
  static constexpr int SCALE_SEG = F == LX_W_NVFP4 ? KSTAGE / 16 : 0;
  static constexpr int STAGE_BYTES = (R * ((kX16 ? PITCH_ROWWISE : SEG) + SCALE_SEG) + 127) / 128 * 128;
  static constexpr int XSTAGE_BYTES = STEPS * XU * NT * 512;  // activation units of one stage, all 8 * NT columns
  static constexpr int XHALF = XKB * 1024;
  static constexpr int XBYTES = 2 * XHALF;
  static constexpr int COLS = 8 * NT;
  static constexpr int RED_BYTES = WK * R * COLS * 4;
  static constexpr int RING_BYTES = S * STAGE_BYTES;
  // Small reduction buffers come in pairs used in turn, so a tile's epilogue can overlap the next tile's products.
  static constexpr int RED_BUFS = RED_BYTES <= 16384 ? 2 : 1;
  static constexpr int MAIN_BYTES = RING_BYTES + RED_BUFS * RED_BYTES;  // the reduction buffers follow the ring
  static_assert(NW % WR == 0, "warps split into WR row groups");
  static_assert(!kX16 || STEPS % 4 == 0, "a BF16X stage is whole 128-value blocks");
  static_assert(XSTAGE_BYTES <= XHALF, "half an activation buffer holds at least one stage");
  static_assert(SEG % BOXW == 0 && SCALE_SEG <= 256, "a stage is whole boxes; a scale copy is at most 256 bytes wide");
  static_assert(COLS <= 64 && R <= 256, "bookkeeping tables are sized for 64 columns and 256 rows");
};

// ---- expanding a lane's 16 bytes into mma operand registers ---------------------------------------------------
// 16-bit maths: p[i] holds values (2i, 2i + 1) of the lane's chunk; mma m takes p[2m] (k-slots 2t, 2t + 1) and
// p[2m + 1] (k-slots 2t + 8, 2t + 9). 8-bit maths: p[i] is word i of the chunk as stored; mma m takes p[2m]
// (k-slots 4t .. 4t + 3) and p[2m + 1] (k-slots 16 + 4t ..).
template <int F>
struct Expand {
  __device__ __forceinline__ static void run(uint4 q, uint32_t, uint32_t (&p)[4]) {
    p[0] = q.x, p[1] = q.y, p[2] = q.z, p[3] = q.w;
  }
};

template <>
struct Expand<LX_W_NVFP4> {
  // sc: the lane's two e4m3 block scales (values 0..15 and 16..31 of the chunk) in its low 16 bits.
  __device__ __forceinline__ static void run(uint4 q, uint32_t sc, uint32_t (&p)[16]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t s2;
    asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(s2) : "r"(sc));
    const uint32_t s0 = __byte_perm(s2, s2, 0x1010), s1 = __byte_perm(s2, s2, 0x3232);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t v0, v1, v2, v3;
      asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %4;\n"
          "cvt.rn.f16x2.e2m1x2 %0, b0; cvt.rn.f16x2.e2m1x2 %1, b1; cvt.rn.f16x2.e2m1x2 %2, b2; cvt.rn.f16x2.e2m1x2 %3, b3; }"
          : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
          : "r"(w[i]));
      const uint32_t s = i < 2 ? s0 : s1;
      asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v0) : "r"(s));
      asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v1) : "r"(s));
      asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v2) : "r"(s));
      asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v3) : "r"(s));
      p[4 * i] = v0, p[4 * i + 1] = v1, p[4 * i + 2] = v2, p[4 * i + 3] = v3;
    }
  }
};

// D += A * B for the four maths. Accumulators are 32-bit: f32, or s32 for kMmaS8 (held in the same registers).
template <int kMma>
__device__ __forceinline__ void mma_step(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  if constexpr (kMma == kMmaBf16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else if constexpr (kMma == kMmaF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else if constexpr (kMma == kMmaE4m3) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

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

template <int F, int NW, int RT, int WR, int NT, int U, int S, int XKB>
size_t stream_smem_bytes(int K) {
  using C = StreamCfg<F, NW, RT, WR, NT, U, S, XKB>;
  size_t b = C::MAIN_BYTES + C::XBYTES + 2 * S * 8 + 64 * (8 + 4) /* row pointers, maxima */ + 128;
  if (C::kX16) b += static_cast<size_t>(C::R) * ((x16::header_bytes(K) + 15) / 16 * 16);
  return b;
}

template <int F, int NW, int RT, int WR, int NT, int U, int S, int XKB, int MODE>
__global__ void __launch_bounds__(32 * NW + 32, 1)
    stream_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap, const StreamParams P) {
  using C = StreamCfg<F, NW, RT, WR, NT, U, S, XKB>;
  constexpr int kMma = C::kMma;
  constexpr int R = C::R, WK = C::WK, COLS = C::COLS, kCT = C::kConsumerThreads;

  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;                                                    // S stages, then the reduction buffer
  uint8_t* xs = smem + C::MAIN_BYTES;                                      // activation units, two halves
  uint64_t* bars = reinterpret_cast<uint64_t*>(xs + C::XBYTES);            // full[S], empty[S]
  const uint8_t** xrow = reinterpret_cast<const uint8_t**>(bars + 2 * S);  // [64] this pass's activation rows
  uint32_t* runmax = reinterpret_cast<uint32_t*>(xrow + 64);               // [64] bits of each row's largest magnitude
  uint8_t* hdr = reinterpret_cast<uint8_t*>(runmax + 64);                  // BF16X: R headers

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K = P.K;
  const bool x_bf16 = P.x_dtype == LX_BF16;
  const int T = terms_for(kMma, x_bf16);  // columns per activation row
  const int cap = COLS / T;               // activation rows one pass over the weights serves
  const int n_stages = (K + C::KSTAGE - 1) / C::KSTAGE;

  // ---- the tiles this CTA walks --------------------------------------------------------------------------------
  const int rows_per_tile = MODE == kGateUp ? R / 2 : R;
  const int rows_total = MODE == kGateUp ? P.I : P.N;
  const int tiles_per_group = (rows_total + rows_per_tile - 1) / rows_per_tile;
  const int n_tiles = tiles_per_group * (MODE == kDense ? 1 : P.groups);
  // The CTA's share, in stages: [u0, u1) of the n_tiles * n_stages stages in tile order. Cut at tile boundaries unless
  // split_k, so that normally every tile is whole.
  const int64_t n_units = static_cast<int64_t>(n_tiles) * n_stages;
  int64_t u0, u1;
  if (P.split_k) {
    u0 = n_units * blockIdx.x / gridDim.x, u1 = n_units * (blockIdx.x + 1) / gridDim.x;
  } else {
    u0 = static_cast<int64_t>(n_tiles) * blockIdx.x / gridDim.x * n_stages;
    u1 = static_cast<int64_t>(n_tiles) * (blockIdx.x + 1) / gridDim.x * n_stages;
  }
  const int tile_begin = static_cast<int>(u0 / n_stages);
  const int tile_end = u1 > u0 ? static_cast<int>((u1 + n_stages - 1) / n_stages) : tile_begin;
  // the stages [sb, se) of a tile that are this CTA's
  auto stage_begin = [&](int tile) { return tile == tile_begin ? static_cast<int>(u0 - static_cast<int64_t>(tile_begin) * n_stages) : 0; };
  auto stage_end = [&](int tile) {
    return tile == tile_end - 1 ? static_cast<int>(u1 - static_cast<int64_t>(tile_end - 1) * n_stages) : n_stages;
  };
  // Order of the CTA's tiles: a last tile it does not finish goes first, so that the partial sums another CTA is
  // going to wait for are written at the start of this CTA's life, not at its end (no chains of waiting CTAs).
  const int my_tiles = tile_end - tile_begin;
  const bool tail_first = my_tiles > 1 && stage_end(tile_end - 1) < n_stages;
  auto tile_at = [&](int i) { return tail_first ? (i == 0 ? tile_end - 1 : tile_begin + i - 1) : tile_begin + i; };

  struct Tile {
    int e, row0, n_cols_total, col_base0, passes;
  };
  auto resolve = [&](int tile) -> Tile {
    Tile t;
    if constexpr (MODE == kDense) {
      t.e = 0, t.row0 = tile * R, t.n_cols_total = P.M, t.col_base0 = 0;
    } else {
      const int group = tile / tiles_per_group;
      t.col_base0 = P.offsets[group];
      t.n_cols_total = P.offsets[group + 1] - t.col_base0;
      t.e = P.group_expert ? P.group_expert[group] : group;
      t.row0 = (tile % tiles_per_group) * rows_per_tile;
    }
    t.passes = t.n_cols_total > 0 ? (t.n_cols_total + cap - 1) / cap : 0;
    return t;
  };
  // local row r of a tile -> row of the expert's matrix (clamped to the last row past the end)
  auto matrix_row = [&](const Tile& t, int r) -> int {
    int n;
    if constexpr (MODE == kGateUp) {
      const int i = t.row0 + (r < R / 2 ? r : r - R / 2);
      n = i < P.I ? (r < R / 2 ? i : P.I + i) : P.N - 1;
    } else {
      n = t.row0 + r;
    }
    return n < P.N ? n : P.N - 1;
  };

  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), NW);
    }
    mbar_init_fence();
  }
  __syncthreads();

  // =========================================================================================================
  // Producer warp
  // =========================================================================================================
  if (warp == NW) {
    pdl_trigger();
    // Expert tiles are laid out by the grouping tables, which the previous kernel in the stream wrote: wait for it.
    // (A dense product reads nothing but the weight here and starts streaming at once.)
    if constexpr (MODE != kDense) pdl_wait();
    const int hb = C::kX16 ? x16::header_bytes(K) : 0;
    if (P.tiled && lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
      if constexpr (F == LX_W_NVFP4) asm volatile("prefetch.tensormap [%0];" ::"l"(&smap) : "memory");
    }
    int gs = 0;  // stages issued so far
    for (int ti = 0; ti < my_tiles; ++ti) {
      const int tile = tile_at(ti);
      const Tile t = resolve(tile);
      const uint8_t* wbase = P.w + static_cast<int64_t>(t.e) * P.N * P.row_bytes;
      const int64_t stack_row0 = static_cast<int64_t>(t.e) * P.N + t.row0;
      for (int pass = 0; pass < t.passes; ++pass) {
        for (int s = stage_begin(tile); s < stage_end(tile); ++s, ++gs) {
          const int slot = gs % S;
          if (gs >= S) mbar_wait(empty_bar(slot), ((gs / S) - 1) & 1, P.status, kStatusEmptyWait);
          const uint32_t stage = smem_u32(ring) + static_cast<uint32_t>(slot) * C::STAGE_BYTES;
          if (P.tiled) {
            // One tile copy per stage: R rows x SEG bytes (rows and bytes past the matrix read as zero). gate_up
            // takes two half-height tiles, the gate rows and the up rows.
            if (lane == 0) {
              mbar_arrive_expect_tx(full_bar(slot), R * (C::SEG + C::SCALE_SEG));
#pragma unroll
              for (int bx = 0; bx < C::NBOX; ++bx) {
                const int x0 = (hb + s * C::SEG + bx * C::BOXW) / 4;  // the weight map counts a row in 4-byte elements
                const uint32_t dst = stage + bx * R * C::BOXW;
                tile_g2s(dst, &wmap, x0, static_cast<int>(stack_row0), full_bar(slot));
                if constexpr (MODE == kGateUp)
                  tile_g2s(dst + (R / 2) * C::BOXW, &wmap, x0, static_cast<int>(stack_row0 + P.I), full_bar(slot));
              }
              if constexpr (F == LX_W_NVFP4) {
                const uint32_t sdst = stage + R * C::SEG;
                tile_g2s(sdst, &smap, s * C::SCALE_SEG, static_cast<int>(stack_row0), full_bar(slot));
                if constexpr (MODE == kGateUp)
                  tile_g2s(sdst + (R / 2) * C::SCALE_SEG, &smap, s * C::SCALE_SEG, static_cast<int>(stack_row0 + P.I),
                           full_bar(slot));
              }
            }
            continue;
          }
          if constexpr (C::kX16) {
            // Row by row. Records are 8-byte aligned: copy from the 16-byte boundary at or below the data, and if
            // the rounded-up end would pass the end of the rows, bring the last 8 bytes with an ordinary load.
            const int b0 = s * (C::KSTAGE / 128);
            const uint32_t bytes = min(C::KSTAGE / 128, x16::blocks(K) - b0) * 192;
            const uint8_t* end_all = wbase + static_cast<int64_t>(P.N) * P.row_bytes;
            uint32_t tx = 0;
            for (int r = lane; r < R; r += 32) {
              const uint8_t* src = wbase + matrix_row(t, r) * P.row_bytes + hb + static_cast<int64_t>(s) * C::SEG;
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
              const uint8_t* src = wbase + matrix_row(t, r) * P.row_bytes + hb + static_cast<int64_t>(s) * C::SEG;
              const uint32_t sh = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & 15);
              uint32_t len = (bytes + sh + 15) & ~15u;
              if (src - sh + len > end_all) len -= 16;
              if (len) bulk_g2s(stage + r * C::PITCH_ROWWISE, src - sh, len, full_bar(slot));
            }
          }
        }
      }
    }
    return;
  }

  // =========================================================================================================
  // Consumer warps
  // =========================================================================================================
  const int g = lane >> 2, t4 = lane & 3;
  const int wr = warp / WK, wk = warp % WK;
  const int hdr_slots = C::kX16 ? x16::patch_slots(K) : 0;
  const int hb = C::kX16 ? x16::header_bytes(K) : 0;
  const int hpitch = (hb + 15) / 16 * 16;
  const int x_elem = x_bf16 ? 2 : 4;
  const int pitch = P.tiled ? C::SEG : C::PITCH_ROWWISE;  // BF16X only (the other formats always come as tiles)
  // The power of two that brings a row's largest magnitude into the math's top binade: 2^14 for f16 (below 65504),
  // 2^7 for e4m3 (below 448), 2^5 for the first int8 digit (at most 64).
  constexpr int kTop = kMma == kMmaF16 ? 14 : kMma == kMmaE4m3 ? 7 : 5;
  auto scale_for = [](uint32_t m) -> float {
    int ex = static_cast<int>((m >> 23) & 0xffu);
    ex = m ? min(max(ex, 30), 230) : 127 + kTop;
    return __uint_as_float(static_cast<uint32_t>(254 + kTop - ex) << 23);
  };

  // Everything below reads activations, which the previous kernel in the stream may have written.
  pdl_wait();

  // Two accumulators per output fragment, fed alternately, so that consecutive products do not wait for each other;
  // they are added (in a fixed order) when the tile is done.
  uint32_t acc[RT][NT][4], acc2[RT][NT][4];
  int gs = 0;            // stages consumed so far
  int staged_key = -1;   // which rows the activation tables and (if resident) the unit buffer hold
  int staged_pass = -1;
  int red_flip = 0;      // which of the two reduction buffers the next tile uses

  for (int ti = 0; ti < my_tiles; ++ti) {
    const int tile = tile_at(ti);
    const Tile tl = resolve(tile);
    if (tl.passes == 0) continue;
    const uint8_t* wbase = P.w + static_cast<int64_t>(tl.e) * P.N * P.row_bytes;
    const uint8_t* sbase = P.scale;
    float global = P.global;
    if constexpr (F == LX_W_INT8 || F == LX_W_FP8) sbase += static_cast<int64_t>(tl.e) * P.N * 4;
    if constexpr (F == LX_W_NVFP4) {
      if (MODE != kDense && P.expert_global) global = P.expert_global[tl.e];
    }

    for (int pass = 0; pass < tl.passes; ++pass) {
      const int col0 = pass * cap;
      const int n_real = min(cap, tl.n_cols_total - col0);  // activation rows of this pass
      const int n_cols = T * n_real;                        // columns they occupy
      // Unit buffers hold 8-column tiles; a single tile is stored compactly (only its live columns).
      const int ncp = NT == 1 ? n_cols : 8;
      const int xs_stage = (C::KSTAGE / C::GV) * 16 * NT * ncp;  // bytes of activation units per weight stage
      // Resident when the whole of K fits the two halves together: staged once. Else one half per chunk of stages.
      const bool resident = static_cast<int64_t>(n_stages) * xs_stage <= C::XBYTES;
      const int xg = resident ? n_stages : max(1, C::XHALF / xs_stage);
      const int stage_key = MODE == kDense ? 0 : tl.col_base0;
      const bool rows_changed = staged_key != stage_key || staged_pass != pass;

      // Dense tiles after the first touch no shared table: they start without waiting for the previous tile's epilogue
      // (which reads the other reduction buffer).
      const bool quiet = MODE == kDense && !C::kX16 && !rows_changed && resident && C::RED_BUFS == 2;
      if (!quiet) named_bar_sync(1, kCT);  // the previous tile's epilogue is done with the shared tables
      if (rows_changed) {
        for (int j = tid; j < n_real; j += kCT) {
          int64_t row;
          if constexpr (MODE == kDense) row = col0 + j;
          else if constexpr (MODE == kGateUp) row = P.pairs[tl.col_base0 + col0 + j] / P.top_k;
          else row = tl.col_base0 + col0 + j;
          xrow[j] = static_cast<const uint8_t*>(P.x) + row * P.ld_x * x_elem;
          runmax[j] = 0u;
        }
      }
      if constexpr (C::kX16) {
        for (int i = tid; i < R * (hb / 8); i += kCT) {
          const int r = i / (hb / 8), c = i % (hb / 8);
          *reinterpret_cast<uint64_t*>(hdr + r * hpitch + 8 * c) =
              *reinterpret_cast<const uint64_t*>(wbase + matrix_row(tl, r) * P.row_bytes + 8 * c);
        }
      }
#pragma unroll
      for (int a = 0; a < RT; ++a)
#pragma unroll
        for (int b = 0; b < NT; ++b)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[a][b][c] = acc2[a][b][c] = 0u;
      if (!quiet) named_bar_sync(1, kCT);

      // What this thread's first epilogue item will need from global memory (row scales, bias, routing), asked for now
      // so that the tile's end does not wait on it.
      auto row_factor = [&](int n) -> float {
        if constexpr (F == LX_W_INT8 || F == LX_W_FP8) return reinterpret_cast<const float*>(sbase)[n];
        else if constexpr (F == LX_W_NVFP4) return global;
        else return 1.0f;
      };
      float pre_f0 = 0.0f, pre_f1 = 0.0f;
      int pre_pair = 0;
      {
        const int rows_out = MODE == kGateUp ? R / 2 : R;
        if (tid < rows_out * n_real) {
          const int j = tid / rows_out, r = tid % rows_out, n = tl.row0 + r;
          if constexpr (MODE == kDense) {
            if (n < P.N) {
              pre_f0 = row_factor(n);
              if (P.bias) pre_f1 = load_f32(P.bias, P.bias_dtype, n);
            }
          } else if constexpr (MODE == kGateUp) {
            if (n < P.I) pre_f0 = row_factor(n), pre_f1 = row_factor(P.I + n);
          } else {
            if (n < P.N) {
              pre_pair = P.pairs[tl.col_base0 + col0 + j];
              pre_f0 = row_factor(n);
              pre_f1 = P.route_w[pre_pair];
            }
          }
        }
      }

      PatchCursor cur[RT][2];
      uint32_t x16_shift[RT][2];  // BF16X row by row: how far the row's data sits past the 16-byte boundary of its copy
      if constexpr (C::kX16) {
#pragma unroll
        for (int a = 0; a < RT; ++a)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int r = (wr * RT + a) * 16 + g + 8 * h;
            const uint8_t* rec = wbase + matrix_row(tl, r) * P.row_bytes;
            cur[a][h].start(reinterpret_cast<const uint32_t*>(hdr + r * hpitch), hdr_slots, rec);
            x16_shift[a][h] = P.tiled ? 0u : static_cast<uint32_t>(reinterpret_cast<uintptr_t>(rec + hb) & 15);
          }
      }

      // ---- activation staging ------------------------------------------------------------------------------
      // An item is GV consecutive k of one activation row; it becomes T 16-byte units, one per column of the row.
      // The GV values of item (row j, k) as f32.
      auto fetch = [&](int j, int k, float (&v)[C::GV]) {
        const uint8_t* xr = xrow[j];
        if (x_bf16 && P.x_vec) {
#pragma unroll
          for (int q = 0; q < C::GV / 8; ++q) {
            const uint4 raw = *reinterpret_cast<const uint4*>(xr + 2 * (k + 8 * q));
            const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int z = 0; z < 4; ++z) {
              v[8 * q + 2 * z] = __uint_as_float(w4[z] << 16);
              v[8 * q + 2 * z + 1] = __uint_as_float(w4[z] & 0xffff0000u);
            }
          }
        } else {
#pragma unroll
          for (int z = 0; z < C::GV; ++z)
            v[z] = x_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(xr)[k + z]) : reinterpret_cast<const float*>(xr)[k + z];
        }
      };
      // Largest magnitude of every row of this pass (the maths that scale need it before the first unit is made).
      auto find_maxima = [&]() {
        const int groups = K / C::GV, items = n_real * groups;
        for (int i = tid; i < items; i += kCT) {
          float v[C::GV], m = 0.0f;
          fetch(i / groups, C::GV * (i % groups), v);
#pragma unroll
          for (int z = 0; z < C::GV; ++z) m = fmaxf(m, fabsf(v[z]));
          atomicMax(&runmax[i / groups], __float_as_uint(m));
        }
        named_bar_sync(1, kCT);
      };
      // Stages the units of stages [s0, s1) into the buffer at `dst`.
      auto stage_units = [&](int s0, int s1, uint8_t* dst) {
        const int k_lo = s0 * C::KSTAGE, k_hi = min(K, s1 * C::KSTAGE);
        const int groups = (k_hi - k_lo) / C::GV, items = n_real * groups;
        for (int i = tid; i < items; i += kCT) {
          const int j = i / groups, kin = C::GV * (i % groups);
          float v[C::GV];
          fetch(j, k_lo + kin, v);
          uint32_t out[3][4];
          if constexpr (kMma == kMmaBf16) {
            if (x_bf16) {
#pragma unroll
              for (int z = 0; z < 4; ++z) out[0][z] = (__float_as_uint(v[2 * z]) >> 16) | (__float_as_uint(v[2 * z + 1]) & 0xffff0000u);
            } else {
#pragma unroll
              for (int z = 0; z < 4; ++z) {
                const uint32_t b0 = f32_to_bf16_bits(v[2 * z]), b1 = f32_to_bf16_bits(v[2 * z + 1]);
                out[0][z] = b0 | (b1 << 16);
                out[1][z] = f32_to_bf16_bits(v[2 * z] - bf16_bits_to_f32(b0)) |
                            (f32_to_bf16_bits(v[2 * z + 1] - bf16_bits_to_f32(b1)) << 16);
              }
            }
          } else if constexpr (kMma == kMmaF16) {
            const float sc = scale_for(runmax[j]);
#pragma unroll
            for (int z = 0; z < 4; ++z) {
              const float a0 = v[2 * z] * sc, a1 = v[2 * z + 1] * sc;
              const __half h0 = __float2half_rn(a0), h1 = __float2half_rn(a1);
              out[0][z] = static_cast<uint32_t>(__half_as_ushort(h0)) | (static_cast<uint32_t>(__half_as_ushort(h1)) << 16);
              const __half l0 = __float2half_rn(a0 - __half2float(h0)), l1 = __float2half_rn(a1 - __half2float(h1));
              out[1][z] = static_cast<uint32_t>(__half_as_ushort(l0)) | (static_cast<uint32_t>(__half_as_ushort(l1)) << 16);
            }
          } else if constexpr (kMma == kMmaE4m3) {
            // digits in base 16 of the scaled value: each e4m3 takes the next four significant bits
            const float sc = scale_for(runmax[j]);
#pragma unroll
            for (int z = 0; z < 4; ++z) {
              uint32_t d0 = 0, d1 = 0, d2 = 0;
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                float r = v[4 * z + b] * sc;
                const uint32_t e0 = __nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
                r = (r - e4m3_to_f32(e0)) * 16.0f;
                const uint32_t e1 = __nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
                r = (r - e4m3_to_f32(e1)) * 16.0f;
                const uint32_t e2 = __nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
                d0 |= e0 << (8 * b), d1 |= e1 << (8 * b), d2 |= e2 << (8 * b);
              }
              out[0][z] = d0, out[1][z] = d1, out[2][z] = d2;
            }
          } else {
            // digits in base 128 of the scaled value, each in [-64, 64]
            const float sc = scale_for(runmax[j]);
#pragma unroll
            for (int z = 0; z < 4; ++z) {
              uint32_t d0 = 0, d1 = 0, d2 = 0;
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                float r = v[4 * z + b] * sc;
                const float q0 = rintf(r);
                r = (r - q0) * 128.0f;
                const float q1 = rintf(r);
                r = (r - q1) * 128.0f;
                const float q2 = rintf(r);
                d0 |= (static_cast<uint32_t>(static_cast<int>(q0)) & 0xffu) << (8 * b);
                d1 |= (static_cast<uint32_t>(static_cast<int>(q1)) & 0xffu) << (8 * b);
                d2 |= (static_cast<uint32_t>(static_cast<int>(q2)) & 0xffu) << (8 * b);
              }
              out[0][z] = d0, out[1][z] = d1, out[2][z] = d2;
            }
          }
          const int step = kin / C::kStepValues, within = kin % C::kStepValues;
          const int tt = within / C::VPT, xu = (within % C::VPT) / C::GV;
          for (int term = 0; term < T; ++term) {
            const int col = j * T + term;
            const int unit = (((step * C::XU + xu) * NT + (NT == 1 ? 0 : col >> 3)) * 4 + tt) * ncp + (NT == 1 ? col : col & 7);
            *reinterpret_cast<uint4*>(dst + unit * 16) = make_uint4(out[term][0], out[term][1], out[term][2], out[term][3]);
          }
        }
        named_bar_sync(1, kCT);
      };

      if (rows_changed) {
        if constexpr (kMma != kMmaBf16) find_maxima();
        if (resident) stage_units(0, n_stages, xs);
        staged_key = stage_key, staged_pass = pass;
      }
      if (!resident) stage_units(0, xg, xs);

      const int sb = stage_begin(tile), se = stage_end(tile);
      for (int s = sb; s < se; ++s, ++gs) {
        const int slot = gs % S;
        const int xc = s / xg;
        const uint8_t* xbase = resident ? xs : xs + (xc & 1) * C::XHALF;
        if (!resident && s % xg == 0 && (xc + 1) * xg < n_stages) {
          // the next chunk goes into the other half, once every warp has left the chunk that was there
          named_bar_sync(1, kCT);
          stage_units((xc + 1) * xg, (xc + 2) * xg, xs + ((xc + 1) & 1) * C::XHALF);
        }

        mbar_wait(full_bar(slot), (gs / S) & 1, P.status, kStatusFullWait);
        const uint8_t* stage = ring + static_cast<size_t>(slot) * C::STAGE_BYTES;
        const int k_stage0 = s * C::KSTAGE;

#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int st = wk * U + u;  // step inside the stage
          const int k_step0 = k_stage0 + st * C::kStepValues;
          if (k_step0 >= K) break;
          // weight operands
          uint32_t plo[RT][C::NREG], phi[RT][C::NREG];
#pragma unroll
          for (int a = 0; a < RT; ++a) {
            const int r_lo = (wr * RT + a) * 16 + g, r_hi = r_lo + 8;
            if constexpr (C::kX16) {
              const int blk = st >> 2, quarter = st & 3;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int r = h ? r_hi : r_lo;
                const uint8_t* b = P.tiled ? stage + (st / C::BOX_STEPS) * R * C::BOXW + r * C::BOXW + (blk % (C::BOXW / 192)) * 192
                                           : stage + r * pitch + x16_shift[a][h] + blk * 192;
                const uint2 sm = *reinterpret_cast<const uint2*>(b + 32 * quarter + 8 * t4);
                const uint32_t codes = *reinterpret_cast<const uint32_t*>(b + 128 + 4 * (4 * quarter + t4));
                const uint32_t base = hdr[r * hpitch + 4 * hdr_slots + (k_step0 >> 7)];
                uint32_t e_lo = base * 0x01010101u - (codes & 0x0f0f0f0fu);
                uint32_t e_hi = base * 0x01010101u - ((codes >> 4) & 0x0f0f0f0fu);
                cur[a][h].apply(static_cast<uint32_t>(k_step0 + 8 * t4), e_lo, e_hi);
                const uint2 v0 = x16_assemble(sm.x, e_lo), v1 = x16_assemble(sm.y, e_hi);
                uint32_t* dst = h ? phi[a] : plo[a];
                dst[0] = v0.x, dst[1] = v0.y, dst[2] = v1.x, dst[3] = v1.y;
              }
            } else {
              const uint8_t* box = stage + (st / C::BOX_STEPS) * R * C::BOXW + (st % C::BOX_STEPS) * 64 + t4 * 16;
              const uint4 qlo = *reinterpret_cast<const uint4*>(box + r_lo * C::BOXW);
              const uint4 qhi = *reinterpret_cast<const uint4*>(box + r_hi * C::BOXW);
              uint32_t sc_lo = 0, sc_hi = 0;
              if constexpr (F == LX_W_NVFP4) {
                const uint8_t* sc = stage + R * C::SEG + st * 8 + t4 * 2;
                sc_lo = *reinterpret_cast<const uint16_t*>(sc + r_lo * C::SCALE_SEG);
                sc_hi = *reinterpret_cast<const uint16_t*>(sc + r_hi * C::SCALE_SEG);
              }
              Expand<F>::run(qlo, sc_lo, plo[a]);
              Expand<F>::run(qhi, sc_hi, phi[a]);
            }
          }
          // activation operands and the products
          const int xstep = (s - xc * xg) * C::STEPS + st;
#pragma unroll
          for (int b = 0; b < NT; ++b) {
#pragma unroll
            for (int xu = 0; xu < C::XU; ++xu) {
              uint4 xb = make_uint4(0, 0, 0, 0);
              if (NT > 1 || g < ncp)
                xb = *reinterpret_cast<const uint4*>(xbase + ((((xstep * C::XU + xu) * NT + b) * 4 + t4) * ncp + g) * 16);
#pragma unroll
              for (int a = 0; a < RT; ++a) {
                mma_step<kMma>(acc[a][b], plo[a][4 * xu], phi[a][4 * xu], plo[a][4 * xu + 1], phi[a][4 * xu + 1], xb.x, xb.y);
                mma_step<kMma>(acc2[a][b], plo[a][4 * xu + 2], phi[a][4 * xu + 2], plo[a][4 * xu + 3], phi[a][4 * xu + 3], xb.z, xb.w);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(slot));
      }

      // ---- the K-split partial sums meet in shared memory, added in warp order ---------------------------
      float* red = reinterpret_cast<float*>(ring + C::RING_BYTES + (C::RED_BUFS == 2 ? (red_flip ^= 1) : 0) * C::RED_BYTES);  // [WK][R][COLS]
#pragma unroll
      for (int a = 0; a < RT; ++a)
#pragma unroll
        for (int b = 0; b < NT; ++b) {
          const int r = (wr * RT + a) * 16 + g, c = 8 * b + 2 * t4;
          float* o = red + (static_cast<size_t>(wk) * R + r) * COLS + c;
          float f[4];
#pragma unroll
          for (int q = 0; q < 4; ++q)
            f[q] = kMma == kMmaS8 ? static_cast<float>(static_cast<int>(acc[a][b][q]) + static_cast<int>(acc2[a][b][q]))
                                  : __uint_as_float(acc[a][b][q]) + __uint_as_float(acc2[a][b][q]);
          o[0] = f[0], o[1] = f[1];
          o[8 * COLS] = f[2], o[8 * COLS + 1] = f[3];
        }
      named_bar_sync(1, kCT);
      if (se < n_stages) {
        // The tile ends in a later CTA: leave this part's sums (K-split partials added in warp order) for it.
        float* mine = P.partials + static_cast<size_t>(blockIdx.x) * R * COLS;
        for (int i = tid; i < R * n_cols; i += kCT) {
          const int r = i / n_cols, c = i % n_cols;
          float part = 0.0f;
#pragma unroll
          for (int q = 0; q < WK; ++q) part += red[(static_cast<size_t>(q) * R + r) * COLS + c];
          mine[r * COLS + c] = part;
        }
        __threadfence();
        named_bar_sync(1, kCT);
        if (tid == 0) st_release(P.flags + blockIdx.x, 1);
        continue;
      }
      if (sb > 0) {
        // The tile began in earlier CTAs: add their parts, in CTA order, to this one's.
        const int64_t tile_u0 = static_cast<int64_t>(tile) * n_stages;
        int first = static_cast<int>(tile_u0 * gridDim.x / n_units);
        while (n_units * (first + 1) / gridDim.x <= tile_u0) ++first;
        while (n_units * first / gridDim.x > tile_u0) --first;
        for (int other = first; other < static_cast<int>(blockIdx.x); ++other) {
          flag_wait(P.flags + other, P.status);
          const float* theirs = P.partials + static_cast<size_t>(other) * R * COLS;
          for (int i = tid; i < R * n_cols; i += kCT) {
            const int r = i / n_cols, c = i % n_cols;
            red[static_cast<size_t>(r) * COLS + c] += ld_cg(theirs + r * COLS + c);
          }
        }
        named_bar_sync(1, kCT);
        for (int other = first + tid; other < static_cast<int>(blockIdx.x); other += kCT) P.flags[other] = 0;
      }
      // the product for local row r and activation row j of this pass: K-split partials in warp order, the row's
      // digits recombined, the activation scale taken back out
      auto total = [&](int r, int j) -> float {
        float sum = 0.0f;
        float digit = 1.0f;
        for (int term = 0; term < T; ++term) {
          float part = 0.0f;
#pragma unroll
          for (int q = 0; q < WK; ++q) part += red[(static_cast<size_t>(q) * R + r) * COLS + j * T + term];
          sum += part * digit;
          digit *= kMma == kMmaS8 ? 0.0078125f : kMma == kMmaE4m3 ? 0.0625f : 1.0f;
        }
        if constexpr (kMma != kMmaBf16) sum *= 1.0f / scale_for(runmax[j]);
        return sum;
      };
      if constexpr (MODE == kDense) {
        for (int i = tid; i < R * n_real; i += kCT) {
          const int j = i / R, r = i % R, n = tl.row0 + r;
          if (n >= P.N) continue;
          const bool first = i == tid;
          float tval = (first ? pre_f0 : row_factor(n)) * total(r, j);
          if (P.bias) tval += first ? pre_f1 : load_f32(P.bias, P.bias_dtype, n);
          float v = P.alpha * tval;
          const int64_t at = static_cast<int64_t>(col0 + j) * P.ld_y + n;
          if (P.beta != 0.0f) v = fmaf(P.beta, load_f32(P.y, P.y_dtype, at), v);
          store_from_f32(P.y, P.y_dtype, at, v);
        }
      } else if constexpr (MODE == kGateUp) {
        // mid[pair, i] = bf16(silu(s_g * gate . x) * (s_u * up . x)), rows in grouped order
        uint16_t* mid = static_cast<uint16_t*>(P.moe_out);
        for (int i = tid; i < (R / 2) * n_real; i += kCT) {
          const int j = i / (R / 2), r = i % (R / 2), row = tl.row0 + r;
          if (row >= P.I) continue;
          const bool first = i == tid;
          const float gv = (first ? pre_f0 : row_factor(row)) * total(r, j);
          const float uv = (first ? pre_f1 : row_factor(P.I + row)) * total(R / 2 + r, j);
          const float act = gv / (1.0f + expf(-gv)) * uv;
          mid[static_cast<int64_t>(tl.col_base0 + col0 + j) * P.I + row] = static_cast<uint16_t>(f32_to_bf16_bits(act));
        }
      } else {
        // rows[pair, l] = weight[pair] * (s_l * down . mid), by pair index
        float* rows = static_cast<float*>(P.moe_out);
        for (int i = tid; i < R * n_real; i += kCT) {
          const int j = i / R, r = i % R, n = tl.row0 + r;
          if (n >= P.N) continue;
          const bool first = i == tid;
          const int pair = first ? pre_pair : P.pairs[tl.col_base0 + col0 + j];
          const float rf = first ? pre_f0 : row_factor(n), rw = first ? pre_f1 : P.route_w[pair];
          rows[static_cast<int64_t>(pair) * P.N + n] = rw * (rf * total(r, j));
        }
      }
    }
  }
}

}  // namespace b200
