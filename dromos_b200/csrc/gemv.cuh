// The decode GEMV: y[m, n] = sum_k x[m, k] * w[n, k] for 1..8 activation rows, every stored weight format, weights read
// once from HBM with plain 16-byte loads straight into registers.
//
// Why loads and not a TMA ring: measured on B200, a persistent kernel that streams a decode-sized matrix (33..235 MB)
// through shared memory with tile copies tops out near 4.7 TB/s, while warps that each keep a few 16-byte loads per lane
// in flight reach 6 TB/s and more, provided L1 is not carved out as shared memory (the in-flight lines live there) and
// the loop stays within ~100 warp instructions per KB of weights (at 6.5 TB/s an SM has 176 issue slots per KB). So:
//
//   * A CTA is 16 warps; warp w owns the w-th sixteenth of K for every row the CTA handles. CTA b owns a contiguous
//     range of rows cut at multiples of 16, taken in units of 16 rows (the rows of one mma.sync; the matrix's last unit
//     may be short). (N = 14336 on 296 CTAs gives 3 units to most CTAs and 4 to eight of them. Cutting the ranges at
//     multiples of 4 rows instead evens that out and was measured: no faster on any configuration, because a CTA that
//     is still streaming when its neighbours are done gets their share of the memory system.) Per
//     64-byte step of a row pair a lane loads 16 bytes of row g and 16 bytes of row g + 8 (lane = 4 g + t, bytes
//     16 t .. 16 t + 15 of the step) and uses them as the k-slots the instruction gives that lane: a dot product does not
//     care about the order of k as long as the activations follow it, and with this assignment they follow it in their
//     natural order (lane (g, t) reads contiguous bytes of column g's activations), so neither side is ever shuffled.
//   * Math per format:
//       BF16, BF16X  bf16 x bf16 (m16n8k16); BF16X steps are decoded in registers to the very bf16 bits the record encodes.
//       INT8         int8 -> f16 pairs in registers (exact: xor the sign bit, splice the byte into 1024 + v, subtract),
//                    f16 x f16 like FP8. (s8 x s8 -> s32 on the stored bytes against three int8 digit columns per row
//                    is exact too and needs no expansion, but was measured slower with 32-byte loads: 17.0 against
//                    16.3 us on the 14336 x 4096 matrix. Wide INT8 weights run on the tcgen05 product instead.)
//       FP8          e4m3 -> f16 pairs in registers (one conversion per two values, exact), f16 x f16 against the
//                    activations as f16 after a per-row power-of-two scaling. (mma.sync with e4m3 operands is not native
//                    on this part: the assembler expands it into ~10 times the instructions.)
//       NVFP4        e2m1 -> f16 pairs times the e4m3 block scale in registers (exact), f16 x f16 likewise.
//     f32 activations on the 16-bit maths are a high and a low column.
//   * The 16 partial sums of an output meet in shared memory and are added in warp order: no atomics, and a row's bits
//     depend on nothing but (format, K, activation dtype): not on M, N, the grid or the variant.
//   * Programmatic dependent launch: the kernel lets its successor start at once, sends its first loads (weights are
//     static) and only then waits for its predecessor, whose output its activations may be.
//
// There is no barrier another CTA could hold up and no copy engine to wait for: the kernel has no bounded waits.
#pragma once

#include "tc.cuh"

namespace b200 {
namespace {

constexpr int kGemvWarps = 16;  // = slices of K; fixed, because it fixes the order a row's products are added in
constexpr int kGemvThreads = 32 * kGemvWarps;
constexpr int kGemvUnitRows = 16;
constexpr int kGemvGranule = 16;  // a CTA's range of rows starts and ends at a multiple of this (any multiple of 4 works)
// words between two warps' sums of a unit in shared memory (NT 8-column tiles)
constexpr int kGemvRedStride(int nt) { return kGemvUnitRows * 8 * nt + 2; }

struct GemvParams {
  const uint8_t* w;
  const uint8_t* scale;  // f32 [N] (INT8 / FP8) or e4m3 [N, K / 16] (NVFP4)
  float global;
  int64_t row_bytes;
  int N, K;
  const void* x;
  int x_dtype, ld_x, M;
  const void* bias;
  int bias_dtype;
  void* y;
  int y_dtype, ld_y;
  float alpha, beta;
  int pitch;   // bytes between two activation columns in shared memory
  int ncols;   // M * planes
  int steps;   // 64-byte steps in a weight row
  int planes;  // digits (or halves) per activation row
};

// Per format: the mma, the bytes of a weight row a lane loads per step (a step is four lanes' worth of a row; BF16X: 8
// sign|mantissa bytes and 4 bytes of codes), the values of K a step covers and the bytes an activation column has per
// step. kSwz: the four 16-byte pieces of a lane's 64 bytes of activations are stored rotated by the lane's t, so that the
// four lanes of a column read different banks.
template <int F>
struct GemvFmt;
template <>
struct GemvFmt<LX_W_BF16> {
  static constexpr int kMma = kMmaBf16, kLane = 32, kStepValues = 64, kXStep = 128, kSwz = 0;
};
template <>
struct GemvFmt<LX_W_BF16X> {  // the same steps, slices and k-slots as BF16, so that the sums come out bit for bit the same
  static constexpr int kMma = kMmaBf16, kLane = 32, kStepValues = 64, kXStep = 128, kSwz = 0;
};
template <>
struct GemvFmt<LX_W_INT8> {  // expanded to f16 pairs like FP8 (kMmaS8 with kXStep 128 and no swizzle is the other, slower, choice)
  static constexpr int kMma = kMmaF16, kLane = 32, kStepValues = 128, kXStep = 256, kSwz = 1;
};
template <>
struct GemvFmt<LX_W_FP8> {
  static constexpr int kMma = kMmaF16, kLane = 32, kStepValues = 128, kXStep = 256, kSwz = 1;
};
template <>
struct GemvFmt<LX_W_NVFP4> {
  static constexpr int kMma = kMmaF16, kLane = 16, kStepValues = 128, kXStep = 256, kSwz = 1;
};
inline int gemv_mma_of(int wtype) {
  return wtype == LX_W_INT8 ? GemvFmt<LX_W_INT8>::kMma : (wtype == LX_W_FP8 || wtype == LX_W_NVFP4) ? kMmaF16 : kMmaBf16;
}
inline int gemv_step_values(int wtype) { return wtype == LX_W_BF16 || wtype == LX_W_BF16X ? 64 : 128; }
inline bool gemv_swizzled(int wtype) { return wtype == LX_W_FP8 || wtype == LX_W_NVFP4 || (wtype == LX_W_INT8 && GemvFmt<LX_W_INT8>::kSwz); }

template <int kMma>
constexpr int gemv_act() {
  return kMma == kMmaBf16 ? kActBf16 : kMma == kMmaF16 ? kActF16 : kMma == kMmaE4m3 ? kActE4m3 : kActS8;
}

// 32 bytes of weights that nothing will read again: around L1. `on` = 0 leaves q as it was.
__device__ __forceinline__ void ldg_stream32(uint32_t (&q)[8], const uint8_t* p, uint32_t on) {
  asm volatile(
      "{ .reg .pred q; setp.ne.u32 q, %9, 0;\n"
      "@q ld.global.nc.L1::no_allocate.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8]; }"
      : "+r"(q[0]), "+r"(q[1]), "+r"(q[2]), "+r"(q[3]), "+r"(q[4]), "+r"(q[5]), "+r"(q[6]), "+r"(q[7])
      : "l"(p), "r"(on));
}
// 16 bytes of weights that nothing will read again: around L1. `on` = 0 leaves v as it was.
__device__ __forceinline__ void ldg_stream16(uint32_t (&q)[4], const uint8_t* p, uint32_t on) {
  asm volatile(
      "{ .reg .pred q; setp.ne.u32 q, %5, 0;\n"
      "@q ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4]; }"
      : "+r"(q[0]), "+r"(q[1]), "+r"(q[2]), "+r"(q[3])
      : "l"(p), "r"(on));
}
__device__ __forceinline__ void ldg_nc8(uint32_t& a, uint32_t& b, const uint8_t* p, uint32_t on) {
  asm volatile("{ .reg .pred q; setp.ne.u32 q, %3, 0;\n@q ld.global.nc.v2.u32 {%0, %1}, [%2]; }" : "+r"(a), "+r"(b) : "l"(p), "r"(on));
}
__device__ __forceinline__ void ldg_nc4(uint32_t& a, const uint8_t* p, uint32_t on) {
  asm volatile("{ .reg .pred q; setp.ne.u32 q, %2, 0;\n@q ld.global.nc.u32 %0, [%1]; }" : "+r"(a) : "l"(p), "r"(on));
}
__device__ __forceinline__ void ldg_nc2(uint32_t& a, const uint8_t* p, uint32_t on) {
  asm volatile("{ .reg .pred q; .reg .b16 h; setp.ne.u32 q, %2, 0; cvt.u16.u32 h, %0;\n@q ld.global.nc.u16 h, [%1];\ncvt.u32.u16 %0, h; }" : "+r"(a) : "l"(p), "r"(on));
}
__device__ __forceinline__ void ldg_nc1(uint32_t& a, const uint8_t* p, uint32_t on) {
  asm volatile("{ .reg .pred q; setp.ne.u32 q, %2, 0;\n@q ld.global.nc.u8 %0, [%1]; }" : "+r"(a) : "l"(p), "r"(on));
}
// 16 bytes of shared memory at a 32-bit shared address; `on` = 0 leaves v as it was (zero, for columns nobody owns).
__device__ __forceinline__ void lds16(uint4& v, uint32_t addr, uint32_t on) {
  asm volatile("{ .reg .pred q; setp.ne.u32 q, %5, 0;\n@q ld.shared.v4.u32 {%0, %1, %2, %3}, [%4]; }"
               : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
               : "r"(addr), "r"(on));
}

// ---- staging the activations as mma B operands: column c = m * planes + digit, K contiguous ------------------------------
// The scaled maths need each row's largest magnitude before the first digit can be made: one pass over the rows for the
// maxima, a second (from L2) for the values. (Keeping the first pass's values in registers for the second was tried:
// the registers it holds across the barrier cost the main loop more than the second pass costs.)
// NAMED: the kGemvThreads callers are not the whole CTA (another warp does something else meanwhile): they meet at named
// barrier 1 instead of the CTA's barrier.
template <int ACT, bool XBF, bool SWZ, bool NAMED = false>
__device__ __forceinline__ void gemv_stage_x(const GemvParams& P, uint8_t* xs, float* inv_scale, float* part, int tid) {
  auto meet = [] {
    if constexpr (NAMED) named_bar_sync(1, kGemvThreads);
    else __syncthreads();
  };
  constexpr int V = 16 / act_elem(ACT);  // activations per 16 bytes of a plane
  const int warp = tid >> 5, lane = tid & 31;
  const bool aligned16 = (reinterpret_cast<uintptr_t>(P.x) & 15) == 0 && P.ld_x % (XBF ? 8 : 4) == 0;
  const int pieces = P.K / V;
  const int items = P.M * pieces;
  uint32_t* row_max = reinterpret_cast<uint32_t*>(part);  // [8]: bits of each row's largest magnitude
  auto store_planes = [&](int m, int p, const float (&v)[V]) {
    const float sc = ACT == kActBf16 ? 1.0f : part[8 * kGemvWarps + 8 + m];
    uint32_t wv[3][4];
    make_planes<ACT, XBF, V>(v, sc, wv);
    // piece p of a column is 16 bytes; with SWZ the four pieces of a lane's 64 bytes sit rotated by the lane's t
    const int at = SWZ ? (p & ~3) | ((p + (p >> 2)) & 3) : p;
#pragma unroll
    for (int j = 0; j < 3; ++j)
      if (j < P.planes)
        *reinterpret_cast<uint4*>(xs + static_cast<size_t>(m * P.planes + j) * P.pitch + static_cast<size_t>(at) * 16) =
            make_uint4(wv[j][0], wv[j][1], wv[j][2], wv[j][3]);
  };
  auto set_scales = [&]() {  // after row_max is complete
    if (tid < 8) {
      const float sc = scale_of<ACT>(__uint_as_float(row_max[tid]));
      part[8 * kGemvWarps + 8 + tid] = sc;
      inv_scale[tid] = 1.0f / sc;
    }
  };
  if constexpr (ACT != kActBf16) {
    for (int m = 0; m < P.M; ++m) {
      const float a = warp_max(row_max_share<XBF>(P.x, static_cast<int64_t>(m) * P.ld_x, P.K, aligned16, tid, kGemvThreads));
      if (lane == 0) part[8 + m * kGemvWarps + warp] = a;
    }
    meet();
    if (tid < 8) {
      float a = 0.0f;
      if (tid < P.M) {
#pragma unroll
        for (int w = 0; w < kGemvWarps; ++w) a = fmaxf(a, part[8 + tid * kGemvWarps + w]);
      }
      row_max[tid] = __float_as_uint(a);
    }
    meet();
    set_scales();
    meet();
  } else {
    if (tid < 8) inv_scale[tid] = 1.0f;
  }
  for (int i = tid, m = 0, p = tid; i < items; i += kGemvThreads, p += kGemvThreads) {
    while (p >= pieces) p -= pieces, ++m;
    float v[V];
    load_values<XBF, V>(P.x, static_cast<int64_t>(m) * P.ld_x, p * V, P.K, aligned16, v);
    store_planes(m, p, v);
  }
  meet();
}

// ---- BF16X: a row's patches, walked forward in k ---------------------------------------------------------------------------
// Two registers per row: the next patch not yet passed ((k << 8) | exponent, 0xffffffff when there is none) and how many
// the lane has taken. Where the list lives (header slots or an overflow record) is looked up again on every take: rows
// with patches are few and their patches fewer. The walking functions are out of line (they are rarely called) and take
// and return everything BY VALUE: a cursor handed over by reference (or as `this`) has to live in local memory, and then
// every check of `next` in the main loop is a local load (that version ran the C4 product in 45 us).
struct X16Cursor {
  uint32_t next, taken;
};
__device__ __noinline__ uint2 x16_take(const uint8_t* rec, int slots, uint32_t taken) {
  const uint32_t* list = reinterpret_cast<const uint32_t*>(rec);
  uint32_t n = static_cast<uint32_t>(slots);
  const uint32_t first = __ldg(list);
  if (first != x16::kNoPatch && (first & 0x80000000u)) {  // more patches than slots: they live in an overflow record
    const uint32_t* r = reinterpret_cast<const uint32_t*>(rec + static_cast<int64_t>(first & 0x7fffffffu) * 8);
    n = __ldg(r);
    list = r + 1;
  }
  return make_uint2(taken < n ? __ldg(list + taken) : x16::kNoPatch, taken + 1);
}
__device__ __forceinline__ X16Cursor x16_start(const uint8_t* rec, int slots, uint32_t k_from) {
  X16Cursor c{__ldg(reinterpret_cast<const uint32_t*>(rec)), 0u};
  if (c.next == x16::kNoPatch) return c;  // most rows
  do {
    const uint2 r = x16_take(rec, slots, c.taken);
    c.next = r.x, c.taken = r.y;
  } while ((c.next >> 8) < k_from);
  return c;
}
// the patches that fall in [k0, k0 + 8) go into the exponent bytes of values k0..k0+3 (e_lo) and k0+4..k0+7 (e_hi);
// returns {next, taken, e_lo, e_hi}
__device__ __noinline__ uint4 x16_apply(const uint8_t* rec, int slots, uint32_t k0, uint32_t next, uint32_t taken, uint32_t e_lo, uint32_t e_hi) {
  while ((next >> 8) < k0) {
    const uint2 r = x16_take(rec, slots, taken);
    next = r.x, taken = r.y;
  }
  while ((next >> 8) < k0 + 8) {
    const uint32_t d = (next >> 8) - k0, sh = 8 * (d & 3), v = (next & 0xffu) << sh, m = ~(0xffu << sh);
    if (d < 4) e_lo = (e_lo & m) | v;
    else e_hi = (e_hi & m) | v;
    const uint2 r = x16_take(rec, slots, taken);
    next = r.x, taken = r.y;
  }
  return make_uint4(next, taken, e_lo, e_hi);
}

// 8 bf16 (4 registers, values in k order) from 8 sign|mantissa bytes (sm0, sm1), their word of codes and the block's base
__device__ __forceinline__ void x16_decode8(uint32_t sm0, uint32_t sm1, uint32_t codes, uint32_t base, X16Cursor& cur, const uint8_t* rec, int slots, uint32_t k0, uint32_t (&a)[4]) {
  const uint32_t base4 = base * 0x01010101u;
  uint32_t e_lo = base4 - (codes & 0x0f0f0f0fu);
  uint32_t e_hi = base4 - ((codes >> 4) & 0x0f0f0f0fu);
  if ((cur.next >> 8) < k0 + 8) {
    const uint4 r = x16_apply(rec, slots, k0, cur.next, cur.taken, e_lo, e_hi);
    cur.next = r.x, cur.taken = r.y, e_lo = r.z, e_hi = r.w;
  }
  const uint2 v0 = x16_assemble(sm0, e_lo), v1 = x16_assemble(sm1, e_hi);
  a[0] = v0.x, a[1] = v0.y, a[2] = v1.x, a[3] = v1.y;
}

// One 32-bit word of NVFP4 (8 e2m1 values) times a block scale (f16x2, the same in both halves): 4 registers of f16 pairs
__device__ __forceinline__ void nvfp4_expand8(uint32_t word, uint32_t scale2, uint32_t (&a)[4]) {
  asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0; cvt.rn.f16x2.e2m1x2 %1, b1; cvt.rn.f16x2.e2m1x2 %2, b2; cvt.rn.f16x2.e2m1x2 %3, b3; }"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
      : "r"(word));
#pragma unroll
  for (int i = 0; i < 4; ++i) asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(a[i]) : "r"(scale2));
}
// One 32-bit word of int8 (4 values) as two registers of f16 pairs, exact: 0x6400 | (b ^ 0x80) is 1024 + 128 + b as f16
__device__ __forceinline__ void s8_expand4(uint32_t word, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = word ^ 0x80808080u;
  lo = __byte_perm(u, 0x64646464u, 0x4140);
  hi = __byte_perm(u, 0x64646464u, 0x4342);
  asm("sub.rn.f16x2 %0, %0, %1;" : "+r"(lo) : "r"(0x64806480u));
  asm("sub.rn.f16x2 %0, %0, %1;" : "+r"(hi) : "r"(0x64806480u));
}
// One 32-bit word of e4m3 (4 values) as two registers of f16 pairs, exact
__device__ __forceinline__ void e4m3_expand4(uint32_t word, uint32_t& lo, uint32_t& hi) {
  asm("{ .reg .b16 l, h; mov.b32 {l, h}, %2; cvt.rn.f16x2.e4m3x2 %0, l; cvt.rn.f16x2.e4m3x2 %1, h; }" : "=r"(lo), "=r"(hi) : "r"(word));
}

// F: weight format; NT: 8-column tiles of activations (digits included); CPS: CTAs per SM the kernel is built for (2: at
// most 64 registers; 1: twice the steps per row in flight).
//
// A warp walks its slice of each unit in batches of D steps: it sends the 2 D loads of a batch (32 bytes per lane and row
// each for the plain formats: a warp's load covers whole 128-byte lines, half the instructions and 5-8 % more bandwidth
// than 16-byte loads), multiplies them as they land, and goes on; the number of batches per unit is the same for all
// warps (a shorter slice has emptier batches) so that all warps meet the same barriers. What keeps memory busy while a
// lane multiplies is the other warps (32 per SM). Measured on B200: two register buffers per lane (the loads of batch
// i + 2 sent while batch i + 1 is multiplied) stream slower than one buffer of twice the depth; prefetching the next
// unit into L2 slows every size down; sending the next unit's loads before the unit's sums are added up makes the
// adding (shared-memory loads, which then queue behind them) slower than what it hides.
template <int F, int NT, int CPS>
__global__ void __launch_bounds__(kGemvThreads, CPS) gemv_kernel(const GemvParams P) {
  using Fm = GemvFmt<F>;
  constexpr int kMma = Fm::kMma;
  constexpr int kAct = gemv_act<kMma>();
  constexpr int COLS = 8 * NT;
  constexpr bool kX16 = F == LX_W_BF16X, kFp4 = F == LX_W_NVFP4;
  constexpr bool kFp8 = F == LX_W_FP8 || (F == LX_W_INT8 && kMma == kMmaF16);  // 8-bit values expanded to f16 pairs
  constexpr int kLane = Fm::kLane, kLW = kLane / 4;  // words a lane holds per row and step (BF16X: 4 + 2 + 1 of the 8)
  constexpr int D = CPS == 2 ? 2 : 4;
  constexpr int kXStep = Fm::kXStep;
  constexpr int kWStep = kX16 ? 0 : 4 * kLane;  // bytes a row pointer moves per step (BF16X addresses its blocks itself)
  extern __shared__ __align__(128) uint8_t smem[];
  float* red = reinterpret_cast<float*>(smem);                       // [2][16 warps][16 rows][COLS] (+ 2 words per warp)
  float* inv_scale = red + 2 * kGemvWarps * kGemvRedStride(NT);    // [8]
  float* part = inv_scale + 8;                                       // staging scratch: 8 + [8 rows][16 warps], then [8] scales
  uint8_t* xs = reinterpret_cast<uint8_t*>(part + 8 * kGemvWarps + 16);

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  // The CTA's rows: granules of kGemvGranule rows dealt out evenly, taken in units of up to 16 rows (only the last unit
  // of a CTA can be short). Where a row lands in a unit changes nothing about its sum.
  const int granules = (P.N + kGemvGranule - 1) / kGemvGranule;
  const int cta_row0 = static_cast<int>(static_cast<int64_t>(granules) * blockIdx.x / gridDim.x) * kGemvGranule;
  const int cta_row1 = min(P.N, static_cast<int>(static_cast<int64_t>(granules) * (blockIdx.x + 1) / gridDim.x) * kGemvGranule);
  const int my_rows = max(0, cta_row1 - cta_row0);
  const int n_units = (my_rows + kGemvUnitRows - 1) / kGemvUnitRows;
  const int s0 = P.steps * warp / kGemvWarps, s1 = P.steps * (warp + 1) / kGemvWarps;
  const int n_b = ((P.steps + kGemvWarps - 1) / kGemvWarps + D - 1) / D;  // batches per unit: the longest slice's
  const int hb = kX16 ? x16::header_bytes(P.K) : 0;
  const int slots = kX16 ? x16::patch_slots(P.K) : 0;
  const int64_t scale_row = kFp4 ? P.K / 16 : 0;

  // ---- a unit's state ----
  // Rows g and g + 8 of the unit; a lane whose row lies past the unit's end reads the unit's last row again (the same
  // bytes as another lane: no extra traffic) and its sums are never written.
  const uint8_t *pa = nullptr, *pb = nullptr;  // the lane's bytes of the slice's next step (BF16X: the two records)
  const uint8_t *sa = nullptr, *sb = nullptr;  // NVFP4: the lane's block scales of that step
  int row0 = 0, nrows = 0, rem = 0, s = 0;
  auto open_unit = [&](int u) {
    row0 = cta_row0 + kGemvUnitRows * u;
    nrows = min(kGemvUnitRows, my_rows - kGemvUnitRows * u);
    const int ra = min(g, nrows - 1), rb = min(g + 8, nrows - 1);
    const uint8_t* base = P.w + static_cast<int64_t>(row0) * P.row_bytes + (kX16 ? 0 : s0 * kWStep + kLane * t);
    pa = base + ra * P.row_bytes;
    pb = base + rb * P.row_bytes;
    if constexpr (kFp4) {
      const uint8_t* sbase = P.scale + static_cast<int64_t>(row0) * scale_row + 2 * (4 * s0 + t);  // values 32 c .., c = 4 s + t
      sa = sbase + ra * scale_row;
      sb = sbase + rb * scale_row;
    }
    s = s0;
    rem = s1 - s0;
  };
  // the loads of the next batch: D steps of both rows; steps past the slice's end are not loaded
  uint32_t qa[D][kLW], qb[D][kLW];
  uint32_t ea[kFp4 ? D : 1], eb[kFp4 ? D : 1];
  auto issue = [&]() {
#pragma unroll
    for (int d = 0; d < D; ++d) {
      const uint32_t on = d < rem ? 1u : 0u;
      if constexpr (kX16) {
        // step s + d is half (s + d) & 1 of block (s + d) >> 1; the lane's 16 values: 16 sign|mantissa bytes (two 8-byte
        // loads: records are only 8-byte aligned), their two words of codes, the block's base exponent
        const int sd = s + d, blk = hb + (sd >> 1) * 192, half = sd & 1;
        ldg_nc8(qa[d][0], qa[d][1], pa + blk + 64 * half + 16 * t, on);
        ldg_nc8(qa[d][2], qa[d][3], pa + blk + 64 * half + 16 * t + 8, on);
        ldg_nc8(qa[d][4], qa[d][5], pa + blk + 128 + 32 * half + 8 * t, on);
        ldg_nc1(qa[d][6], pa + 4 * slots + (sd >> 1), on);
        ldg_nc8(qb[d][0], qb[d][1], pb + blk + 64 * half + 16 * t, on);
        ldg_nc8(qb[d][2], qb[d][3], pb + blk + 64 * half + 16 * t + 8, on);
        ldg_nc8(qb[d][4], qb[d][5], pb + blk + 128 + 32 * half + 8 * t, on);
        ldg_nc1(qb[d][6], pb + 4 * slots + (sd >> 1), on);
      } else if constexpr (kLane == 32) {
        ldg_stream32(qa[d], pa + d * kWStep, on);
        ldg_stream32(qb[d], pb + d * kWStep, on);
      } else {
        ldg_stream16(qa[d], pa + d * kWStep, on);
        ldg_stream16(qb[d], pb + d * kWStep, on);
        if constexpr (kFp4) {
          ldg_nc2(ea[d], sa + d * 8, on);
          ldg_nc2(eb[d], sb + d * 8, on);
        }
      }
    }
  };
  // What a unit's epilogue wants from global memory (row factors, bias; static like the weights) is asked for with the
  // unit's first loads: thread 16 m + r finishes output (m, row r) of the unit.
  float rf = 1.0f, bias = 0.0f;
  auto ask_row_terms = [&]() {
    rf = 1.0f, bias = 0.0f;
    if ((tid & 15) < nrows && (tid >> 4) < P.M) {
      const int n = row0 + (tid & 15);
      if constexpr (F == LX_W_INT8 || F == LX_W_FP8) rf = __ldg(reinterpret_cast<const float*>(P.scale) + n);
      if constexpr (kFp4) rf = P.global;
      if (P.bias) bias = load_f32(P.bias, P.bias_dtype, n);
    }
  };

#pragma unroll
  for (int d = 0; d < D; ++d) {
#pragma unroll
    for (int i = 0; i < kLW; ++i) qa[d][i] = qb[d][i] = 0u;
    if constexpr (kFp4) ea[d] = eb[d] = 0;
  }
  // The first loads go out before the wait: weights, their scales and the bias are static (nothing earlier in the stream
  // writes them).
  if (n_units > 0) {
    open_unit(0);
    issue();
    ask_row_terms();
  }
  pdl_wait();
  if (P.x_dtype == LX_BF16) gemv_stage_x<kAct, true, Fm::kSwz != 0>(P, xs, inv_scale, part, tid);
  else gemv_stage_x<kAct, false, Fm::kSwz != 0>(P, xs, inv_scale, part, tid);

  const int T = P.planes;
  const float digit = kMma == kMmaS8 ? 0.0078125f : 1.0f;
  // this lane's activations: column 8 b + g of tile b, kXStep / 4 bytes per step starting t quarters in
  uint32_t x_on[NT], x_at[NT];
#pragma unroll
  for (int b = 0; b < NT; ++b) {
    const int col = 8 * b + g;
    x_on[b] = col < P.ncols ? 1u : 0u;
    x_at[b] = smem_u32(xs) + static_cast<uint32_t>(min(col, P.ncols - 1)) * static_cast<uint32_t>(P.pitch) + static_cast<uint32_t>(t) * (kXStep / 4);
  }
  uint4 xv[NT];  // 16 bytes of a column at a time
#pragma unroll
  for (int b = 0; b < NT; ++b) xv[b] = make_uint4(0, 0, 0, 0);
  constexpr int kRedStride = kGemvRedStride(NT);

  for (int u = 0; u < n_units; ++u) {
    // unit u is open, its first batch is in flight and its row terms have been asked for
    uint32_t acc[NT][4];
#pragma unroll
    for (int b = 0; b < NT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[b][c] = 0u;
    X16Cursor ca, cb;
    if constexpr (kX16) {
      ca = cb = X16Cursor{x16::kNoPatch, 0u};
      if (rem > 0) {
        ca = x16_start(pa, slots, static_cast<uint32_t>(s0) * 64u);
        cb = x16_start(pb, slots, static_cast<uint32_t>(s0) * 64u);
      }
    }
    for (int j = 0; j < n_b; ++j) {
      if (j) issue();
      const uint32_t xo = static_cast<uint32_t>(s) * kXStep;
#pragma unroll
      for (int d = 0; d < D; ++d) {
        if (d >= rem) break;
        if constexpr (kFp4 || kFp8) {
          // The lane's 32 values per row against 64 bytes of f16 activations, 8 values (one 16-byte piece, stored
          // rotated by t) at a time. NVFP4: word i of the 16 bytes, times the first (i < 2) or second block scale.
          // FP8: words 2 i and 2 i + 1 of the 32 bytes.
          uint32_t sa_lo = 0, sa_hi = 0, sb_lo = 0, sb_hi = 0;
          if constexpr (kFp4) {
            uint32_t sa2, sb2;
            asm("{ .reg .b16 h; cvt.u16.u32 h, %1; cvt.rn.f16x2.e4m3x2 %0, h; }" : "=r"(sa2) : "r"(ea[d]));
            asm("{ .reg .b16 h; cvt.u16.u32 h, %1; cvt.rn.f16x2.e4m3x2 %0, h; }" : "=r"(sb2) : "r"(eb[d]));
            sa_lo = __byte_perm(sa2, sa2, 0x1010), sa_hi = __byte_perm(sa2, sa2, 0x3232);
            sb_lo = __byte_perm(sb2, sb2, 0x1010), sb_hi = __byte_perm(sb2, sb2, 0x3232);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int b = 0; b < NT; ++b) lds16(xv[b], x_at[b] + xo + d * kXStep + 16 * ((i + t) & 3), x_on[b]);
            uint32_t pa4[4], pb4[4];
            if constexpr (kFp4) {
              nvfp4_expand8(qa[d][i], i < 2 ? sa_lo : sa_hi, pa4);
              nvfp4_expand8(qb[d][i], i < 2 ? sb_lo : sb_hi, pb4);
            } else if constexpr (F == LX_W_INT8) {
              s8_expand4(qa[d][2 * i], pa4[0], pa4[1]);
              s8_expand4(qa[d][2 * i + 1], pa4[2], pa4[3]);
              s8_expand4(qb[d][2 * i], pb4[0], pb4[1]);
              s8_expand4(qb[d][2 * i + 1], pb4[2], pb4[3]);
            } else {
              e4m3_expand4(qa[d][2 * i], pa4[0], pa4[1]);
              e4m3_expand4(qa[d][2 * i + 1], pa4[2], pa4[3]);
              e4m3_expand4(qb[d][2 * i], pb4[0], pb4[1]);
              e4m3_expand4(qb[d][2 * i + 1], pb4[2], pb4[3]);
            }
#pragma unroll
            for (int b = 0; b < NT; ++b) {
              mma_step<kMma>(acc[b], pa4[0], pb4[0], pa4[1], pb4[1], xv[b].x, xv[b].y);
              mma_step<kMma>(acc[b], pa4[2], pb4[2], pa4[3], pb4[3], xv[b].z, xv[b].w);
            }
          }
        } else if constexpr (kX16) {
          // the lane's 16 values as two halves of 8, decoded to what a BF16 lane would have loaded
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t a4[4], b4[4];
            const uint32_t k0 = static_cast<uint32_t>(s + d) * 64u + 16u * t + 8u * h;
            x16_decode8(qa[d][2 * h], qa[d][2 * h + 1], qa[d][4 + h], qa[d][6], ca, pa, slots, k0, a4);
            x16_decode8(qb[d][2 * h], qb[d][2 * h + 1], qb[d][4 + h], qb[d][6], cb, pb, slots, k0, b4);
#pragma unroll
            for (int b = 0; b < NT; ++b) {
              lds16(xv[b], x_at[b] + xo + d * kXStep + 16 * h, x_on[b]);
              mma_step<kMma>(acc[b], a4[0], b4[0], a4[1], b4[1], xv[b].x, xv[b].y);
              mma_step<kMma>(acc[b], a4[2], b4[2], a4[3], b4[3], xv[b].z, xv[b].w);
            }
          }
        } else {
          // BF16 / INT8: the lane's 32 bytes as two 16-byte halves, each against 16 bytes of a column
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int b = 0; b < NT; ++b) {
              lds16(xv[b], x_at[b] + xo + d * kXStep + 16 * h, x_on[b]);
              mma_step<kMma>(acc[b], qa[d][4 * h], qb[d][4 * h], qa[d][4 * h + 1], qb[d][4 * h + 1], xv[b].x, xv[b].y);
              mma_step<kMma>(acc[b], qa[d][4 * h + 2], qb[d][4 * h + 2], qa[d][4 * h + 3], qb[d][4 * h + 3], xv[b].z, xv[b].w);
            }
          }
        }
      }
      pa += D * kWStep, pb += D * kWStep;
      if constexpr (kFp4) sa += D * 8, sb += D * 8;
      s += D, rem -= D;
    }
    // ---- the 16 slices of every output meet in shared memory and are added in warp order ----
    // (warp stride padded by two words so that a unit's 16 x 16 sums spread over the banks)
    uint32_t* mine = reinterpret_cast<uint32_t*>(red) + (static_cast<size_t>(u & 1) * kGemvWarps + warp) * kRedStride;
#pragma unroll
    for (int b = 0; b < NT; ++b) {
      const int c = 8 * b + 2 * t;
      *reinterpret_cast<uint2*>(mine + g * COLS + c) = make_uint2(acc[b][0], acc[b][1]);
      *reinterpret_cast<uint2*>(mine + (g + 8) * COLS + c) = make_uint2(acc[b][2], acc[b][3]);
    }
    __syncthreads();
    if ((tid & 15) < nrows && (tid >> 4) < P.M) {
      const int out_m = tid >> 4, out_r = tid & 15;
      const uint32_t* all = reinterpret_cast<const uint32_t*>(red) + static_cast<size_t>(u & 1) * kGemvWarps * kRedStride;
      float sum = 0.0f, dw = 1.0f;
      for (int term = 0; term < T; ++term) {
        const int at = out_r * COLS + out_m * T + term;
        float p;
        if constexpr (kMma == kMmaS8) {
          int isum = 0;  // exact: the order does not matter
#pragma unroll
          for (int w = 0; w < kGemvWarps; ++w) isum += static_cast<int>(all[w * kRedStride + at]);
          p = static_cast<float>(isum);
        } else {
          p = 0.0f;
#pragma unroll
          for (int w = 0; w < kGemvWarps; ++w) p += __uint_as_float(all[w * kRedStride + at]);
        }
        sum += p * dw;
        dw *= digit;
      }
      if constexpr (kMma != kMmaBf16) sum *= inv_scale[out_m];
      float tval = rf * sum;
      if (P.bias) tval += bias;
      float v = P.alpha * tval;
      const int64_t at = static_cast<int64_t>(out_m) * P.ld_y + row0 + out_r;
      if (P.beta != 0.0f) v = fmaf(P.beta, load_f32(P.y, P.y_dtype, at), v);
      store_from_f32(P.y, P.y_dtype, at, v);
    }
    if (u + 1 < n_units) {
      open_unit(u + 1);
      issue();
      ask_row_terms();
    }
  }
}

// The column pitch and the shared memory a launch takes for `ncols` activation columns.
inline int gemv_pitch(int K, int wtype) {
  const int elem = gemv_mma_of(wtype) == kMmaS8 ? 1 : 2;
  const int mod = 16;  // columns g and g + 1 of a quarter warp read disjoint bank groups
  return (K * elem + 127) / 128 * 128 + mod;
}
inline size_t gemv_smem(int K, int wtype, int ncols) {
  const int NT = (ncols + 7) / 8;
  return static_cast<size_t>(2 * kGemvWarps * kGemvRedStride(NT) + 8 + 8 * kGemvWarps + 16) * 4 + static_cast<size_t>(ncols) * gemv_pitch(K, wtype);
}
constexpr size_t kGemvSmemMax = 220 * 1024;

}  // namespace
}  // namespace b200
