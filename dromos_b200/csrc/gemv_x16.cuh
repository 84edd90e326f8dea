// The decode GEMV of the lossless format (LX_W_BF16X), M = 1..8: gemv_kernel's sums (gemv.cuh) on records that bulk copies
// bring into shared memory.
//
// Why not gemv_kernel's loads here. A lane's 16 values of a step are 16 sign|mantissa bytes, 8 bytes of codes and a base
// exponent, at three places of a record whose blocks start on no line boundary: a warp's load touches 8 rows x 64 (or 32,
// or 1) bytes, one or two lines each, and the SM's table of lines in flight fills with requests that carry 24 to 64 bytes
// where a bf16 row carries 128. Measured on a 14336 x 4096 matrix (89 MB, 14 us to stream): 39 us, each SM taking about
// 8 bytes per clock whatever the depth of the loads in flight (a second register buffer per lane changed nothing). A bulk
// copy moves a record's bytes as the contiguous run they are and asks nothing of the load unit; the decode then reads
// shared memory.
//
//   * Roles: warps 0..15 multiply, warp 16 copies, warp 17 adds up. A stage is a whole unit where two fit in shared memory
//     (its 16 records are one contiguous run: one copy, headers included), else the same `cb` blocks (128 values, 192 bytes
//     each) of the unit's 16 rows, one copy per row (lanes 0..15) into a ring of S slots (rows 64 or 128 bytes further apart
//     than their bytes, so that a quarter warp's 16-byte reads of two rows fall on different banks), with the unit's headers
//     (patch slots and base exponents) in a ring of two. full/empty mbarriers per slot; every multiplying warp waits for
//     every stage in turn, multiplies what its slice of K has in it and releases it. Its 16 x M sums of a unit go to
//     shared memory (two units deep) and an mbarrier tells the adding warp, which adds the 16 slices in warp order and
//     stores y: no multiplying warp ever waits for another.
//   * Everything that sets a sum is gemv_kernel<LX_W_BF16>'s: 16 warps = 16 slices of K cut at the same steps, lane (g, t)
//     holds values 16 t .. 16 t + 15 of each 64-value step of rows g and g + 8 as the same mma.sync A fragments, the steps of
//     a slice are added in k order, the 16 slices in warp order. So y equals the bf16 product of the decoded matrix bit for
//     bit, whichever kernel runs.
//   * Patches (values whose exponent lies more than 15 below its block's largest: a few in 100000 of trained weights) are
//     walked by a cursor of two registers per row; the check is one comparison per step, the walk is out of line and
//     rewrites the assembled bf16 words.
//   * Records are only 8-byte aligned when the header's size is an odd multiple of 8: a copy then starts 8 bytes early and
//     ends up to 8 bytes late (inside the matrix: the host side sends a matrix whose last record would be read past its
//     end to gemv_kernel instead), and the reads of shared memory are 8-byte ones.
//   * Every wait is bounded (0.25 s): a role that gives up records status 5, marks the CTA dead, and every later wait
//     returns at once; the copying warp still waits (bounded) for the copies it has in flight before it leaves.
#pragma once

#include <type_traits>

#include "gemv.cuh"

namespace b200 {
namespace {

constexpr int kX16Threads = kGemvThreads + 64;

struct X16Ring {
  int cb;        // blocks of K per stage
  int spu;       // stages per unit
  int S;         // ring slots
  int whole;     // a stage is a whole unit, headers included, in one copy
  uint32_t stride, slot_bytes;    // of a row within a slot, of a slot
  uint32_t hstride, hslot_bytes;  // the same for the header ring
  uint32_t hdr_off, ring_off, bar_off;  // from the start of dynamic shared memory
  int* status;
};

// The geometry for (K, columns of activations): false when no useful ring fits beside the activations. Measured on a
// 14336 x 4096 matrix: the fewer and larger the copies the better (per-row copies of 4 / 8 / 11 / 16 blocks per stage: 55 /
// 34 / 30 / 26 us; one copy per unit: 23.5 us), so a whole unit per stage where two of them fit (its 16 records are one
// contiguous run: one copy, headers included), else the most blocks per stage that leave three slots. (Stages of 8 or 4
// whole records would be single copies too, but a unit can only be multiplied when all its rows are there, so they buy
// nothing unless two whole units fit anyway. Cutting the CTAs' row ranges at multiples of 8 rows, with the second row of
// each lane left out of a last unit of 8, evens the CTAs out to within half a unit and was measured slower: 24.3 us. One
// 2-D tile copy per stage through a tensor map (8-byte elements, boxes of 16 rows x 8 blocks, ring of 7; possible where
// records are 16-byte aligned) in place of the 16 per-row copies: 26.8 us at M = 1, 28.1 / 32.3 at M = 4 / 8 against 27.5 /
// 32.8: nothing gained, so the stages that are not whole units stay per-row bulk copies, which take every alignment.)
inline bool x16_ring_for(int K, int ncols, X16Ring& r, size_t& smem_total) {
  const int nblk = x16::blocks(K), hb = x16::header_bytes(K);
  const uint32_t fixed = static_cast<uint32_t>((gemv_smem(K, LX_W_BF16X, ncols) + 127) / 128 * 128);
  const uint32_t room = 226u * 1024u - 256u;
  const uint32_t unit_bytes = 16u * static_cast<uint32_t>(x16::row_bytes(K));
  auto finish = [&] {
    r.bar_off = r.ring_off + static_cast<uint32_t>(r.S) * r.slot_bytes;
    smem_total = r.bar_off + 8u * (2u * r.S + 8u) + 16u;
    return true;
  };
  if (fixed + 2u * ((unit_bytes + 127u) & ~127u) <= room) {
    r.whole = 1;
    r.cb = nblk, r.spu = 1;
    r.stride = static_cast<uint32_t>(x16::row_bytes(K));
    r.slot_bytes = (unit_bytes + 127u) & ~127u;
    r.hstride = r.hslot_bytes = 0;
    r.hdr_off = r.ring_off = fixed;
    r.S = static_cast<int>(std::min<uint32_t>(8u, (room - fixed) / r.slot_bytes));
    return finish();
  }
  r.whole = 0;
  r.hstride = static_cast<uint32_t>((hb + 8 + 15) / 16 * 16);
  r.hslot_bytes = 16u * r.hstride;
  r.hdr_off = fixed;
  r.ring_off = (fixed + 2u * r.hslot_bytes + 127u) / 128u * 128u;
  auto shape = [&](int cb) {
    r.cb = cb;
    r.stride = static_cast<uint32_t>(cb) * 192u + (cb % 2 ? 128u : 64u);  // = 64 mod 128, and 16 bytes to spare
    r.slot_bytes = 16u * r.stride;
    r.spu = (nblk + cb - 1) / cb;
    return r.ring_off + 3u * r.slot_bytes <= room;
  };
  for (int cb = std::min(32, nblk); cb >= 1; --cb) {
    if (!shape(cb)) continue;
    shape((nblk + r.spu - 1) / r.spu);  // the same number of stages, of even sizes
    r.S = static_cast<int>(std::min<uint32_t>(8u, (room - r.ring_off) / r.slot_bytes));
    return finish();
  }
  return false;
}

// Four bf16 (two words, values in k order) from four sign|mantissa bytes and their four exponents: x16_assemble with each
// (a & m) | (b & ~m) as the one three-input logic instruction it is (left to itself the compiler emitted two).
__device__ __forceinline__ void x16_pairs4(uint32_t sm, uint32_t e, uint32_t& w0, uint32_t& w1) {
  uint32_t hi, lo;
  asm("lop3.b32 %0, %1, %2, 0x80808080, 0xe4;" : "=r"(hi) : "r"(sm), "r"(e >> 1));  // sign | exponent >> 1
  asm("lop3.b32 %0, %1, %2, 0x80808080, 0xe4;" : "=r"(lo) : "r"(e << 7), "r"(sm));  // exponent & 1 | mantissa
  w0 = __byte_perm(lo, hi, 0x5140);
  w1 = __byte_perm(lo, hi, 0x7362);
}
// 8 bf16 (4 registers, values in k order) from 8 sign|mantissa bytes, their word of codes and the block's base in every byte
__device__ __forceinline__ void x16_words8(uint32_t sm0, uint32_t sm1, uint32_t codes, uint32_t base4, uint32_t* w) {
  const uint32_t e_lo = base4 - (codes & 0x0f0f0f0fu);
  const uint32_t e_hi = base4 - ((codes >> 4) & 0x0f0f0f0fu);
  x16_pairs4(sm0, e_lo, w[0], w[1]);
  x16_pairs4(sm1, e_hi, w[2], w[3]);
}

// The cursor of a row that has patches, placed at the first one at or after k_from.
__device__ __noinline__ uint2 x16_begin(const uint8_t* rec, int slots, uint32_t k_from) {
  const X16Cursor c = x16_start(rec, slots, k_from);
  return make_uint2(c.next, c.taken);
}
// The patches of [k0, k0 + 16) written into the 16 assembled values (word i = values 2 i and 2 i + 1): a patch replaces
// the exponent, bits 14..7 of its half. Everything by value: see X16Cursor.
struct X16Fix {
  uint32_t next, taken;
  uint32_t w[8];
};
__device__ __noinline__ X16Fix x16_fix16(const uint8_t* rec, int slots, uint32_t k0, X16Fix f) {
  while ((f.next >> 8) < k0) {
    const uint2 r = x16_take(rec, slots, f.taken);
    f.next = r.x, f.taken = r.y;
  }
  while ((f.next >> 8) < k0 + 16) {
    const uint32_t d = (f.next >> 8) - k0, sh = 16 * (d & 1) + 7;
    f.w[d >> 1] = (f.w[d >> 1] & ~(0xffu << sh)) | ((f.next & 0xffu) << sh);
    const uint2 r = x16_take(rec, slots, f.taken);
    f.next = r.x, f.taken = r.y;
  }
  return f;
}

// A wait of this kernel: at most 0.25 s, and none at all once the CTA is marked dead (unless `even_dead`: the last waits
// of the copying warp, for its own copies).
__device__ __forceinline__ bool x16_wait(uint32_t bar, uint32_t parity, volatile int* dead, int* status, bool even_dead = false) {
  if (*dead && !even_dead) return false;
  if (tc_wait(bar, parity, status)) return true;
  *dead = 1;
  return false;
}

// NT: 8-column tiles of activations (bf16 activations: one; f32 activations are a high and a low column each: two from
// M = 5 on). A16: every record starts on a 16-byte boundary.
template <int NT, bool A16>
__global__ void __launch_bounds__(kX16Threads, 1) gemv_x16_kernel(const GemvParams P, const X16Ring R) {
  constexpr int COLS = 8 * NT;
  constexpr int kXStep = GemvFmt<LX_W_BF16X>::kXStep;
  constexpr int kRedStride = kGemvRedStride(NT);
  extern __shared__ __align__(128) uint8_t smem[];
  float* red = reinterpret_cast<float*>(smem);                    // [2][16 warps][16 rows][COLS] (+ 2 words per warp)
  float* inv_scale = red + 2 * kGemvWarps * kRedStride;           // [8] (unused by this math; the layout is gemv_kernel's)
  float* part = inv_scale + 8;
  uint8_t* xs = reinterpret_cast<uint8_t*>(part + 8 * kGemvWarps + 16);
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t bars = smem0 + R.bar_off;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (R.S + s); };
  auto hfull_bar = [&](int s) { return bars + 8u * (2 * R.S + s); };
  auto hempty_bar = [&](int s) { return bars + 8u * (2 * R.S + 2 + s); };
  auto sums_bar = [&](int s) { return bars + 8u * (2 * R.S + 4 + s); };   // a unit's 16 partial sums are written
  auto taken_bar = [&](int s) { return bars + 8u * (2 * R.S + 6 + s); };  // and have been added up
  volatile int* dead = reinterpret_cast<volatile int*>(smem + R.bar_off + 8u * (2 * R.S + 8));

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < R.S; ++s) {
      mbar_init(full_bar(s), R.whole ? 1 : 16);  // the copying lanes, each with the bytes of its copy
      mbar_init(empty_bar(s), kGemvWarps);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(hfull_bar(s), 16);
      mbar_init(hempty_bar(s), kGemvWarps);
      mbar_init(sums_bar(s), kGemvWarps);
      mbar_init(taken_bar(s), 1);
    }
    *dead = 0;
    mbar_init_fence();
  }
  __syncthreads();

  const int granules = (P.N + kGemvGranule - 1) / kGemvGranule;
  const int cta_row0 = static_cast<int>(static_cast<int64_t>(granules) * blockIdx.x / gridDim.x) * kGemvGranule;
  const int cta_row1 = min(P.N, static_cast<int>(static_cast<int64_t>(granules) * (blockIdx.x + 1) / gridDim.x) * kGemvGranule);
  const int my_rows = max(0, cta_row1 - cta_row0);
  const int n_units = (my_rows + kGemvUnitRows - 1) / kGemvUnitRows;
  const int nblk = x16::blocks(P.K);
  const uint32_t hb = static_cast<uint32_t>(x16::header_bytes(P.K));
  const int slots = x16::patch_slots(P.K);

  if (warp == kGemvWarps) {
    // ---- the copying warp: weights are static, so it does not wait for the kernel before ----
    Ring ring;
    for (int u = 0; u < n_units; ++u) {
      const int row0 = cta_row0 + kGemvUnitRows * u;
      const int nrows = min(kGemvUnitRows, my_rows - kGemvUnitRows * u);
      if (R.whole) {
        // the unit's records are one run that starts on a 128-byte boundary (row0 is a multiple of 16, records of 8)
        x16_wait(empty_bar(ring.slot), ring.lap ^ 1u, dead, R.status);
        if (lane == 0) {
          const uint32_t bytes = (static_cast<uint32_t>(nrows) * static_cast<uint32_t>(P.row_bytes) + 15u) & ~15u;
          mbar_arrive_expect_tx(full_bar(ring.slot), bytes);
          bulk_g2s(smem0 + R.ring_off + ring.slot * R.slot_bytes, P.w + static_cast<int64_t>(row0) * P.row_bytes, bytes, full_bar(ring.slot));
        }
        ring.advance(R.S);
        continue;
      }
      const uint8_t* rec = P.w + static_cast<int64_t>(row0 + min(lane, nrows - 1)) * P.row_bytes;
      const int hs = u & 1;
      x16_wait(hempty_bar(hs), ((u >> 1) & 1) ^ 1u, dead, R.status);
      if (lane < 16) {
        if (lane < nrows) {
          const uint32_t sh = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(rec) & 15u), bytes = (sh + hb + 15u) & ~15u;
          mbar_arrive_expect_tx(hfull_bar(hs), bytes);
          bulk_g2s(smem0 + R.hdr_off + hs * R.hslot_bytes + lane * R.hstride, rec - sh, bytes, hfull_bar(hs));
        } else {
          mbar_arrive(hfull_bar(hs));
        }
      }
      for (int st = 0; st < R.spu; ++st) {
        x16_wait(empty_bar(ring.slot), ring.lap ^ 1u, dead, R.status);
        if (lane < 16) {
          if (lane < nrows) {
            const int blk_lo = st * R.cb, nb = min(R.cb, nblk - blk_lo);
            const uint8_t* src = rec + hb + static_cast<uint32_t>(blk_lo) * 192u;
            const uint32_t sh = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & 15u), bytes = (sh + static_cast<uint32_t>(nb) * 192u + 15u) & ~15u;
            mbar_arrive_expect_tx(full_bar(ring.slot), bytes);
            bulk_g2s(smem0 + R.ring_off + ring.slot * R.slot_bytes + lane * R.stride, src - sh, bytes, full_bar(ring.slot));
          } else {
            mbar_arrive(full_bar(ring.slot));
          }
        }
        ring.advance(R.S);
      }
    }
    // its copies have all landed before it leaves (the multiplying warps have waited for them too, unless they gave up)
    const int total = n_units * R.spu;
    Ring back;
    for (int i = 0; i < total; ++i) {
      if (i >= total - R.S) x16_wait(full_bar(back.slot), back.lap, dead, R.status, true);
      back.advance(R.S);
    }
    if (!R.whole)
      for (int u = max(0, n_units - 2); u < n_units; ++u) x16_wait(hfull_bar(u & 1), (u >> 1) & 1, dead, R.status, true);
    return;
  }

  if (warp == kGemvWarps + 1) {
    // ---- the adding warp: a unit's 16 slices are added in warp order (gemv_kernel's epilogue), 32 outputs at a time ----
    pdl_wait();  // y may still be in use by the kernel before
    const int T = P.planes;
    for (int u = 0; u < n_units; ++u) {
      const int row0 = cta_row0 + kGemvUnitRows * u;
      const int nrows = min(kGemvUnitRows, my_rows - kGemvUnitRows * u);
      const int rs = u & 1;
      x16_wait(sums_bar(rs), (u >> 1) & 1, dead, R.status);
      const uint32_t* all = reinterpret_cast<const uint32_t*>(red) + static_cast<size_t>(rs) * kGemvWarps * kRedStride;
      for (int o = lane; o < 16 * P.M; o += 32) {
        const int out_m = o >> 4, out_r = o & 15;
        if (out_r >= nrows) continue;
        float sum = 0.0f;
        for (int term = 0; term < T; ++term) {
          const int at = out_r * COLS + out_m * T + term;
          float p = 0.0f;
#pragma unroll
          for (int w = 0; w < kGemvWarps; ++w) p += __uint_as_float(all[w * kRedStride + at]);
          sum += p * 1.0f;
        }
        float tval = 1.0f * sum;
        if (P.bias) tval += load_f32(P.bias, P.bias_dtype, row0 + out_r);
        float v = P.alpha * tval;
        const int64_t at = static_cast<int64_t>(out_m) * P.ld_y + row0 + out_r;
        if (P.beta != 0.0f) v = fmaf(P.beta, load_f32(P.y, P.y_dtype, at), v);
        store_from_f32(P.y, P.y_dtype, at, v);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(taken_bar(rs));
    }
    return;
  }

  // ---- the multiplying warps ----
  const int g = lane >> 2, t = lane & 3;
  const int s0 = P.steps * warp / kGemvWarps, s1 = P.steps * (warp + 1) / kGemvWarps;
  pdl_wait();
  if (P.x_dtype == LX_BF16) gemv_stage_x<kActBf16, true, false, true>(P, xs, inv_scale, part, tid);
  else gemv_stage_x<kActBf16, false, false, true>(P, xs, inv_scale, part, tid);
  uint32_t x_on[NT], x_at[NT];
  uint4 xv[NT];
#pragma unroll
  for (int b = 0; b < NT; ++b) {
    const int col = 8 * b + g;
    x_on[b] = col < P.ncols ? 1u : 0u;
    x_at[b] = smem_u32(xs) + static_cast<uint32_t>(min(col, P.ncols - 1)) * static_cast<uint32_t>(P.pitch) + static_cast<uint32_t>(t) * (kXStep / 4);
    xv[b] = make_uint4(0, 0, 0, 0);
  }
  const uint32_t k_from = static_cast<uint32_t>(s0) * 64u;

  Ring ring;
  for (int u = 0; u < n_units; ++u) {
    const int row0 = cta_row0 + kGemvUnitRows * u;
    const int nrows = min(kGemvUnitRows, my_rows - kGemvUnitRows * u);
    const int ra = min(g, nrows - 1), rb = min(g + 8, nrows - 1);  // a lane past the unit's end reads its last row again
    auto rec_of = [&](int r) { return P.w + static_cast<int64_t>(row0 + r) * P.row_bytes; };
    const int hs = u & 1;
    // Where the two rows' headers and blocks are. A whole unit per stage: the records as they lie in memory, in the stage's
    // slot. Else: the header ring and, per stage, rows `stride` apart whose copies began 8 bytes early for records that are
    // not 16-byte aligned.
    const uint8_t *hdr_a, *hdr_b;
    uint32_t blocks_a, blocks_b;  // of block 0 of the stage's first block, from the slot's start
    if (R.whole) {
      const uint8_t* slot = smem + R.ring_off + ring.slot * R.slot_bytes;
      hdr_a = slot + ra * R.stride, hdr_b = slot + rb * R.stride;
      blocks_a = ra * R.stride + hb, blocks_b = rb * R.stride + hb;
    } else {
      uint32_t sh_a = 0, sh_b = 0;
      if constexpr (!A16) {
        sh_a = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(rec_of(ra)) & 15u);
        sh_b = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(rec_of(rb)) & 15u);
      }
      hdr_a = smem + R.hdr_off + hs * R.hslot_bytes + ra * R.hstride + sh_a;
      hdr_b = smem + R.hdr_off + hs * R.hslot_bytes + rb * R.hstride + sh_b;
      blocks_a = ra * R.stride + (A16 ? 0u : ((sh_a + hb) & 15u));
      blocks_b = rb * R.stride + (A16 ? 0u : ((sh_b + hb) & 15u));
      x16_wait(hfull_bar(hs), (u >> 1) & 1, dead, R.status);
    }
    uint32_t acc[NT][4];
#pragma unroll
    for (int b = 0; b < NT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[b][c] = 0u;

    // The patch cursors, from the header copies: a row's list is in its header slots (ascending, unused slots hold the
    // no-patch word, whose position is past every k), except a row with more patches than slots, whose slot 0 points to
    // a record after the rows: that one is walked out of line, in global memory.
    auto cursor_at = [&](const uint8_t* hdr, int r) {
      X16Cursor c{x16::kNoPatch, static_cast<uint32_t>(slots)};
      const uint32_t first = *reinterpret_cast<const uint32_t*>(hdr);
      if (first == x16::kNoPatch || s1 <= s0 || *dead) return c;
      if (first & 0x80000000u) {
        const uint2 v = x16_begin(rec_of(r), slots, k_from);
        c.next = v.x, c.taken = v.y;
        return c;
      }
      for (int i = 0; i < slots; ++i) {
        const uint32_t p = reinterpret_cast<const uint32_t*>(hdr)[i];
        if ((p >> 8) >= k_from) {
          c.next = p, c.taken = static_cast<uint32_t>(i) + 1u;
          break;
        }
      }
      return c;
    };
    X16Cursor ca{x16::kNoPatch, 0u}, cb{x16::kNoPatch, 0u};
    if (!R.whole) ca = cursor_at(hdr_a, ra), cb = cursor_at(hdr_b, rb);

    for (int st = 0; st < R.spu; ++st) {
      const int blk_lo = st * R.cb, blk_hi = min(nblk, blk_lo + R.cb);
      const int a = max(s0, 2 * blk_lo), b = min(s1, 2 * blk_hi);
      // Every warp waits for every stage, also one its slice has nothing in: a warp that ran ahead of the copies could
      // release a slot's next lap before the others have released this one.
      x16_wait(full_bar(ring.slot), ring.lap, dead, R.status);
      if (R.whole) ca = cursor_at(hdr_a, ra), cb = cursor_at(hdr_b, rb);  // the headers came with the stage
      if (a < b) {
        const uint8_t* slot = smem + R.ring_off + ring.slot * R.slot_bytes;
        // The lane's place in the block step `a` lies in, and on from there block by block: nothing in the loop multiplies.
        const uint32_t first = static_cast<uint32_t>(a >> 1) - static_cast<uint32_t>(blk_lo);
        const uint8_t* row_a = slot + blocks_a + first * 192u + 16u * t;
        const uint8_t* row_b = slot + blocks_b + first * 192u + 16u * t;
        const uint8_t* base_at_a = hdr_a + 4 * slots + (a >> 1);
        const uint8_t* base_at_b = hdr_b + 4 * slots + (a >> 1);
        uint32_t xo = static_cast<uint32_t>(a) * kXStep;
        uint32_t lim = (static_cast<uint32_t>(a) * 64u + 16u * t + 16u) << 8;  // the end of this lane's values of the step, as a patch word
        uint32_t base_a = 0, base_b = 0;
        // one step: half H of the block at row_a / row_b
        auto step = [&](auto half_c) {
          constexpr uint32_t H = decltype(half_c)::value;
          uint4 sm_a, sm_b;
          if constexpr (A16) {
            sm_a = *reinterpret_cast<const uint4*>(row_a + 64u * H);
            sm_b = *reinterpret_cast<const uint4*>(row_b + 64u * H);
          } else {
            const uint2 a0 = *reinterpret_cast<const uint2*>(row_a + 64u * H), a1 = *reinterpret_cast<const uint2*>(row_a + 64u * H + 8);
            const uint2 b0 = *reinterpret_cast<const uint2*>(row_b + 64u * H), b1 = *reinterpret_cast<const uint2*>(row_b + 64u * H + 8);
            sm_a = make_uint4(a0.x, a0.y, a1.x, a1.y);
            sm_b = make_uint4(b0.x, b0.y, b1.x, b1.y);
          }
          // the codes of the lane's 16 values: 8 bytes at 128 + 32 H + 8 t of the block (row_a already stands 16 t in)
          const uint2 cd_a = *reinterpret_cast<const uint2*>(row_a + 128u + 32u * H - 8u * t);
          const uint2 cd_b = *reinterpret_cast<const uint2*>(row_b + 128u + 32u * H - 8u * t);
          uint32_t wa[8], wb[8];
          x16_words8(sm_a.x, sm_a.y, cd_a.x, base_a, wa);
          x16_words8(sm_a.z, sm_a.w, cd_a.y, base_a, wa + 4);
          x16_words8(sm_b.x, sm_b.y, cd_b.x, base_b, wb);
          x16_words8(sm_b.z, sm_b.w, cd_b.y, base_b, wb + 4);
          if (min(ca.next, cb.next) < lim) {  // rare: a patch of one of the two rows lies below the end of this lane's values
            const uint32_t k0 = (lim >> 8) - 16u;
            if (ca.next < lim) {
              X16Fix f{ca.next, ca.taken, {wa[0], wa[1], wa[2], wa[3], wa[4], wa[5], wa[6], wa[7]}};
              f = x16_fix16(rec_of(ra), slots, k0, f);
              ca.next = f.next, ca.taken = f.taken;
#pragma unroll
              for (int i = 0; i < 8; ++i) wa[i] = f.w[i];
            }
            if (cb.next < lim) {
              X16Fix f{cb.next, cb.taken, {wb[0], wb[1], wb[2], wb[3], wb[4], wb[5], wb[6], wb[7]}};
              f = x16_fix16(rec_of(rb), slots, k0, f);
              cb.next = f.next, cb.taken = f.taken;
#pragma unroll
              for (int i = 0; i < 8; ++i) wb[i] = f.w[i];
            }
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int c = 0; c < NT; ++c) {
              lds16(xv[c], x_at[c] + xo + 16 * h, x_on[c]);
              mma_step<kMmaBf16>(acc[c], wa[4 * h], wb[4 * h], wa[4 * h + 1], wb[4 * h + 1], xv[c].x, xv[c].y);
              mma_step<kMmaBf16>(acc[c], wa[4 * h + 2], wb[4 * h + 2], wa[4 * h + 3], wb[4 * h + 3], xv[c].z, xv[c].w);
            }
          }
          xo += kXStep, lim += 64u << 8;
        };
        auto open_block = [&] {
          base_a = *base_at_a * 0x01010101u, base_b = *base_at_b * 0x01010101u;
        };
        auto next_block = [&] {
          row_a += 192, row_b += 192, ++base_at_a, ++base_at_b;
        };
        int s = a;
        if (s & 1) {  // the slice begins in the second half of a block
          open_block();
          step(std::integral_constant<uint32_t, 1>{});
          next_block();
          ++s;
        }
#pragma unroll 1
        for (; s + 1 < b; s += 2) {
          open_block();
          step(std::integral_constant<uint32_t, 0>{});
          step(std::integral_constant<uint32_t, 1>{});
          next_block();
        }
        if (s < b) {  // and ends in the first half of one
          open_block();
          step(std::integral_constant<uint32_t, 0>{});
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(ring.slot));
      ring.advance(R.S);
    }
    if (!R.whole && lane == 0) mbar_arrive(hempty_bar(hs));  // after the __syncwarp of the last stage: every lane has read its bases

    // ---- the warp's sums go to the adding warp: no multiplying warp waits for another ----
    x16_wait(taken_bar(u & 1), ((u >> 1) & 1) ^ 1u, dead, R.status);  // the sums of two units ago have been added up
    uint32_t* mine = reinterpret_cast<uint32_t*>(red) + (static_cast<size_t>(u & 1) * kGemvWarps + warp) * kRedStride;
#pragma unroll
    for (int b = 0; b < NT; ++b) {
      const int c = 8 * b + 2 * t;
      *reinterpret_cast<uint2*>(mine + g * COLS + c) = make_uint2(acc[b][0], acc[b][1]);
      *reinterpret_cast<uint2*>(mine + (g + 8) * COLS + c) = make_uint2(acc[b][2], acc[b][3]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(sums_bar(u & 1));
  }
}

}  // namespace
}  // namespace b200
