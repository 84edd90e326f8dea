// The decode GEMV of the 8-bit formats (LX_W_INT8, LX_W_FP8) and of LX_W_NVFP4 for rows short enough, M = 1..8: gemv_kernel's
// sums (gemv.cuh) on units that one bulk copy each (NVFP4: one for the values, one for their block scales) brings into
// shared memory.
//
// Why. A unit of gemv_kernel is 16 rows x K bytes; at K = 4096 that is two 128-value steps per warp: one batch of loads,
// one round trip to memory, then the meeting of the 16 slices, the epilogue and only then the next unit's loads. With so
// little per unit the fixed part dominates: measured on a 14336 x 4096 matrix (58.8 MB, 9 us to stream) 18.5 us for FP8
// where the same kernel streams K = 8192 rows at 0.87 of the copy bandwidth. Here the three roles of gemv_x16.cuh take that
// apart: warp 16 copies unit after unit (a unit's 16 rows are one contiguous run: ONE cp.async.bulk, no multicast) into a
// ring of 2..6 slots, warps 0..15 multiply from shared memory and never wait for one another, warp 17 adds the 16 slices
// of a unit in warp order and stores y.
//
// Everything that sets a sum is gemv_kernel's for the same format: the 16 slices of K cut at the same steps, lane (g, t)
// holding bytes 32 t .. 32 t + 31 of each 128-byte step of rows g and g + 8, expanded to f16 pairs the same way and
// multiplied in the same order against the same staged activations (gemv_stage_x), the epilogue's operations in the
// same order. So a row's bits are gemv_kernel's, whichever of the two runs. NVFP4 (16 bytes per lane, row and step, one
// pair of e4m3 block scales per lane and row) has a second reason to come this way: a warp's 16-byte loads of 8 rows ask
// for half a line each, as the lossless format's do (gemv_x16.cuh).
//
// Every wait is bounded (x16_wait: 0.25 s, then status 5 and no more waiting in this CTA); the copying warp waits, bounded,
// for its own copies before it leaves.
#pragma once

#include "gemv_x16.cuh"

namespace b200 {
namespace {

struct Ring8 {
  int S;                 // ring slots, each 16 rows of values (and, NVFP4, of block scales after them)
  uint32_t slot_bytes;
  uint32_t scale_off;    // NVFP4: where the 16 rows of block scales start within a slot
  uint32_t ring_off, bar_off;  // from the start of dynamic shared memory
  int* status;
};

// false when two units do not fit beside the activation columns
inline bool ring8_for(int K, int wtype, int ncols, Ring8& r, size_t& smem_total) {
  const uint32_t fixed = static_cast<uint32_t>((gemv_smem(K, wtype, ncols) + 127) / 128 * 128);
  const uint32_t room = 226u * 1024u - 256u;
  const uint32_t values = 16u * static_cast<uint32_t>(wtype == LX_W_NVFP4 ? K / 2 : K);
  r.scale_off = values;
  r.slot_bytes = values + (wtype == LX_W_NVFP4 ? static_cast<uint32_t>(K) : 0u);  // 16 rows x K / 16 scale bytes
  r.ring_off = fixed;
  if (fixed + 2u * r.slot_bytes > room) return false;
  r.S = static_cast<int>(std::min<uint32_t>(6u, (room - fixed) / r.slot_bytes));
  r.bar_off = r.ring_off + static_cast<uint32_t>(r.S) * r.slot_bytes;
  smem_total = r.bar_off + 8u * (2u * r.S + 4u) + 16u;
  return true;
}

// F: LX_W_INT8 or LX_W_FP8 (one byte per value, K % 128 == 0, rows K bytes apart, the matrix 16-byte aligned) or LX_W_NVFP4
// (K % 256 == 0, values and scales 16-byte aligned).
// NT: 8-column tiles of activations.
template <int F, int NT>
__global__ void __launch_bounds__(kX16Threads, 1) gemv_ring8_kernel(const GemvParams P, const Ring8 R) {
  using Fm = GemvFmt<F>;
  constexpr bool kFp4 = F == LX_W_NVFP4;
  static_assert(Fm::kMma == kMmaF16 && Fm::kLane == (kFp4 ? 16 : 32) && Fm::kSwz == 1, "formats expanded to f16 pairs");
  constexpr uint32_t kWStep = 4 * Fm::kLane;  // bytes of a row per step
  constexpr int COLS = 8 * NT;
  constexpr int kXStep = Fm::kXStep;
  constexpr int kRedStride = kGemvRedStride(NT);
  extern __shared__ __align__(128) uint8_t smem[];
  float* red = reinterpret_cast<float*>(smem);                    // [2][16 warps][16 rows][COLS] (+ 2 words per warp)
  float* inv_scale = red + 2 * kGemvWarps * kRedStride;           // [8]
  float* part = inv_scale + 8;
  uint8_t* xs = reinterpret_cast<uint8_t*>(part + 8 * kGemvWarps + 16);
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t bars = smem0 + R.bar_off;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (R.S + s); };
  auto sums_bar = [&](int s) { return bars + 8u * (2 * R.S + s); };       // a unit's 16 partial sums are written
  auto taken_bar = [&](int s) { return bars + 8u * (2 * R.S + 2 + s); };  // and have been added up
  volatile int* dead = reinterpret_cast<volatile int*>(smem + R.bar_off + 8u * (2 * R.S + 4));

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < R.S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kGemvWarps);
    }
    for (int s = 0; s < 2; ++s) {
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
  const uint32_t row_bytes = static_cast<uint32_t>(P.row_bytes);
  const uint32_t scale_row = kFp4 ? static_cast<uint32_t>(P.K / 16) : 0u;  // bytes of a row's block scales

  if (warp == kGemvWarps) {
    // ---- the copying warp: weights are static, so it does not wait for the kernel before ----
    Ring ring;
    for (int u = 0; u < n_units; ++u) {
      const int row0 = cta_row0 + kGemvUnitRows * u;
      const int nrows = min(kGemvUnitRows, my_rows - kGemvUnitRows * u);
      x16_wait(empty_bar(ring.slot), ring.lap ^ 1u, dead, R.status);
      if (lane == 0) {
        const uint32_t bytes = static_cast<uint32_t>(nrows) * row_bytes;  // a multiple of 64
        const uint32_t sbytes = kFp4 ? static_cast<uint32_t>(nrows) * scale_row : 0u;  // of 16
        mbar_arrive_expect_tx(full_bar(ring.slot), bytes + sbytes);
        bulk_g2s(smem0 + R.ring_off + ring.slot * R.slot_bytes, P.w + static_cast<int64_t>(row0) * P.row_bytes, bytes, full_bar(ring.slot));
        if constexpr (kFp4)
          bulk_g2s(smem0 + R.ring_off + ring.slot * R.slot_bytes + R.scale_off, P.scale + static_cast<int64_t>(row0) * scale_row, sbytes, full_bar(ring.slot));
      }
      ring.advance(R.S);
    }
    Ring back;
    for (int i = 0; i < n_units; ++i) {
      if (i >= n_units - R.S) x16_wait(full_bar(back.slot), back.lap, dead, R.status, true);
      back.advance(R.S);
    }
    return;
  }

  if (warp == kGemvWarps + 1) {
    // ---- the adding warp: gemv_kernel's epilogue, 32 outputs at a time ----
    pdl_wait();  // y may still be in use by the kernel before
    const int T = P.planes;
    for (int u = 0; u < n_units; ++u) {
      const int row0 = cta_row0 + kGemvUnitRows * u;
      const int nrows = min(kGemvUnitRows, my_rows - kGemvUnitRows * u);
      const int rs = u & 1;
      // what the outputs of this lane's first round want from global memory is asked for before the wait
      float rf0 = 1.0f, bias0 = 0.0f;
      if (lane < 16 * P.M && (lane & 15) < nrows) {
        if constexpr (kFp4) rf0 = P.global;
        else rf0 = __ldg(reinterpret_cast<const float*>(P.scale) + row0 + (lane & 15));
        if (P.bias) bias0 = load_f32(P.bias, P.bias_dtype, row0 + (lane & 15));
      }
      x16_wait(sums_bar(rs), (u >> 1) & 1, dead, R.status);
      const uint32_t* all = reinterpret_cast<const uint32_t*>(red) + static_cast<size_t>(rs) * kGemvWarps * kRedStride;
      for (int o = lane; o < 16 * P.M; o += 32) {
        const int out_m = o >> 4, out_r = o & 15;  // out_r is the same in every round of a lane
        if (out_r >= nrows) continue;
        float sum = 0.0f, dw = 1.0f;
        for (int term = 0; term < T; ++term) {
          const int at = out_r * COLS + out_m * T + term;
          float p = 0.0f;
#pragma unroll
          for (int w = 0; w < kGemvWarps; ++w) p += __uint_as_float(all[w * kRedStride + at]);
          sum += p * dw;
          dw *= 1.0f;
        }
        sum *= inv_scale[out_m];
        float tval = rf0 * sum;
        if (P.bias) tval += bias0;
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
  if (P.x_dtype == LX_BF16) gemv_stage_x<kActF16, true, true, true>(P, xs, inv_scale, part, tid);
  else gemv_stage_x<kActF16, false, true, true>(P, xs, inv_scale, part, tid);
  uint32_t x_on[NT], x_at[NT];
  uint4 xv[NT];
#pragma unroll
  for (int b = 0; b < NT; ++b) {
    const int col = 8 * b + g;
    x_on[b] = col < P.ncols ? 1u : 0u;
    x_at[b] = smem_u32(xs) + static_cast<uint32_t>(min(col, P.ncols - 1)) * static_cast<uint32_t>(P.pitch) + static_cast<uint32_t>(t) * (kXStep / 4);
    xv[b] = make_uint4(0, 0, 0, 0);
  }

  Ring ring;
  for (int u = 0; u < n_units; ++u) {
    const int nrows = min(kGemvUnitRows, my_rows - kGemvUnitRows * u);
    const int ra = min(g, nrows - 1), rb = min(g + 8, nrows - 1);  // a lane past the unit's end reads its last row again
    uint32_t acc[NT][4];
#pragma unroll
    for (int b = 0; b < NT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[b][c] = 0u;

    x16_wait(full_bar(ring.slot), ring.lap, dead, R.status);
    const uint8_t* slot = smem + R.ring_off + ring.slot * R.slot_bytes;
    const uint8_t* pa = slot + static_cast<uint32_t>(ra) * row_bytes + static_cast<uint32_t>(s0) * kWStep + Fm::kLane * t;
    const uint8_t* pb = slot + static_cast<uint32_t>(rb) * row_bytes + static_cast<uint32_t>(s0) * kWStep + Fm::kLane * t;
    // NVFP4: the lane's two block scales of a step (values 32 c .. 32 c + 31, c = 4 s + t)
    const uint8_t* sa = slot + R.scale_off + static_cast<uint32_t>(ra) * scale_row + 2u * (4u * s0 + t);
    const uint8_t* sb = slot + R.scale_off + static_cast<uint32_t>(rb) * scale_row + 2u * (4u * s0 + t);
    uint32_t xo = static_cast<uint32_t>(s0) * kXStep;
#pragma unroll 2
    for (int s = s0; s < s1; ++s) {
      uint32_t qa[8], qb[8];
      uint32_t sa_lo = 0, sa_hi = 0, sb_lo = 0, sb_hi = 0;
      {
        const uint4 a0 = *reinterpret_cast<const uint4*>(pa), b0 = *reinterpret_cast<const uint4*>(pb);
        qa[0] = a0.x, qa[1] = a0.y, qa[2] = a0.z, qa[3] = a0.w;
        qb[0] = b0.x, qb[1] = b0.y, qb[2] = b0.z, qb[3] = b0.w;
      }
      if constexpr (kFp4) {
        const uint32_t ea = *reinterpret_cast<const uint16_t*>(sa), eb = *reinterpret_cast<const uint16_t*>(sb);
        uint32_t sa2, sb2;
        asm("{ .reg .b16 h; cvt.u16.u32 h, %1; cvt.rn.f16x2.e4m3x2 %0, h; }" : "=r"(sa2) : "r"(ea));
        asm("{ .reg .b16 h; cvt.u16.u32 h, %1; cvt.rn.f16x2.e4m3x2 %0, h; }" : "=r"(sb2) : "r"(eb));
        sa_lo = __byte_perm(sa2, sa2, 0x1010), sa_hi = __byte_perm(sa2, sa2, 0x3232);
        sb_lo = __byte_perm(sb2, sb2, 0x1010), sb_hi = __byte_perm(sb2, sb2, 0x3232);
      } else {
        const uint4 a1 = *reinterpret_cast<const uint4*>(pa + 16), b1 = *reinterpret_cast<const uint4*>(pb + 16);
        qa[4] = a1.x, qa[5] = a1.y, qa[6] = a1.z, qa[7] = a1.w;
        qb[4] = b1.x, qb[5] = b1.y, qb[6] = b1.z, qb[7] = b1.w;
      }
      // the lane's 32 values per row against 64 bytes of f16 activations, 8 values (one 16-byte piece, stored rotated by
      // t) at a time. 8-bit: words 2 i and 2 i + 1 of the 32 bytes. NVFP4: word i of the 16 bytes, times the first
      // (i < 2) or second block scale.
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int b = 0; b < NT; ++b) lds16(xv[b], x_at[b] + xo + 16 * ((i + t) & 3), x_on[b]);
        uint32_t pa4[4], pb4[4];
        if constexpr (kFp4) {
          nvfp4_expand8(qa[i], i < 2 ? sa_lo : sa_hi, pa4);
          nvfp4_expand8(qb[i], i < 2 ? sb_lo : sb_hi, pb4);
        } else if constexpr (F == LX_W_INT8) {
          s8_expand4(qa[2 * i], pa4[0], pa4[1]);
          s8_expand4(qa[2 * i + 1], pa4[2], pa4[3]);
          s8_expand4(qb[2 * i], pb4[0], pb4[1]);
          s8_expand4(qb[2 * i + 1], pb4[2], pb4[3]);
        } else {
          e4m3_expand4(qa[2 * i], pa4[0], pa4[1]);
          e4m3_expand4(qa[2 * i + 1], pa4[2], pa4[3]);
          e4m3_expand4(qb[2 * i], pb4[0], pb4[1]);
          e4m3_expand4(qb[2 * i + 1], pb4[2], pb4[3]);
        }
#pragma unroll
        for (int b = 0; b < NT; ++b) {
          mma_step<kMmaF16>(acc[b], pa4[0], pb4[0], pa4[1], pb4[1], xv[b].x, xv[b].y);
          mma_step<kMmaF16>(acc[b], pa4[2], pb4[2], pa4[3], pb4[3], xv[b].z, xv[b].w);
        }
      }
      pa += kWStep, pb += kWStep, sa += 8, sb += 8, xo += kXStep;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(ring.slot));
    ring.advance(R.S);

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
