// Element-wise decoding of every weight format, for the scalar kernels that take the shapes and alignments the
// streaming kernel does not (short or odd K, unaligned rows).
#pragma once

#include "stream.cuh"

namespace b200 {

// Element k of weight row n as f32 without the row factor.
template <int F>
__device__ __forceinline__ float weight_element(const StreamParams& P, int64_t n, int k) {
  const int K = P.K;
  if constexpr (F == LX_W_BF16) {
    return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(P.w)[n * K + k]);
  } else if constexpr (F == LX_W_INT8) {
    return static_cast<float>(reinterpret_cast<const int8_t*>(P.w)[n * K + k]);
  } else if constexpr (F == LX_W_FP8) {
    return e4m3_to_f32(P.w[n * K + k]);
  } else if constexpr (F == LX_W_NVFP4) {
    const uint32_t byte = P.w[n * (K / 2) + k / 2];
    return e2m1_to_f32((k & 1) ? (byte >> 4) : (byte & 15u)) * e4m3_to_f32(P.scale[n * (K / 16) + k / 16]);
  } else {
    // BF16X: sign|mantissa byte, 4-bit code below the block's base exponent, then the row's patches
    const uint8_t* rec = P.w + n * P.row_bytes;
    const int H = x16::header_bytes(K), slots = x16::patch_slots(K);
    const int blk = k >> 7, off = k & 127;
    const uint8_t* b = rec + H + blk * 192;
    const uint32_t sm = b[off];
    const uint32_t cbyte = b[128 + (off >> 3) * 4 + (off & 3)];
    const uint32_t code = (off & 4) ? cbyte >> 4 : cbyte & 15u;
    uint32_t e = (rec[4 * slots + blk] - code) & 0xffu;
    const uint32_t* list = reinterpret_cast<const uint32_t*>(rec);
    int n_list = slots;
    const uint32_t s0 = list[0];
    if (s0 != x16::kNoPatch && (s0 & 0x80000000u)) {
      const uint32_t* r = reinterpret_cast<const uint32_t*>(rec + static_cast<int64_t>(s0 & 0x7fffffffu) * 8);
      n_list = static_cast<int>(r[0]);
      list = r + 1;
    }
    for (int i = 0; i < n_list; ++i) {
      const uint32_t p = list[i];
      if (p == x16::kNoPatch || (p >> 8) > static_cast<uint32_t>(k)) break;
      if ((p >> 8) == static_cast<uint32_t>(k)) e = p & 0xffu;
    }
    return __uint_as_float(((sm & 0x80u) << 24) | (e << 23) | ((sm & 0x7fu) << 16));
  }
}


// The per-row factor of row n of expert e (rows counted over the whole stack).
template <int F>
__device__ __forceinline__ float scalar_row_factor(const StreamParams& P, int64_t n, int e) {
  if constexpr (F == LX_W_INT8 || F == LX_W_FP8) return reinterpret_cast<const float*>(P.scale)[n];
  else if constexpr (F == LX_W_NVFP4) return P.expert_global ? P.expert_global[e] : P.global;
  else return 1.0f;
}

}  // namespace b200
