// Load-time conversions of the kernel ABI: lx_quantize_weight, lx_dequantize_weight, lx_quantize_w8 and the per-token
// activation quantizer lx_quantize_act. Every rounding is to nearest, ties to even, saturating; weight quantizers
// divide with IEEE division, the FP4 activation quantizer multiplies by the block's reciprocal (the ABI's rules:
// lernex/dromos engine/cuda/kernels.h:479-493, 513-523).
#include <algorithm>

#include "launch.cuh"

namespace b200 {
namespace {

constexpr int kBlock = 256;

// Nearest e2m1 code (0, .5, 1, 1.5, 2, 3, 4, 6 with a sign bit): the code is how many midpoints lie below |x|, a
// value on a midpoint goes to the even neighbour, magnitudes saturate at 6, and a zero result carries no sign.
__device__ __forceinline__ uint32_t e2m1_encode(float x) {
  const float a = fminf(fabsf(x), 6.0f);
  uint32_t code = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
  return code | ((x < 0.0f && code) ? 8u : 0u);
}

// One warp per row: the row's absmax, then its values. kFp8: e4m3 with scale absmax / 448; else int8, absmax / 127.
template <bool kFp8>
__global__ void __launch_bounds__(kBlock) quantize_rows_kernel(const uint16_t* __restrict__ w, uint8_t* __restrict__ q,
                                                               float* __restrict__ scale, int64_t rows, int cols) {
  // no early trigger: what this kernel writes may be the weight of the next product, whose kernels read weights
  // before their own wait
  pdl_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kBlock / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint16_t* src = w + row * cols;
  float amax = 0.0f;
  for (int c = lane; c < cols; c += 32) amax = fmaxf(amax, fabsf(bf16_bits_to_f32(src[c])));
  amax = warp_max(amax);
  constexpr float qmax = kFp8 ? 448.0f : 127.0f;
  const float s = amax > 0.0f ? __fdiv_rn(amax, qmax) : 1.0f;
  if (lane == 0) scale[row] = s;
  uint8_t* dst = q + row * cols;
  for (int c = lane; c < cols; c += 32) {
    const float v = __fdiv_rn(bf16_bits_to_f32(src[c]), s);
    if constexpr (kFp8) {
      dst[c] = static_cast<uint8_t>(e4m3_encode(fminf(fmaxf(v, -448.0f), 448.0f)));
    } else {
      dst[c] = static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(fminf(fmaxf(rintf(v), -127.0f), 127.0f))));
    }
  }
}

// max |w| of the whole matrix, as the bit pattern of a non-negative float (which orders like the value).
__global__ void __launch_bounds__(kBlock) absmax_kernel(const uint16_t* __restrict__ w, int64_t n, unsigned int* out) {
  // no early trigger: what this kernel writes may be the weight of the next product, whose kernels read weights
  // before their own wait
  pdl_wait();
  float m = 0.0f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * kBlock)
    m = fmaxf(m, fabsf(bf16_bits_to_f32(w[i])));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(m));
}

// One thread per 16-value block: the block's e4m3 scale (absmax / (6 * global)), then its codes, w / (scale * global).
__global__ void __launch_bounds__(kBlock) quantize_nvfp4_kernel(const uint16_t* __restrict__ w, uint8_t* __restrict__ q,
                                                                uint8_t* __restrict__ scale, float global, int64_t rows,
                                                                int cols) {
  // no early trigger: what this kernel writes may be the weight of the next product, whose kernels read weights
  // before their own wait
  pdl_wait();
  const int64_t per_row = cols / 16;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x;
  if (i >= rows * per_row) return;
  const uint16_t* src = w + i * 16;
  float v[16], amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    v[j] = bf16_bits_to_f32(src[j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
  const uint32_t sb = e4m3_encode(__fdiv_rn(amax, 6.0f * global));
  scale[i] = static_cast<uint8_t>(sb);
  const float eff = e4m3_to_f32(sb) * global;
  uint8_t* dst = q + i * 8;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    uint32_t lo = 0, hi = 0;
    if (eff > 0.0f) {
      lo = e2m1_encode(__fdiv_rn(v[2 * p], eff));
      hi = e2m1_encode(__fdiv_rn(v[2 * p + 1], eff));
    }
    dst[p] = static_cast<uint8_t>(lo | (hi << 4));
  }
}

// out[n, k] = bf16(element * row factor), one thread per element.
template <int F>
__global__ void __launch_bounds__(kBlock) dequantize_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scale,
                                                            float global, uint16_t* __restrict__ out, int64_t rows, int cols) {
  // no early trigger: what this kernel writes may be the weight of the next product, whose kernels read weights
  // before their own wait
  pdl_wait();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x;
  if (i >= rows * cols) return;
  const int64_t n = i / cols, k = i % cols;
  float v;
  if constexpr (F == LX_W_INT8) {
    v = static_cast<float>(reinterpret_cast<const int8_t*>(data)[i]) * reinterpret_cast<const float*>(scale)[n];
  } else if constexpr (F == LX_W_FP8) {
    v = e4m3_to_f32(data[i]) * reinterpret_cast<const float*>(scale)[n];
  } else {
    const uint32_t byte = data[n * (cols / 2) + k / 2];
    v = e2m1_to_f32((k & 1) ? byte >> 4 : byte & 15u) * e4m3_to_f32(scale[n * (cols / 16) + k / 16]) * global;
  }
  out[i] = static_cast<uint16_t>(f32_to_bf16_bits(v));
}

// One CTA per activation row: absmax, then the row's values in the math's number type.
__global__ void __launch_bounds__(kBlock) quantize_act_kernel(const void* __restrict__ x, int x_dtype, int ld_x, int math,
                                                              uint8_t* __restrict__ q, int ld_q, float* __restrict__ scale,
                                                              uint8_t* __restrict__ block_scale, int ld_bs, int K) {
  // no early trigger: what this kernel writes may be the weight of the next product, whose kernels read weights
  // before their own wait
  pdl_wait();
  __shared__ float part[kBlock / 32];
  const int m = blockIdx.x;
  const int64_t base = static_cast<int64_t>(m) * ld_x;
  float a = 0.0f;
  for (int k = threadIdx.x; k < K; k += kBlock) a = fmaxf(a, fabsf(load_f32(x, x_dtype, base + k)));
  a = warp_max(a);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = a;
  __syncthreads();
  a = 0.0f;
  for (int i = 0; i < kBlock / 32; ++i) a = fmaxf(a, part[i]);
  uint8_t* qr = q + static_cast<int64_t>(m) * ld_q;
  if (math == LX_MATH_INT8 || math == LX_MATH_FP8) {
    const float qmax = math == LX_MATH_INT8 ? 127.0f : 448.0f;
    const float inv = a > 0.0f ? __fdiv_rn(qmax, a) : 0.0f;
    for (int k = threadIdx.x; k < K; k += kBlock) {
      const float v = load_f32(x, x_dtype, base + k) * inv;
      if (math == LX_MATH_INT8)
        qr[k] = static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(fminf(fmaxf(rintf(v), -127.0f), 127.0f))));
      else
        qr[k] = static_cast<uint8_t>(e4m3_encode(v));
    }
    if (threadIdx.x == 0) scale[m] = a > 0.0f ? __fdiv_rn(a, qmax) : 1.0f;
    return;
  }
  const float g = a > 0.0f ? __fdiv_rn(a, 2688.0f) : 1.0f;
  if (threadIdx.x == 0) scale[m] = g;
  uint8_t* bs = block_scale + static_cast<int64_t>(m) * ld_bs;
  for (int b = threadIdx.x; b < K / 16; b += kBlock) {
    float v[16], amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = load_f32(x, x_dtype, base + 16 * b + j);
      amax = fmaxf(amax, fabsf(v[j]));
    }
    const uint32_t s8 = e4m3_encode(__fdiv_rn(amax, 6.0f * g));
    bs[b] = static_cast<uint8_t>(s8);
    const float d = e4m3_to_f32(s8) * g;
    const float r = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      uint32_t lo = 0, hi = 0;
      if (d > 0.0f) {
        lo = e2m1_encode(v[2 * p] * r);
        hi = e2m1_encode(v[2 * p + 1] * r);
      }
      qr[8 * b + p] = static_cast<uint8_t>(lo | (hi << 4));
    }
  }
}

unsigned blocks_for(int64_t n, int per_block) { return static_cast<unsigned>((n + per_block - 1) / per_block); }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int lx_quantize_w8(const void* w, int8_t* q, float* scale, int64_t rows, int cols, void* stream) {
  if (rows <= 0) return kOk;
  if (cols <= 0 || !w || !q || !scale) return kInvalid;
  return launch_kernel(quantize_rows_kernel<false>, dim3(blocks_for(rows, kBlock / 32)), dim3(kBlock), 0,
                       static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(w), reinterpret_cast<uint8_t*>(q),
                       scale, rows, cols);
}

extern "C" int lx_quantize_weight(const void* w, lx_weight* out, int64_t rows, int cols, void* stream) {
  if (!out || !w) return kInvalid;
  if (rows <= 0) return kOk;
  if (cols <= 0) return kInvalid;
  auto s = static_cast<cudaStream_t>(stream);
  auto* data = static_cast<uint8_t*>(const_cast<void*>(out->data));
  auto* scale = const_cast<void*>(out->scale);
  const auto* src = static_cast<const uint16_t*>(w);
  switch (out->type) {
    case LX_W_BF16X: {
      if (!data) return kInvalid;
      const int64_t bytes = lx_bf16x_bytes(w, rows, cols, stream);
      if (bytes < 0) return static_cast<int>(-bytes);
      return lx_bf16x_encode(w, rows, cols, data, bytes, stream);
    }
    case LX_W_INT8:
      if (!data || !scale) return kInvalid;
      return lx_quantize_w8(w, reinterpret_cast<int8_t*>(data), static_cast<float*>(scale), rows, cols, stream);
    case LX_W_FP8:
      if (!data || !scale) return kInvalid;
      return launch_kernel(quantize_rows_kernel<true>, dim3(blocks_for(rows, kBlock / 32)), dim3(kBlock), 0, s, src, data,
                           static_cast<float*>(scale), rows, cols);
    case LX_W_NVFP4: {
      if (!data || !scale || cols % 16 != 0) return kInvalid;
      // The global scale is max|w| / (448 * 6); it is a host field of lx_weight, so this load-time call reads the
      // maximum back (it synchronizes the stream). The scratch word comes from the stream's memory pool.
      unsigned int* amax_dev = nullptr;
      if (cudaMallocAsync(&amax_dev, sizeof(unsigned int), s) != cudaSuccess) return static_cast<int>(cudaGetLastError());
      cudaMemsetAsync(amax_dev, 0, sizeof(unsigned int), s);
      const int64_t n = rows * cols;
      int e = launch_kernel(absmax_kernel, dim3(std::min<unsigned>(blocks_for(n, kBlock), 148 * 8)), dim3(kBlock), 0, s,
                            src, n, amax_dev);
      unsigned int bits = 0;
      cudaMemcpyAsync(&bits, amax_dev, sizeof(bits), cudaMemcpyDeviceToHost, s);
      const cudaError_t sync = cudaStreamSynchronize(s);
      cudaFreeAsync(amax_dev, s);
      if (e) return e;
      if (sync != cudaSuccess) return static_cast<int>(sync);
      float amax;
      memcpy(&amax, &bits, sizeof(amax));
      const float global = amax / 2688.0f;
      out->global = global;
      return launch_kernel(quantize_nvfp4_kernel, dim3(blocks_for(rows * (cols / 16), kBlock)), dim3(kBlock), 0, s, src,
                           data, static_cast<uint8_t*>(scale), global, rows, cols);
    }
    default:
      return kInvalid;  // BF16: nothing to quantize
  }
}

extern "C" int lx_dequantize_weight(const lx_weight* w, void* out, int64_t rows, int cols, void* stream) {
  if (!w || !w->data || !out) return kInvalid;
  if (rows <= 0) return kOk;
  if (cols <= 0) return kInvalid;
  if (w->type < LX_W_BF16 || w->type > LX_W_BF16X) return kInvalid;
  if (w->type != LX_W_BF16 && w->type != LX_W_BF16X && !w->scale) return kInvalid;
  if (w->type == LX_W_NVFP4 && cols % 16 != 0) return kInvalid;
  auto s = static_cast<cudaStream_t>(stream);
  if (w->type == LX_W_BF16X) return lx_bf16x_decode(w->data, rows, cols, out, stream);
  if (w->type == LX_W_BF16)
    return static_cast<int>(cudaMemcpyAsync(out, w->data, 2 * rows * cols, cudaMemcpyDeviceToDevice, s));
  const dim3 grid(blocks_for(rows * cols, kBlock));
  const auto* data = static_cast<const uint8_t*>(w->data);
  const auto* scale = static_cast<const uint8_t*>(w->scale);
  auto* o = static_cast<uint16_t*>(out);
  switch (w->type) {
    case LX_W_INT8: return launch_kernel(dequantize_kernel<LX_W_INT8>, grid, dim3(kBlock), 0, s, data, scale, 1.0f, o, rows, cols);
    case LX_W_FP8: return launch_kernel(dequantize_kernel<LX_W_FP8>, grid, dim3(kBlock), 0, s, data, scale, 1.0f, o, rows, cols);
    default: return launch_kernel(dequantize_kernel<LX_W_NVFP4>, grid, dim3(kBlock), 0, s, data, scale, w->global, o, rows, cols);
  }
}

extern "C" int lx_quantize_act(const void* x, lx_dtype x_dtype, int ld_x, lx_math math, void* q, int ld_q, float* scale,
                               void* block_scale, int ld_bs, int M, int K, void* stream) {
  if (M <= 0) return kOk;
  if (!x || !q || !scale || K <= 0 || !valid_dtype(x_dtype) || (M > 1 && ld_x < K)) return kInvalid;
  if (math != LX_MATH_INT8 && math != LX_MATH_FP8 && math != LX_MATH_FP4) return kInvalid;
  if (math == LX_MATH_FP4) {
    if (K % 16 != 0 || !block_scale || (M > 1 && (ld_q < K / 2 || ld_bs < K / 16))) return kInvalid;
  } else if (M > 1 && ld_q < K) {
    return kInvalid;
  }
  return launch_kernel(quantize_act_kernel, dim3(M), dim3(kBlock), 0, static_cast<cudaStream_t>(stream), x,
                       static_cast<int>(x_dtype), ld_x, static_cast<int>(math), static_cast<uint8_t*>(q), ld_q, scale,
                       static_cast<uint8_t*>(block_scale), ld_bs, K);
}
