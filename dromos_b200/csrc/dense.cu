// Dense products of the kernel ABI: lx_gemv_w, lx_gemv, lx_gemv_decode_bf16, lx_gemv_bf16x (M <= 8) and lx_gemm_w,
// lx_gemm_skinny (any M), all on the weight-streaming kernel of stream.cuh, plus a scalar kernel for shapes and
// alignments the streaming kernel does not take (short or odd K, unaligned rows).
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "launch.cuh"
#include "variants.h"

namespace b200 {
namespace {

// ---- scalar path: one warp per weight row, any K, any alignment ------------------------------------------------
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

template <int F>
__global__ void __launch_bounds__(256) scalar_kernel(const StreamParams P) {
  pdl_trigger();
  pdl_wait();
  const int64_t n = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (n >= P.N) return;
  const int lane = threadIdx.x & 31;
  for (int m0 = 0; m0 < P.M; m0 += 8) {
    const int mc = min(8, P.M - m0);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = lane; k < P.K; k += 32) {
      const float wv = weight_element<F>(P, n, k);
#pragma unroll
      for (int m = 0; m < 8; ++m)
        if (m < mc) acc[m] = fmaf(load_f32(P.x, P.x_dtype, static_cast<int64_t>(m0 + m) * P.ld_x + k), wv, acc[m]);
    }
    float rf = 1.0f;
    if constexpr (F == LX_W_INT8 || F == LX_W_FP8) rf = reinterpret_cast<const float*>(P.scale)[n];
    if constexpr (F == LX_W_NVFP4) rf = P.global;
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      if (m >= mc) continue;  // uniform across the warp
      const float sum = warp_sum(acc[m]);
      if (lane == 0) {
        float t = rf * sum;
        if (P.bias) t += load_f32(P.bias, P.bias_dtype, n);
        float v = P.alpha * t;
        const int64_t at = static_cast<int64_t>(m0 + m) * P.ld_y + n;
        if (P.beta != 0.0f) v = fmaf(P.beta, load_f32(P.y, P.y_dtype, at), v);
        store_from_f32(P.y, P.y_dtype, at, v);
      }
    }
  }
}

template <int F>
int launch_scalar(const StreamParams& P, cudaStream_t stream) {
  const unsigned blocks = static_cast<unsigned>((P.N + 7) / 8);
  return launch_kernel(scalar_kernel<F>, dim3(blocks), dim3(256), 0, stream, P);
}

// ---- choosing a streaming configuration ---------------------------------------------------------------------
// Columns a call needs: one per activation row, two for f32 activations (high and low halves).
int columns_needed(int M, int x_dtype) { return x_dtype == LX_BF16 ? M : 2 * M; }

// Can the streaming kernel take this weight? Rows must be whole 64-byte steps and 16-byte aligned (NVFP4 scale rows
// too); BF16X records are 8-byte aligned by contract and K must be whole 32-value steps.
bool stream_ok(const lx_weight& w, int K) {
  switch (w.type) {
    case LX_W_BF16: return K % 32 == 0 && aligned(w.data, 16);
    case LX_W_INT8:
    case LX_W_FP8: return K % 64 == 0 && aligned(w.data, 16);
    case LX_W_NVFP4: return K % 256 == 0 && aligned(w.data, 16) && aligned(w.scale, 16);
    case LX_W_BF16X: return K % 32 == 0 && aligned(w.data, 8);
    default: return false;
  }
}

template <int F>
int launch_dense_format(const StreamParams& P, cudaStream_t stream) {
  const int cols = columns_needed(std::min(P.M, 64), P.x_dtype);
  constexpr int UW = F == LX_W_NVFP4 ? 1 : 2;  // NVFP4 holds four times the values per byte: shorter stages
  if (cols <= 8) {
    // decode GEMV: the variant the table holds for this shape (keyed on M's power-of-two bucket), else variant 0
    switch (lx_tune_get(gemv_kernel_name(F), P.M, P.N, P.K)) {
      case 1: return launch_stream<F, 1, 1, 1, 1, 4, kDense>(P, dim3((P.N + 15) / 16), stream, P.N);
      case 2: return launch_stream<F, 1, 2, 1, 4, 3, kDense>(P, dim3((P.N + 31) / 32), stream, P.N);
      case 3: return launch_stream<F, 1, 4, 1, 4, 3, kDense>(P, dim3((P.N + 63) / 64), stream, P.N);
      case 4: return launch_stream<F, 1, 2, 1, 2, 6, kDense>(P, dim3((P.N + 31) / 32), stream, P.N);
      case 5: return launch_stream<F, 1, 1, 1, 1, 8, kDense>(P, dim3((P.N + 15) / 16), stream, P.N);
      case 6: return launch_stream<F, 1, 4, 1, 2, 4, kDense>(P, dim3((P.N + 63) / 64), stream, P.N);
      case 7: return launch_stream<F, 1, 1, 1, 2, 6, kDense>(P, dim3((P.N + 15) / 16), stream, P.N);
      default: return launch_stream<F, 1, 2, 1, 2, 4, kDense>(P, dim3((P.N + 31) / 32), stream, P.N);
    }
  }
  if (cols <= 16) return launch_stream<F, 1, 2, 2, 2, 4, kDense>(P, dim3((P.N + 31) / 32), stream, P.N);
  if (cols <= 32) return launch_stream<F, 2, 2, 4, UW, 3, kDense>(P, dim3((P.N + 63) / 64), stream, P.N);
  return launch_stream<F, 2, 4, 8, UW, 2, kDense>(P, dim3((P.N + 127) / 128), stream, P.N);
}

int row_bytes_of(int type, int K) {
  switch (type) {
    case LX_W_BF16: return 2 * K;
    case LX_W_NVFP4: return K / 2;
    case LX_W_BF16X: return static_cast<int>(x16::row_bytes(K));
    default: return K;
  }
}

// The product itself, arguments already validated.
int dense_product(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype, void* y,
                  int y_dtype, int ld_y, int M, int N, int K, float alpha, float beta, cudaStream_t stream) {
  StreamParams P{};
  P.w = static_cast<const uint8_t*>(w.data);
  P.scale = static_cast<const uint8_t*>(w.scale);
  P.global = w.global;
  P.expert_global = nullptr;
  P.row_bytes = row_bytes_of(w.type, K);
  P.N = N, P.K = K;
  P.x = x, P.x_dtype = x_dtype, P.ld_x = ld_x, P.M = M;
  P.x_vec = x_dtype == LX_BF16 && aligned(x, 16) && (M == 1 || ld_x % 8 == 0);
  P.bias = bias, P.bias_dtype = bias_dtype;
  P.y = y, P.y_dtype = y_dtype, P.ld_y = ld_y;
  P.alpha = alpha, P.beta = beta;
  P.status = status_word();
  const bool fast = stream_ok(w, K) && !force_scalar();
  switch (w.type) {
    case LX_W_BF16: return fast ? launch_dense_format<LX_W_BF16>(P, stream) : launch_scalar<LX_W_BF16>(P, stream);
    case LX_W_INT8: return fast ? launch_dense_format<LX_W_INT8>(P, stream) : launch_scalar<LX_W_INT8>(P, stream);
    case LX_W_FP8: return fast ? launch_dense_format<LX_W_FP8>(P, stream) : launch_scalar<LX_W_FP8>(P, stream);
    case LX_W_NVFP4: return fast ? launch_dense_format<LX_W_NVFP4>(P, stream) : launch_scalar<LX_W_NVFP4>(P, stream);
    case LX_W_BF16X: return fast ? launch_dense_format<LX_W_BF16X>(P, stream) : launch_scalar<LX_W_BF16X>(P, stream);
  }
  return kInvalid;
}

bool valid_weight(const lx_weight* w, int K, bool allow_x16) {
  if (!w || !w->data) return false;
  switch (w->type) {
    case LX_W_BF16: return true;
    case LX_W_BF16X: return allow_x16 && K < (1 << 23);
    case LX_W_INT8:
    case LX_W_FP8: return w->scale != nullptr;
    case LX_W_NVFP4: return w->scale != nullptr && K % 16 == 0;
    default: return false;
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int lx_gemv_w(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, const void* bias,
                         lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                         float beta, void* stream) {
  if (M == 0 || N == 0) return kOk;
  if (M < 0 || M > 8 || N < 0 || K <= 0 || ld_x < K || ld_y < N) return kInvalid;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype) || !valid_dtype(bias_dtype)) return kInvalid;
  if (!x || !y || !valid_weight(w, K, true)) return kInvalid;
  return dense_product(x, x_dtype, ld_x, *w, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int lx_gemv(const void* x, lx_dtype x_dtype, int ld_x, const void* w, lx_wtype w_type, const float* w_scale,
                       const void* bias, lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K,
                       float alpha, float beta, void* stream) {
  if (w_type != LX_W_BF16 && w_type != LX_W_INT8) return kInvalid;
  lx_weight lw{};
  lw.type = w_type;
  lw.data = w;
  lw.scale = w_scale;
  lw.global = 1.0f;
  return lx_gemv_w(x, x_dtype, ld_x, &lw, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta, stream);
}

extern "C" int lx_gemv_decode_bf16(const void* x, lx_dtype x_dtype, int ld_x, const void* w, const void* bias,
                                   lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K,
                                   float alpha, float beta, void* stream) {
  return lx_gemv(x, x_dtype, ld_x, w, LX_W_BF16, nullptr, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta,
                 stream);
}

extern "C" int lx_gemv_bf16x(const void* x, lx_dtype x_dtype, int ld_x, const void* w, const void* bias,
                             lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                             float beta, void* stream) {
  if (M == 0 || N == 0) return kOk;
  if (!aligned(w, 8)) return kInvalid;
  lx_weight lw{};
  lw.type = LX_W_BF16X;
  lw.data = w;
  lw.global = 1.0f;
  return lx_gemv_w(x, x_dtype, ld_x, &lw, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta, stream);
}

// The activation workspace of lx_gemm_w: where the per-token quantization of the low-precision maths goes (values,
// per-row scales, FP4 block scales, each 256-byte aligned). BF16 math needs none here, but the size answered is the
// reference's so that callers sized for either library work with both.
namespace b200 {
ActLayout act_layout(int M, int K, int math) {
  auto round_up = [](int64_t v, int64_t a) { return (v + a - 1) / a * a; };
  ActLayout l{};
  switch (math) {
    case LX_MATH_BF16: l.ld_q = round_up(static_cast<int64_t>(K) * 2, 16); break;
    case LX_MATH_INT8:
    case LX_MATH_FP8: l.ld_q = round_up(K, 16); break;
    default:
      l.ld_q = round_up((K + 1) / 2, 16);
      l.ld_bs = round_up((K + 15) / 16, 16);
      break;
  }
  l.q_off = 0;
  l.scale_off = round_up(l.q_off + l.ld_q * M, 256);
  l.bs_off = round_up(l.scale_off + 4 * static_cast<int64_t>(M), 256);
  l.total = round_up(l.bs_off + l.ld_bs * M, 256);
  return l;
}
}  // namespace b200

extern "C" int64_t lx_gemm_workspace_bytes(int M, int K, lx_math math) {
  if (M <= 0 || K <= 0) return 0;
  return act_layout(M, K, math).total;
}

extern "C" int lx_gemm_w(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, lx_math math, const void* bias,
                         lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                         float beta, void* workspace, void* stream) {
  (void)workspace;
  if (M < 0 || N < 0 || K <= 0 || ld_x < K || ld_y < N || !w) return kInvalid;
  if (M == 0 || N == 0) return kOk;
  if (!x || !y || !w->data) return kInvalid;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype) || (bias && !valid_dtype(bias_dtype))) return kInvalid;
  if (math < LX_MATH_BF16 || math > LX_MATH_FP4) return kInvalid;
  if (w->type < LX_W_BF16 || w->type > LX_W_NVFP4) return kNotSupported;
  if (math != LX_MATH_BF16) return kNotSupported;  // activations stay bf16: weight-only products
  if (w->type != LX_W_BF16 && !w->scale) return kInvalid;
  // Weight rows must be whole 16-byte chunks, as for the reference's tensor-core kernels.
  const int64_t rowb = row_bytes_of(w->type, K);
  if (rowb % 16 != 0 || !aligned(w->data, 16) || (w->type == LX_W_NVFP4 && K % 64 != 0)) return kNotSupported;
  return dense_product(x, x_dtype, ld_x, *w, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int lx_gemm_skinny(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, const void* bias,
                              lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                              float beta, void* stream) {
  if (M < 0 || N < 0 || K <= 0 || ld_x < K || ld_y < N || !w) return kInvalid;
  if (M == 0 || N == 0) return kOk;
  if (!x || !y || !w->data) return kInvalid;
  if (!valid_dtype(y_dtype) || (bias && !valid_dtype(bias_dtype))) return kInvalid;
  if (w->type != LX_W_BF16 || x_dtype != LX_BF16 || N % 16 != 0 || K % 64 != 0) return kNotSupported;
  return dense_product(x, x_dtype, ld_x, *w, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta,
                       static_cast<cudaStream_t>(stream));
}
