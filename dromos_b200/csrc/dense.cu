// Dense products of the kernel ABI: lx_gemv_w, lx_gemv, lx_gemv_decode_bf16, lx_gemv_bf16x (M <= 8) and lx_gemm_w,
// lx_gemm_skinny (any M), all on the weight-streaming kernel of stream.cuh, plus a scalar kernel for shapes and
// alignments the streaming kernel does not take (short or odd K, unaligned rows).
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "launch.cuh"
#include "scalar.cuh"
#include "variants.h"

namespace b200 {
namespace {

// ---- scalar path: one warp per weight row, any K, any alignment ------------------------------------------------
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
  constexpr int kMma = Fmt<F>::kMma;
  constexpr bool k8 = kMma == kMmaE4m3 || kMma == kMmaS8;
  // Columns the call needs: one per activation row and digit (see stream.cuh); more than 64 are served in passes.
  const int T = terms_for(kMma, P.x_dtype == LX_BF16);
  const int cols = std::min(P.M * T, 64);
  // NVFP4 holds four times the values per byte, so its stages span four times the K: shorter stages for wide tiles.
  constexpr int UW = F == LX_W_NVFP4 ? 1 : 2;
  if (cols <= 8) {
    // Bytes of activation units for the whole of K; up to 32 KB stays resident in the small buffer.
    const int64_t unit_bytes = static_cast<int64_t>(P.K) / (k8 ? 16 : 8) * 16 * cols;
    const bool big_x = unit_bytes > 32 * 1024;
    const int tuned = lx_tune_get(gemv_kernel_name(F), P.M, P.N, P.K);
    if (tuned < 0) {
      // Defaults. A format keeps ONE warp layout (consumer warps, warp rows, steps per stage: what fixes the order a
      // row's products are added in) for every M = 1..8, with the large activation buffer when the rows need it, so a
      // row's bits do not depend on its batch; BF16 and BF16X share theirs, so the lossless format reproduces bf16's
      // bits. Picked from sweeps of the variants at M = 1 on the decode shapes.
      if constexpr (F == LX_W_BF16 || F == LX_W_BF16X)
        return big_x ? launch_stream<F, 16, 1, 2, 1, 2, 2, 64, kDense>(P, stream, P.N) : launch_stream<F, 16, 1, 2, 1, 2, 5, 16, kDense>(P, stream, P.N);
      if constexpr (F == LX_W_NVFP4)
        return big_x ? launch_stream<F, 16, 1, 4, 1, 2, 2, 64, kDense>(P, stream, P.N) : launch_stream<F, 16, 1, 4, 1, 2, 4, 16, kDense>(P, stream, P.N);
    }
    if (big_x) return launch_stream<F, 8, 1, 2, 1, 2, 4, 64, kDense>(P, stream, P.N);
    // decode GEMV: the variant the table holds for this shape (keyed on M's power-of-two bucket), else variant 0
    switch (tuned) {
      case 1: return launch_stream<F, 8, 1, 2, 1, 2, 8, 16, kDense>(P, stream, P.N);
      case 2: return launch_stream<F, 8, 1, 2, 1, 2 * UW, 4, 16, kDense>(P, stream, P.N);
      case 3: return launch_stream<F, 16, 1, 4, 1, 2, 4, 16, kDense>(P, stream, P.N);
      case 4: return launch_stream<F, 8, 1, 1, 1, 1, 6, 16, kDense>(P, stream, P.N);
      case 5: return launch_stream<F, 16, 1, 2, 1, 1, 6, 16, kDense>(P, stream, P.N);
      case 6: return launch_stream<F, 8, 1, 1, 1, 2 * UW, 4, 32, kDense>(P, stream, P.N);
      case 7: return launch_stream<F, 16, 1, 2, 1, UW, 4, 16, kDense>(P, stream, P.N);
      case 8: return launch_stream<F, 16, 1, 2, 1, UW, 5, 16, kDense>(P, stream, P.N);
      case 9: return launch_stream<F, 16, 1, 4, 1, 2 * UW, 3, 16, kDense>(P, stream, P.N);
      // the deepest rings shared memory allows, for activations of at most 16 KB (32 KB for NVFP4)
      case 10: return launch_stream<F, 8, 1, 2, 1, 2 * UW, (F == LX_W_NVFP4 ? 9 : 6), (F == LX_W_NVFP4 ? 16 : 8), kDense>(P, stream, P.N);
      case 11: return launch_stream<F, 16, 1, 2, 1, UW, (F == LX_W_NVFP4 ? 9 : 6), (F == LX_W_NVFP4 ? 16 : 8), kDense>(P, stream, P.N);
      case 12: return launch_stream<F, 8, 1, 2, 1, UW, (F == LX_W_NVFP4 ? 18 : 12), (F == LX_W_NVFP4 ? 16 : 8), kDense>(P, stream, P.N);
      case 13: return launch_stream<F, 16, 1, 4, 1, UW, (F == LX_W_NVFP4 ? 9 : 6), (F == LX_W_NVFP4 ? 16 : 8), kDense>(P, stream, P.N);
      default: return launch_stream<F, 8, 1, 2, 1, 2, 4, 16, kDense>(P, stream, P.N);
    }
  }
  if (cols <= 16) return launch_stream<F, 8, 1, 2, 2, 2, 4, 64, kDense>(P, stream, P.N);
  if (cols <= 24) return launch_stream<F, 8, 1, 2, 3, 2, 4, 64, kDense>(P, stream, P.N);
  if (cols <= 32) return launch_stream<F, 8, 2, 2, 4, UW, 3, 32, kDense>(P, stream, P.N);
  return launch_stream<F, 8, 2, 4, 8, UW, 2, 32, kDense>(P, stream, P.N);
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
  // Up to 8 rows of INT8 / FP8 weights with enough rows per SM: the tensor-core product (the choice never depends on M)
  if (M <= 8 && !force_scalar() && tc_rows_ok(w, N, K))
    return tc_product_rows(x, x_dtype, ld_x, w, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta, stream);
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
  // the reference's layout, or what the prepared activations of the tensor-core product take, whichever is larger
  return std::max(act_layout(M, K, math).total, tc_workspace_bytes(M, K));
}

extern "C" int lx_gemm_w(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, lx_math math, const void* bias,
                         lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                         float beta, void* workspace, void* stream) {
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
  // With a workspace every row count goes through the tcgen05 product, so that a row's bits do not depend on M
  // (up to 8 rows of INT8 / FP8 prepare their own activations there and give the same bits). LX_B200_TC=0 keeps the
  // mma.sync streaming kernel.
  if (tc_enabled() && workspace && aligned(workspace, 16) && !(M <= 8 && tc_rows_ok(*w, N, K)) &&
      (w->type != LX_W_NVFP4 || (K % 256 == 0 && aligned(w->scale, 16))))
    return tc_product(x, x_dtype, ld_x, *w, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta, workspace,
                      static_cast<cudaStream_t>(stream));
  return dense_product(x, x_dtype, ld_x, *w, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta,
                       static_cast<cudaStream_t>(stream));
}

// ---- additions: a row-sharded product whose epilogue is the all-gather ---------------------------------------------
// Every rank multiplies its rows of W and stores its slice of y straight into every rank's copy of the whole y through
// peer-mapped pointers (NVLink stores from the epilogue threads); the grid's last warp then adds one arrival to every
// rank's semaphore; a
// consumer waits (lx_b200_wait_arrivals, bounded) until its counter holds what all ranks add, and takes it. No collective
// kernel runs: the transfer overlaps the tiles. BF16 / INT8 / FP8 weights on the tcgen05 product; beta = 0.
extern "C" int lx_b200_linear_allgather(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, const void* bias,
                                        lx_dtype bias_dtype, void* const* y_all, int* const* arrivals, int ranks, int rank, int64_t col0,
                                        lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha, void* workspace,
                                        int* arrivals_added, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || ld_x < K || ld_y < N || !w || !w->data || !x || !y_all || !arrivals) return kInvalid;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype) || (bias && !valid_dtype(bias_dtype))) return kInvalid;
  if (ranks < 1 || ranks > 8 || rank < 0 || rank >= ranks || col0 < 0 || col0 + N > ld_y) return kInvalid;
  if (w->type != LX_W_BF16 && !w->scale) return kInvalid;
  const int64_t rowb = row_bytes_of(w->type, K);
  if (rowb % 16 != 0 || !aligned(w->data, 16)) return kNotSupported;
  const PeerTargets T{y_all, arrivals, ranks, rank, col0};
  return tc_product_allgather(x, x_dtype, ld_x, *w, bias, bias_dtype, T, y_dtype, ld_y, M, N, K, alpha, workspace, arrivals_added,
                              static_cast<cudaStream_t>(stream));
}

extern "C" int lx_b200_wait_arrivals(int* counter, int total, void* stream) {
  if (!counter || total <= 0) return kInvalid;
  return tc_wait_arrivals(counter, total, static_cast<cudaStream_t>(stream));
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

