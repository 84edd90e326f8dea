// Dense products of the kernel ABI: lx_gemv_w, lx_gemv, lx_gemv_decode_bf16, lx_gemv_bf16x (M <= 8) and lx_gemm_w,
// lx_gemm_skinny (any M), all on the weight-streaming kernel of stream.cuh, plus a scalar kernel for shapes and
// alignments the streaming kernel does not take (short or odd K, unaligned rows).
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "gemv.cuh"
#include "gemv_x16.cuh"
#include "gemv_ring8.cuh"
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
  if (P.M <= 8) {
    // Up to 8 activation rows. A format keeps ONE warp layout (consumer warps, warp rows, steps per stage: what fixes
    // the order a row's products are added in) whatever M and the activation dtype are; only the number of 8-column
    // tiles follows them. So a row's bits do not depend on its batch; BF16 and BF16X share their layout, so the
    // lossless format reproduces bf16's bits.
    const int64_t unit_bytes = static_cast<int64_t>(P.K) / (k8 ? 16 : 8) * 16 * cols;
    const bool big_x = unit_bytes > 32 * 1024;  // up to 32 KB of activation units stay resident in the small buffer
    if constexpr (F == LX_W_BF16 || F == LX_W_BF16X) {
      if (cols <= 8) return big_x ? launch_stream<F, 16, 1, 2, 1, 2, 2, 64, kDense>(P, stream, P.N) : launch_stream<F, 16, 1, 2, 1, 2, 5, 16, kDense>(P, stream, P.N);
      return cols <= 16 ? launch_stream<F, 16, 1, 2, 2, 2, 2, 64, kDense>(P, stream, P.N) : launch_stream<F, 16, 1, 2, 3, 2, 2, 64, kDense>(P, stream, P.N);
    } else if constexpr (F == LX_W_NVFP4) {
      if (cols <= 8) return big_x ? launch_stream<F, 16, 1, 4, 1, 2, 2, 64, kDense>(P, stream, P.N) : launch_stream<F, 16, 1, 4, 1, 2, 4, 16, kDense>(P, stream, P.N);
      // (48 KB halves: with 64 KB the two-tile layout no longer fits an SM's shared memory)
      return cols <= 16 ? launch_stream<F, 16, 1, 4, 2, 2, 2, 48, kDense>(P, stream, P.N) : launch_stream<F, 16, 1, 4, 3, 2, 2, 48, kDense>(P, stream, P.N);
    } else {
      if (cols <= 8) return big_x ? launch_stream<F, 8, 1, 2, 1, 2, 4, 64, kDense>(P, stream, P.N) : launch_stream<F, 8, 1, 2, 1, 2, 4, 16, kDense>(P, stream, P.N);
      return cols <= 16 ? launch_stream<F, 8, 1, 2, 2, 2, 4, 64, kDense>(P, stream, P.N) : launch_stream<F, 8, 1, 2, 3, 2, 4, 64, kDense>(P, stream, P.N);
    }
  }
  if (cols <= 16) return launch_stream<F, 8, 1, 2, 2, 2, 4, 64, kDense>(P, stream, P.N);
  if (cols <= 24) return launch_stream<F, 8, 1, 2, 3, 2, 4, 64, kDense>(P, stream, P.N);
  if (cols <= 32) return launch_stream<F, 8, 2, 2, 4, UW, 3, 32, kDense>(P, stream, P.N);
  return launch_stream<F, 8, 2, 4, 8, UW, 2, 32, kDense>(P, stream, P.N);
}

// ---- the decode GEMV (gemv.cuh): up to 8 rows, every format ----------------------------------------------------------
template <int F, int NT, int CPS>
int launch_gemv_inst(const GemvParams& P, size_t smem, cudaStream_t stream) {
  auto kernel = gemv_kernel<F, NT, CPS>;
  if (int e = allow_dynamic_smem<4096 + F * 64 + NT * 8 + CPS>(kernel)) return e;
  const int sms = sm_count();
  if (!sms) return kInvalid;
  const unsigned grid = static_cast<unsigned>(std::max(1, std::min((P.N + kGemvGranule - 1) / kGemvGranule, sms * CPS)));
  return launch_kernel(kernel, dim3(grid), dim3(kGemvThreads), smem, stream, P);
}

// The lossless format's own kernel (gemv_x16.cuh): one CTA per SM, records brought in by bulk copies. `taken` = false when
// the shape is not for it (no ring fits beside the activations, or the copy of the last record would read past the
// matrix: records that are not 16-byte aligned are copied from 8 bytes before to 8 bytes after).
template <int NT>
int launch_x16(const GemvParams& P, cudaStream_t stream, bool& taken) {
  taken = false;
  X16Ring R{};
  size_t smem = 0;
  const bool a16 = P.row_bytes % 16 == 0;
  if (!aligned(P.w, 16) || (!a16 && P.N % 2 != 0) || !x16_ring_for(P.K, P.ncols, R, smem)) return kOk;
  const int sms = sm_count();
  if (!sms) return kInvalid;
  R.status = status_word();
  taken = true;
  const unsigned grid = static_cast<unsigned>(std::max(1, std::min((P.N + kGemvGranule - 1) / kGemvGranule, sms)));
  if (a16) {
    auto kernel = gemv_x16_kernel<NT, true>;
    if (int e = allow_dynamic_smem<4800 + NT * 2 + 1>(kernel)) return e;
    return launch_kernel(kernel, dim3(grid), dim3(kX16Threads), smem, stream, P, R);
  }
  auto kernel = gemv_x16_kernel<NT, false>;
  if (int e = allow_dynamic_smem<4800 + NT * 2>(kernel)) return e;
  return launch_kernel(kernel, dim3(grid), dim3(kX16Threads), smem, stream, P, R);
}

// The 8-bit formats' kernel on bulk copies (gemv_ring8.cuh): one CTA per SM. `taken` = false when two units do not fit.
template <int F, int NT>
int launch_ring8(const GemvParams& P, int min_slots, cudaStream_t stream, bool& taken) {
  taken = false;
  Ring8 R{};
  size_t smem = 0;
  if (!aligned(P.w, 16) || P.K % 128 != 0 || (F == LX_W_NVFP4 && (P.K % 256 != 0 || !aligned(P.scale, 16))) || !ring8_for(P.K, F, P.ncols, R, smem) ||
      R.S < min_slots)
    return kOk;
  const int sms = sm_count();
  if (!sms) return kInvalid;
  R.status = status_word();
  taken = true;
  const unsigned grid = static_cast<unsigned>(std::max(1, std::min((P.N + kGemvGranule - 1) / kGemvGranule, sms)));
  auto kernel = gemv_ring8_kernel<F, NT>;
  if (int e = allow_dynamic_smem<4900 + F * 4 + NT>(kernel)) return e;
  return launch_kernel(kernel, dim3(grid), dim3(kX16Threads), smem, stream, P, R);
}

// variant: an index into kGemvVariantNames (see variants.h), -1 = two CTAs per SM when their shared memory allows
template <int F>
int launch_gemv(GemvParams P, int variant, cudaStream_t stream) {
  P.planes = terms_for(GemvFmt<F>::kMma, P.x_dtype == LX_BF16);
  P.ncols = P.M * P.planes;
  P.pitch = gemv_pitch(P.K, F);
  P.steps = P.K / GemvFmt<F>::kStepValues;
  const size_t smem = gemv_smem(P.K, F, P.ncols);
  const int NT = (P.ncols + 7) / 8;
  // BF16X: its own kernel by default (gemv_x16.cuh); the table can still name this one's two forms, of which d8c1 is the
  // fallback (two CTAs per SM leave the in-register decode too few registers: 55 us against 39 on a 14336 x 4096 matrix).
  if constexpr (F == LX_W_BF16X) {
    if ((variant == kGemvX16Pipe || variant < 0) && NT <= 2) {
      bool taken = false;
      const int e = NT == 1 ? launch_x16<1>(P, stream, taken) : launch_x16<2>(P, stream, taken);
      if (taken) return e;
    }
  }
  // INT8 / FP8 / NVFP4 on rows short enough for two units in shared memory: the kernel on bulk copies (gemv_ring8.cuh)
  // where it was measured ahead, up to four activation rows. The same sums either way, so the choice may look at M.
  //   8-bit, 14336 x 4096 at M = 1 / 2 / 4: FP8 14.1 / 14.6 / 17.3 against 14.4 / 15.2 / 17.8 us, INT8 at M = 1 14.4 against
  //   17.9; 16384 x 2048 FP8 9.9 against 10.6; at M = 8 it is behind, 24.5 against 22.8.
  //   NVFP4 (whose 16-byte loads of 8 rows ask for half a line each), 28672 x 8192 at M = 1 / 2 / 4: 31.5 / 33.8 / 40.1
  //   against 37.7 / 39.3 / 43.4 us; 14336 x 4096 at M = 1: 13.3 against 14.4.
  if constexpr (F == LX_W_INT8 || F == LX_W_FP8 || F == LX_W_NVFP4) {
    if ((variant == kGemvX16Pipe || (variant < 0 && P.M <= 4)) && NT <= 2) {
      bool taken = false;
      const int e = NT == 1 ? launch_ring8<F, 1>(P, 2, stream, taken) : launch_ring8<F, 2>(P, 2, stream, taken);
      if (taken) return e;
    }
  }
  const bool two = variant == kGemvD4C2 || (variant < 0 && F != LX_W_BF16X);
  const int cps = (smem <= 110 * 1024 && two) ? 2 : 1;
  switch (NT * 10 + cps) {
    case 11: return launch_gemv_inst<F, 1, 1>(P, smem, stream);
    case 12: return launch_gemv_inst<F, 1, 2>(P, smem, stream);
    case 21: return launch_gemv_inst<F, 2, 1>(P, smem, stream);
    case 22: return launch_gemv_inst<F, 2, 2>(P, smem, stream);
    case 31: return launch_gemv_inst<F, 3, 1>(P, smem, stream);
    case 32: return launch_gemv_inst<F, 3, 2>(P, smem, stream);
  }
  return kInvalid;
}

int row_bytes_of(int type, int K) {
  switch (type) {
    case LX_W_BF16: return 2 * K;
    case LX_W_NVFP4: return K / 2;
    case LX_W_BF16X: return static_cast<int>(x16::row_bytes(K));
    default: return K;
  }
}

int gemv_env_variant() {
  static const int v = [] {
    return gemv_variant_by_name(std::getenv("LX_B200_GEMV_VARIANT"));
  }();
  return v;
}

bool gemv_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LX_B200_GEMV");
    return !(v && v[0] == '0');
  }();
  return on;
}

// Can the decode GEMV take this weight? Whole 64-byte steps per row, the data aligned for the widest load the format
// uses, and the activation columns of EIGHT rows within shared memory (so that the answer is the same for every M).
bool gemv_ok(const lx_weight& w, int K, bool x_bf16) {
  if (!gemv_shape_ok(w.type, K, x_bf16)) return false;
  switch (w.type) {
    case LX_W_BF16X: return aligned(w.data, 8);
    case LX_W_NVFP4: return aligned(w.data, 16) && aligned(w.scale, 2);
    default: return aligned(w.data, 16);
  }
}

// The product itself, arguments already validated.
int dense_product(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype, void* y,
                  int y_dtype, int ld_y, int M, int N, int K, float alpha, float beta, cudaStream_t stream) {
  // Up to 8 rows: the decode GEMV of gemv.cuh whenever the weight's shape and alignment allow, except INT8 weights wide
  // enough for the tcgen05 product, which is the faster one there (measured on 14336 x 4096: 15.4 / 17.1 us at M = 1 / 8
  // against 16.5 / 23.2). The choice never depends on M. The variant table can name another residency of the GEMV (same
  // bits), or, through lx_tune_force only, another implementation: the TMA-ring mma.sync kernel of stream.cuh ("s8ring"),
  // the tcgen05 product ("s1tc", INT8 / FP8 weights with enough rows per SM). LX_B200_GEMV=0 restores the ring / tc pair.
  if (M <= 8 && !force_scalar()) {
    int tuned = lx_tune_get(gemv_kernel_name(w.type), M, N, K);
    if (w.type == LX_W_BF16X) tuned = x16_variant(tuned);  // its list has its own third entry
    if (tuned < 0) tuned = gemv_env_variant();  // LX_B200_GEMV_VARIANT=<name>: the variant of shapes the table does not hold
    const bool gemv_named = tuned == kGemvD4C2 || tuned == kGemvD8C1 || tuned == kGemvX16Pipe;
    const bool want_tc = tuned == kGemvTc || (tuned < 0 && (!gemv_enabled() || w.type == LX_W_INT8));
    const bool want_ring = tuned == kGemvRing || (tuned < 0 && !gemv_enabled());
    if (want_tc && tc_rows_ok(w, N, K))
      return tc_product_rows(x, x_dtype, ld_x, w, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta, stream);
    if (!want_ring && (!want_tc || gemv_named || !tc_rows_ok(w, N, K)) && gemv_ok(w, K, x_dtype == LX_BF16)) {
      GemvParams G{};
      G.w = static_cast<const uint8_t*>(w.data);
      G.scale = static_cast<const uint8_t*>(w.scale);
      G.global = w.global;
      G.row_bytes = row_bytes_of(w.type, K);
      G.N = N, G.K = K;
      G.x = x, G.x_dtype = x_dtype, G.ld_x = ld_x, G.M = M;
      G.bias = bias, G.bias_dtype = bias_dtype;
      G.y = y, G.y_dtype = y_dtype, G.ld_y = ld_y;
      G.alpha = alpha, G.beta = beta;
      switch (w.type) {
        case LX_W_BF16: return launch_gemv<LX_W_BF16>(G, tuned, stream);
        case LX_W_INT8: return launch_gemv<LX_W_INT8>(G, tuned, stream);
        case LX_W_FP8: return launch_gemv<LX_W_FP8>(G, tuned, stream);
        case LX_W_NVFP4: return launch_gemv<LX_W_NVFP4>(G, tuned, stream);
        case LX_W_BF16X: return launch_gemv<LX_W_BF16X>(G, tuned, stream);
      }
    }
  }
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
// The part of the decode GEMV's admission that depends on the format, K and the activation dtype only.
bool gemv_shape_ok(int wtype, int K, bool x_bf16) {
  if (wtype < LX_W_BF16 || wtype > LX_W_BF16X) return false;
  if (K <= 0 || K % gemv_step_values(wtype) != 0) return false;
  if (wtype == LX_W_BF16X && K >= (1 << 23)) return false;
  return gemv_smem(K, wtype, 8 * terms_for(gemv_mma_of(wtype), x_bf16)) <= kGemvSmemMax;
}

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
  if (int e = math_admitted(math, w->type)) return e;
  const bool quantized = math != LX_MATH_BF16;
  if (w->type != LX_W_BF16 && !w->scale) return kInvalid;
  // Weight rows must be whole 16-byte chunks, as for the reference's tensor-core kernels.
  const int64_t rowb = row_bytes_of(w->type, K);
  if (rowb % 16 != 0 || !aligned(w->data, 16) || (w->type == LX_W_NVFP4 && K % 64 != 0)) return kNotSupported;
  // With a workspace every row count goes through the tcgen05 product, so that within this entry point a row's bits
  // do not depend on M. LX_B200_TC=0 keeps the mma.sync kernels.
  // f32 activations are rounded to bf16 (BF16 math) or quantized (the other maths) into the workspace, as in the
  // reference (engine/cuda/gemm_w.cu:213-252), which answers "invalid" when there is none.
  if (x_dtype == LX_F32 && !workspace) return kInvalid;
  if (quantized) {  // activations quantized per token into the workspace, then s8 x s8 -> s32 or e4m3 x e4m3 -> f32 on the tensor cores
    if (!workspace) return kInvalid;
    if (!tc_enabled() || !aligned(workspace, 16)) return kNotSupported;
    return tc_product(x, x_dtype, ld_x, *w, bias, bias_dtype, y, y_dtype, ld_y, M, N, K, alpha, beta, workspace,
                      static_cast<cudaStream_t>(stream), true);
  }
  if (tc_enabled() && workspace && aligned(workspace, 16) && (w->type != LX_W_NVFP4 || (K % 256 == 0 && aligned(w->scale, 16))))
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

// The shared-memory plan of the decode GEMV kernels that bring their weights in with bulk copies (gemv_x16.cuh,
// gemv_ring8.cuh) for a weight format, K and M, without launching anything: the same geometry functions the launches use.
// Fills out[0..11] (see the header); out[0], the ring's slots, stays 0 when the format has no such kernel or no ring fits.
extern "C" int lx_b200_gemv_ring_plan(int wtype, int K, int M, int x_is_bf16, int32_t* out) {
  if (!out || K <= 0 || M < 1 || M > 8) return kInvalid;
  for (int i = 0; i < 12; ++i) out[i] = 0;
  if (wtype != LX_W_BF16X && wtype != LX_W_INT8 && wtype != LX_W_FP8 && wtype != LX_W_NVFP4) return kOk;
  if (!gemv_shape_ok(wtype, K, x_is_bf16 != 0)) return kOk;
  const int planes = terms_for(gemv_mma_of(wtype), x_is_bf16 != 0), ncols = M * planes;
  if ((ncols + 7) / 8 > 2) return kOk;
  size_t smem = 0;
  if (wtype == LX_W_BF16X) {
    X16Ring r{};
    if (!x16_ring_for(K, ncols, r, smem)) return kOk;
    const int32_t v[12] = {r.S, r.whole, r.cb, r.spu, static_cast<int32_t>(r.stride), static_cast<int32_t>(r.slot_bytes),
                           static_cast<int32_t>(r.hstride), static_cast<int32_t>(r.hslot_bytes), static_cast<int32_t>(r.hdr_off),
                           static_cast<int32_t>(r.ring_off), static_cast<int32_t>(r.bar_off), static_cast<int32_t>(smem)};
    for (int i = 0; i < 12; ++i) out[i] = v[i];
    return kOk;
  }
  if (K % 128 != 0 || (wtype == LX_W_NVFP4 && K % 256 != 0)) return kOk;
  Ring8 r{};
  if (!ring8_for(K, wtype, ncols, r, smem)) return kOk;
  const int32_t v[12] = {r.S, 1, 0, 1, row_bytes_of(wtype, K), static_cast<int32_t>(r.slot_bytes), static_cast<int32_t>(r.scale_off), 0,
                         static_cast<int32_t>(r.ring_off), static_cast<int32_t>(r.ring_off), static_cast<int32_t>(r.bar_off), static_cast<int32_t>(smem)};
  for (int i = 0; i < 12; ++i) out[i] = v[i];
  return kOk;
}

extern "C" int lx_b200_wait_arrivals(int* counter, int total, void* stream) {
  if (!counter || total <= 0) return kInvalid;
  return tc_wait_arrivals(counter, total, static_cast<cudaStream_t>(stream));
}

// The skinny decode GEMM's contract is that a row's bits depend on that row, the weight and the epilogue alone: not on
// M, not on the row's place in the call (kernels.h:457-475). The decode GEMV gives exactly that for up to 8 rows, so
// the call runs as chunks of 8 rows on it: every row of every M goes through the same kernel with the same K slices.
// (Beyond 8 rows the chunks re-read the weight, from L2 where it fits; the engine itself never calls this entry point.)
extern "C" int lx_gemm_skinny(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, const void* bias,
                              lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                              float beta, void* stream) {
  if (M < 0 || N < 0 || K <= 0 || ld_x < K || ld_y < N || !w) return kInvalid;
  if (M == 0 || N == 0) return kOk;
  if (!x || !y || !w->data) return kInvalid;
  if (!valid_dtype(y_dtype) || (bias && !valid_dtype(bias_dtype))) return kInvalid;
  if (w->type != LX_W_BF16 || x_dtype != LX_BF16 || N % 16 != 0 || K % 64 != 0) return kNotSupported;
  if (!gemv_ok(*w, K, true)) return kNotSupported;
  GemvParams G{};
  G.w = static_cast<const uint8_t*>(w->data);
  G.row_bytes = 2ll * K;
  G.global = 1.0f;
  G.N = N, G.K = K;
  G.x_dtype = x_dtype, G.ld_x = ld_x;
  G.bias = bias, G.bias_dtype = bias_dtype;
  G.y_dtype = y_dtype, G.ld_y = ld_y;
  G.alpha = alpha, G.beta = beta;
  for (int m0 = 0; m0 < M; m0 += 8) {
    G.M = std::min(8, M - m0);
    G.x = static_cast<const uint8_t*>(x) + static_cast<int64_t>(m0) * ld_x * 2;
    G.y = static_cast<uint8_t*>(y) + static_cast<int64_t>(m0) * ld_y * (y_dtype == LX_BF16 ? 2 : 4);
    if (int e = launch_gemv<LX_W_BF16>(G, -1, static_cast<cudaStream_t>(stream))) return e;
  }
  return kOk;
}
