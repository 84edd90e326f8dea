// Routed experts for a few tokens (lx_moe_experts_decode, lx_moe_experts_bf16x, lx_moe_experts_decode_bf16) and the
// bf16 entry point of any length that shares their kernels (lx_moe_experts).
//
// Contract (kernels.h:217-225, 495-511, 596-611 of the reference): out[t] = sum_k weights[t, k] * down[e] @
// bf16(silu(gate_up[e][:I] @ x) * (gate_up[e][I:] @ x)), e = ids[t, k]; weight-only f32 sums; a token's bits do not
// depend on its batch; BF16X stacks give the bits of the bf16 stacks they encode.
//
// With a handful of tokens the call is nothing but the chosen experts' bytes crossing HBM once, so both stages are
// plain streaming kernels: one warp per weight row, whole 16-byte words per lane, several words in flight per lane,
// no shared memory, no atomics, every output written once.
//   1. gate/up: a block belongs to one (pair, 16 intermediate rows). The first pair that names an expert leads it:
//      its blocks serve every pair of that expert (one pass over the expert's rows however many tokens picked it);
//      the blocks of the other pairs leave at once. A warp reads gate row i and up row I + i together and writes
//      bf16(silu(gate) * up) to each member pair's row of the workspace.
//   2. down: a block belongs to one (token, 8 output rows); a warp sums the token's top_k experts in k order in
//      registers and writes out[t, l].
// Each (pair, row) sum is one lane-ordered chain of fmaf over k followed by a fixed shuffle tree, whatever else the
// block serves, which is what makes the rows batch-invariant and BF16X equal to bf16 bit for bit (both walk 8 values
// per lane per step).
#include <cuda_runtime.h>

#include "launch.cuh"

namespace b200 {
namespace {

constexpr int kDecodeMaxT = 8;      // moe_decode.cu:40-41 of the reference: the decode contract
constexpr int kDecodeMaxTopK = 8;
constexpr int kRowsPerBlock = 8;    // one warp per row
constexpr int kGateUpRows = 16;     // intermediate rows a gate/up block walks (two per warp)
constexpr int kDecodeThreads = 32 * kRowsPerBlock;
constexpr int kScanPairs = kDecodeMaxT * kDecodeMaxTopK;  // pairs a block scans for its expert's members

// One stack of expert matrices as the kernels read it.
struct Stack {
  const uint8_t* data;
  const uint8_t* scale;        // f32 per row (INT8 / FP8), e4m3 per 16 values (NVFP4)
  const float* expert_global;  // NVFP4: per-expert global or null
  float global;
  int64_t row_bytes;           // bytes from one row to the next (BF16X: one record)
  int rows;                    // rows per expert
  int K;                       // values per row
  int vec;                     // rows (and NVFP4 scales) start on 16-byte boundaries: whole-word loads
};

// Values a lane takes per step: one 16-byte word; NVFP4 one block of 16 values (8 bytes and its scale); BF16X the 8
// values one bf16 word would hold, so that both formats sum in the same order.
template <int F>
constexpr int kLaneValues = F == LX_W_BF16 || F == LX_W_BF16X ? 8 : 16;

// A lane's bytes of one row and step, as loaded.
struct Raw {
  uint4 w;     // BF16X: x, y = sign|mantissa bytes, z = 4-bit codes, w = the block's base exponent
  uint32_t s;  // NVFP4: the block's scale byte; BF16X: 1 when the row has patches
};

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(static_cast<const uint4*>(p)); }

// The word of row `row` (a pointer to its first byte) at value k0, zero past K.
template <int F>
__device__ __forceinline__ Raw load_raw(const Stack& S, const uint8_t* row, const uint8_t* row_scale, int k0) {
  Raw r{make_uint4(0, 0, 0, 0), 0};
  const int K = S.K;
  if (k0 >= K) return r;
  constexpr int V = kLaneValues<F>;
  if constexpr (F == LX_W_BF16X) {
    const int H = x16::header_bytes(K), slots = x16::patch_slots(K);
    const int blk = k0 >> 7, off = k0 & 127;
    const uint8_t* b = row + H + blk * 192;
    const uint2 sm = __ldg(reinterpret_cast<const uint2*>(b + off));
    r.w.x = sm.x, r.w.y = sm.y;
    r.w.z = __ldg(reinterpret_cast<const uint32_t*>(b + 128 + (off >> 1)));
    r.w.w = __ldg(row + 4 * slots + blk);
    return r;
  } else {
    constexpr int kBytes = F == LX_W_NVFP4 ? 8 : 16;
    const int64_t at = F == LX_W_BF16 ? 2ll * k0 : F == LX_W_NVFP4 ? k0 / 2 : k0;
    if constexpr (F == LX_W_NVFP4) r.s = __ldg(row_scale + k0 / 16);
    if (S.vec && k0 + V <= K) {
      if constexpr (F == LX_W_NVFP4) {
        const uint2 u = __ldg(reinterpret_cast<const uint2*>(row + at));
        r.w.x = u.x, r.w.y = u.y;
      } else {
        r.w = ldg16(row + at);
      }
    } else {
      // byte by byte: short or unaligned rows, and the last partial word of a row
      const int64_t row_len = F == LX_W_BF16 ? 2ll * K : F == LX_W_NVFP4 ? K / 2 : K;
      uint32_t w[4] = {0, 0, 0, 0};
      for (int j = 0; j < kBytes; ++j)
        if (at + j < row_len) w[j >> 2] |= static_cast<uint32_t>(__ldg(row + at + j)) << (8 * (j & 3));
      r.w = make_uint4(w[0], w[1], w[2], w[3]);
    }
    return r;
  }
}

// V activations from value k0 of a bf16 row as f32, zero past K.
template <int V>
__device__ __forceinline__ void load_x(const uint16_t* x, int k0, int K, bool vec, float (&xf)[V]) {
  if (vec && k0 + V <= K) {
#pragma unroll
    for (int q = 0; q < V / 8; ++q) {
      const uint4 u = *reinterpret_cast<const uint4*>(x + k0 + 8 * q);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xf[8 * q + 2 * j] = __uint_as_float(w[j] << 16);
        xf[8 * q + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) xf[j] = k0 + j < K ? bf16_bits_to_f32(x[k0 + j]) : 0.0f;
  }
}

// The exponent a patch list gives value k of a BF16X row, or `e` when the list does not name it.
__device__ __noinline__ uint32_t patched_exponent(const uint8_t* row, int K, int k, uint32_t e) {
  const uint32_t* list = reinterpret_cast<const uint32_t*>(row);
  int n_list = x16::patch_slots(K);
  const uint32_t s0 = list[0];
  if (s0 & 0x80000000u) {  // the row's patches live in an overflow record behind the rows
    const uint32_t* rec = reinterpret_cast<const uint32_t*>(row + static_cast<int64_t>(s0 & 0x7fffffffu) * 8);
    n_list = static_cast<int>(rec[0]);
    list = rec + 1;
  }
  for (int i = 0; i < n_list; ++i) {
    const uint32_t p = list[i];
    if (p == x16::kNoPatch || (p >> 8) > static_cast<uint32_t>(k)) break;
    if ((p >> 8) == static_cast<uint32_t>(k)) e = p & 0xffu;
  }
  return e;
}

// acc += sum_j x[j] * value_j of the word, j ascending (NVFP4: the block's sum times its scale).
template <int F>
__device__ __forceinline__ float dot_word(const Raw& r, const float (&xf)[kLaneValues<F>], float acc, const uint8_t* row, int k0,
                                          int K) {
  constexpr int V = kLaneValues<F>;
  const uint32_t w[4] = {r.w.x, r.w.y, r.w.z, r.w.w};
  if constexpr (F == LX_W_BF16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc = fmaf(xf[2 * j], __uint_as_float(w[j] << 16), acc);
      acc = fmaf(xf[2 * j + 1], __uint_as_float(w[j] & 0xffff0000u), acc);
    }
  } else if constexpr (F == LX_W_BF16X) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t sm = (w[j >> 2] >> (8 * (j & 3))) & 0xffu;
      const uint32_t code = (w[2] >> (8 * (j & 3) + 4 * (j >> 2))) & 15u;
      uint32_t e = (w[3] - code) & 0xffu;
      if (r.s) e = patched_exponent(row, K, k0 + j, e);
      float v = __uint_as_float(((sm & 0x80u) << 24) | (e << 23) | ((sm & 0x7fu) << 16));
      if (k0 + j >= K) v = 0.0f;  // padding of the last block decodes to 2^(base - 127), not to zero
      acc = fmaf(xf[j], v, acc);
    }
  } else if constexpr (F == LX_W_INT8) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t b = w[j] ^ 0x80808080u;  // byte + 128 in the mantissa of 2^23, then minus (2^23 + 128): exact
#pragma unroll
      for (int i = 0; i < 4; ++i)
        acc = fmaf(xf[4 * j + i], __uint_as_float(0x4b000000u | ((b >> (8 * i)) & 0xffu)) - 8388736.0f, acc);
    }
  } else if constexpr (F == LX_W_FP8) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t lo, hi;
      asm("{ .reg .b16 a, b; mov.b32 {a, b}, %2; cvt.rn.f16x2.e4m3x2 %0, a; cvt.rn.f16x2.e4m3x2 %1, b; }" : "=r"(lo), "=r"(hi) : "r"(w[j]));
      const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&lo)), f1 = __half22float2(*reinterpret_cast<const __half2*>(&hi));
      acc = fmaf(xf[4 * j], f0.x, acc);
      acc = fmaf(xf[4 * j + 1], f0.y, acc);
      acc = fmaf(xf[4 * j + 2], f1.x, acc);
      acc = fmaf(xf[4 * j + 3], f1.y, acc);
    }
  } else {
    float part = 0.0f;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t v[4];
      asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %4;\n"
          "cvt.rn.f16x2.e2m1x2 %0, b0; cvt.rn.f16x2.e2m1x2 %1, b1; cvt.rn.f16x2.e2m1x2 %2, b2; cvt.rn.f16x2.e2m1x2 %3, b3; }"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
          : "r"(w[q]));
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v[i]));
        part = fmaf(xf[8 * q + 2 * i], f.x, part);
        part = fmaf(xf[8 * q + 2 * i + 1], f.y, part);
      }
    }
    acc = fmaf(e4m3_to_f32(r.s & 0xffu), part, acc);
  }
  (void)V;
  return acc;
}

// The factor of row n (counted over the whole stack) of expert e.
template <int F>
__device__ __forceinline__ float stack_row_factor(const Stack& S, int64_t n, int e) {
  if constexpr (F == LX_W_INT8 || F == LX_W_FP8) return __ldg(reinterpret_cast<const float*>(S.scale) + n);
  else if constexpr (F == LX_W_NVFP4) return S.expert_global ? __ldg(S.expert_global + e) : S.global;
  else return 1.0f;
}

template <int F>
__device__ __forceinline__ const uint8_t* scale_row(const Stack& S, int64_t n) {
  return F == LX_W_NVFP4 ? S.scale + n * (S.K / 16) : nullptr;
}
// BF16X: whether the row has patches (Raw::s of its words)
template <int F>
__device__ __forceinline__ uint32_t row_flag(const uint8_t* row) {
  if constexpr (F == LX_W_BF16X) return __ldg(reinterpret_cast<const uint32_t*>(row)) != x16::kNoPatch;
  else return 0;
}

// acc[r][t] += rows[r] . x[t] over all of K: the warp's lanes take consecutive words, kSteps words of each row in
// flight per lane. A token's sum is the same chain of operations whatever NT is.
template <int F, int NR, int NT>
__device__ __forceinline__ void dot_rows(const Stack& S, const uint8_t* const (&row)[NR], const uint8_t* const (&row_scale)[NR],
                                         const uint32_t (&flag)[NR], const uint16_t* const (&x)[NT], bool xvec, int lane,
                                         float (&acc)[NR][NT]) {
  constexpr int V = kLaneValues<F>;
  constexpr int kSteps = NT == 1 ? 4 : 2;
  const int K = S.K;
  for (int k_base = 0; k_base < K; k_base += 32 * V * kSteps) {
    Raw raw[kSteps][NR];
#pragma unroll
    for (int j = 0; j < kSteps; ++j)
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        raw[j][r] = load_raw<F>(S, row[r], row_scale[r], k_base + (32 * j + lane) * V);
        if constexpr (F == LX_W_BF16X) raw[j][r].s = flag[r];
      }
#pragma unroll
    for (int j = 0; j < kSteps; ++j) {
      const int k0 = k_base + (32 * j + lane) * V;
      if (k0 >= K) continue;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        float xf[V];
        load_x<V>(x[t], k0, K, xvec, xf);
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r][t] = dot_word<F>(raw[j][r], xf, acc[r][t], row[r], k0, K);
      }
    }
  }
}

// Stage 1 for the NT member pairs of one expert: mid[pair, i] = bf16(silu(s_g * gate_i . x) * (s_u * up_i . x)).
template <int F, int NT>
__device__ __forceinline__ void gate_up_members(const Stack& S, int e, int i, int I, const uint16_t* latent, int ld, bool xvec,
                                                const int (&member)[NT], int count, int top_k, uint16_t* mid, int lane) {
  const int64_t ng = static_cast<int64_t>(e) * S.rows + i, nu = ng + I;
  const uint8_t* const row[2] = {S.data + ng * S.row_bytes, S.data + nu * S.row_bytes};
  const uint8_t* const row_scale[2] = {scale_row<F>(S, ng), scale_row<F>(S, nu)};
  const uint32_t flag[2] = {row_flag<F>(row[0]), row_flag<F>(row[1])};
  const uint16_t* x[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) x[t] = latent + static_cast<int64_t>(member[t < count ? t : 0] / top_k) * ld;
  float acc[2][NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) acc[0][t] = acc[1][t] = 0.0f;
  dot_rows<F, 2, NT>(S, row, row_scale, flag, x, xvec, lane, acc);
  const float fg = stack_row_factor<F>(S, ng, e), fu = stack_row_factor<F>(S, nu, e);
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const float g = fg * warp_sum(acc[0][t]), u = fu * warp_sum(acc[1][t]);
    if (lane == 0 && t < count)
      mid[static_cast<int64_t>(member[t]) * I + i] = static_cast<uint16_t>(f32_to_bf16_bits(g / (1.0f + expf(-g)) * u));
  }
}

// grid (ceil(I / kGateUpRows), P). dedupe: P <= 64 and the first pair of an expert serves all of its pairs, two at a
// time (more members than two read the rows again, from L1 / L2: the registers of wider passes would halve the warps
// an SM holds for the common case of one or two).
template <int F>
__global__ void __launch_bounds__(kDecodeThreads) decode_gate_up_kernel(const Stack S, const uint16_t* __restrict__ latent, int ld,
                                                                        int xvec, const int32_t* __restrict__ ids,
                                                                        uint16_t* __restrict__ mid, int P, int top_k, int I,
                                                                        int dedupe) {
  pdl_trigger();
  pdl_wait();  // the latent rows and the routing come from earlier kernels
  const int p = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = ids[p];
  unsigned long long members = 1ull;
  if (dedupe) {
    const unsigned lo = __ballot_sync(0xffffffffu, lane < P && ids[lane] == e);
    const unsigned hi = __ballot_sync(0xffffffffu, lane + 32 < P && ids[lane + 32] == e);
    members = (static_cast<unsigned long long>(hi) << 32) | lo;
    if ((members & (0 - members)) != (1ull << p)) return;  // an earlier pair leads this expert
  }
  const int i_end = min(I, (static_cast<int>(blockIdx.x) + 1) * kGateUpRows);
  for (int i = blockIdx.x * kGateUpRows + warp; i < i_end; i += kRowsPerBlock) {
    unsigned long long left = members;
    while (left) {
      int member[2];
      member[0] = dedupe ? __ffsll(static_cast<long long>(left)) - 1 : p;
      left &= left - 1;
      if (left) {
        member[1] = __ffsll(static_cast<long long>(left)) - 1;
        left &= left - 1;
        gate_up_members<F, 2>(S, e, i, I, latent, ld, xvec != 0, member, 2, top_k, mid, lane);
      } else {
        const int m1[1] = {member[0]};
        gate_up_members<F, 1>(S, e, i, I, latent, ld, xvec != 0, m1, 1, top_k, mid, lane);
      }
    }
  }
}

// Stage 2: out[t, l] = sum over k, in order, of weights[t, k] * (s_l * down[e_k]_l . mid[t, k]). grid (ceil(L / 8), T).
template <int F>
__global__ void __launch_bounds__(kDecodeThreads) decode_down_kernel(const Stack S, const uint16_t* __restrict__ mid, int xvec,
                                                                     const int32_t* __restrict__ ids,
                                                                     const float* __restrict__ weights, float* __restrict__ out,
                                                                     int top_k, int L) {
  pdl_trigger();
  pdl_wait();  // the intermediates come from the gate/up kernel
  const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int l = blockIdx.x * kRowsPerBlock + warp;
  if (l >= L) return;
  float total = 0.0f;
#pragma unroll 1
  for (int k = 0; k < top_k; ++k) {
    const int p = t * top_k + k, e = ids[p];
    const int64_t n = static_cast<int64_t>(e) * S.rows + l;
    const uint8_t* const row[1] = {S.data + n * S.row_bytes};
    const uint8_t* const row_scale[1] = {scale_row<F>(S, n)};
    const uint32_t flag[1] = {row_flag<F>(row[0])};
    const uint16_t* const x[1] = {mid + static_cast<int64_t>(p) * S.K};
    float acc[1][1] = {{0.0f}};
    dot_rows<F, 1, 1>(S, row, row_scale, flag, x, xvec != 0, lane, acc);
    const float term = __fmul_rn(weights[p], __fmul_rn(stack_row_factor<F>(S, n, e), warp_sum(acc[0][0])));
    total = __fadd_rn(total, term);
  }
  if (lane == 0) out[static_cast<int64_t>(t) * L + l] = total;
}

// ---- host ------------------------------------------------------------------------------------------------------------
Stack make_stack(int type, const void* data, const void* scale, const float* expert_global, float global, int rows, int K) {
  Stack S{};
  S.data = static_cast<const uint8_t*>(data);
  S.scale = static_cast<const uint8_t*>(scale);
  S.expert_global = type == LX_W_NVFP4 ? expert_global : nullptr;
  S.global = global;
  S.rows = rows, S.K = K;
  switch (type) {
    case LX_W_BF16: S.row_bytes = 2ll * K; break;
    case LX_W_NVFP4: S.row_bytes = K / 2; break;
    case LX_W_BF16X: S.row_bytes = x16::row_bytes(K); break;
    default: S.row_bytes = K; break;
  }
  const int word = type == LX_W_NVFP4 ? 8 : 16;
  S.vec = aligned(data, word) && S.row_bytes % word == 0;
  return S;
}

template <int F>
int launch_gate_up(const Stack& S, const void* latent, const int32_t* ids, uint16_t* mid, int P, int L, int I, int top_k,
                   cudaStream_t s) {
  const int xvec = aligned(latent, 16) && L % 8 == 0;
  const dim3 grid(static_cast<unsigned>((I + kGateUpRows - 1) / kGateUpRows), static_cast<unsigned>(P));
  return launch_kernel(decode_gate_up_kernel<F>, grid, dim3(kDecodeThreads), 0, s, S, static_cast<const uint16_t*>(latent), L, xvec,
                       ids, mid, P, top_k, I, P <= kScanPairs ? 1 : 0);
}
template <int F>
int launch_down(const Stack& S, const uint16_t* mid, const int32_t* ids, const float* weights, float* out, int T, int L, int I,
                int top_k, cudaStream_t s) {
  const int xvec = aligned(mid, 16) && I % 8 == 0;
  const dim3 grid(static_cast<unsigned>((L + kRowsPerBlock - 1) / kRowsPerBlock), static_cast<unsigned>(T));
  return launch_kernel(decode_down_kernel<F>, grid, dim3(kDecodeThreads), 0, s, S, mid, xvec, ids, weights, out, top_k, L);
}

// Both stages on stacks already checked. The grid's second extent holds pairs (tokens): up to 65535 of them per launch.
int decode_experts(const void* latent, const int32_t* ids, const float* weights, int gu_type, const Stack& gu, int dn_type,
                   const Stack& dn, float* out, void* workspace, int T, int L, int I, int top_k, cudaStream_t s) {
  const int P = T * top_k;
  if (P > 65535) return kNotSupported;
  auto* mid = static_cast<uint16_t*>(workspace);
  int e = kInvalid;
  switch (gu_type) {
    case LX_W_BF16: e = launch_gate_up<LX_W_BF16>(gu, latent, ids, mid, P, L, I, top_k, s); break;
    case LX_W_INT8: e = launch_gate_up<LX_W_INT8>(gu, latent, ids, mid, P, L, I, top_k, s); break;
    case LX_W_FP8: e = launch_gate_up<LX_W_FP8>(gu, latent, ids, mid, P, L, I, top_k, s); break;
    case LX_W_NVFP4: e = launch_gate_up<LX_W_NVFP4>(gu, latent, ids, mid, P, L, I, top_k, s); break;
    case LX_W_BF16X: e = launch_gate_up<LX_W_BF16X>(gu, latent, ids, mid, P, L, I, top_k, s); break;
  }
  if (e) return e;
  switch (dn_type) {
    case LX_W_BF16: return launch_down<LX_W_BF16>(dn, mid, ids, weights, out, T, L, I, top_k, s);
    case LX_W_INT8: return launch_down<LX_W_INT8>(dn, mid, ids, weights, out, T, L, I, top_k, s);
    case LX_W_FP8: return launch_down<LX_W_FP8>(dn, mid, ids, weights, out, T, L, I, top_k, s);
    case LX_W_NVFP4: return launch_down<LX_W_NVFP4>(dn, mid, ids, weights, out, T, L, I, top_k, s);
    case LX_W_BF16X: return launch_down<LX_W_BF16X>(dn, mid, ids, weights, out, T, L, I, top_k, s);
  }
  return kInvalid;
}

// Whole 8-byte words per row, the reference's condition (moe_decode.cu:385-394).
bool whole_words(int type, int K) {
  switch (type) {
    case LX_W_BF16: return K % 4 == 0;
    case LX_W_INT8:
    case LX_W_FP8: return K % 8 == 0;
    case LX_W_NVFP4: return K % 16 == 0;
    default: return false;
  }
}

// The checks of the bf16 / BF16X entry points (bf16x.cu:1336-1345 of the reference).
int check_plain(const void* latent, const int32_t* ids, const float* weights, const void* gate_up, const void* down, float* out,
                void* workspace, int L, int I, int top_k) {
  if (L <= 0 || I <= 0 || top_k < 1 || top_k > kDecodeMaxTopK || !latent || !ids || !weights || !gate_up || !down || !out ||
      !workspace || !aligned(workspace, 16) || !aligned(latent, 16) || !aligned(gate_up, 16) || !aligned(down, 16) ||
      L >= (1 << 23) || I >= (1 << 23))
    return kInvalid;
  return kOk;
}

int plain_experts(int type, const void* latent, const int32_t* ids, const float* weights, const void* gate_up, const void* down,
                  float* out, void* workspace, int T, int L, int I, int top_k, cudaStream_t s) {
  const Stack gu = make_stack(type, gate_up, nullptr, nullptr, 1.0f, 2 * I, L);
  const Stack dn = make_stack(type, down, nullptr, nullptr, 1.0f, L, I);
  return decode_experts(latent, ids, weights, type, gu, type, dn, out, workspace, T, L, I, top_k, s);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int64_t lx_moe_bf16x_workspace_bytes(int T, int I, int top_k) {
  if (T <= 0 || I <= 0 || top_k <= 0) return 0;
  return (2 * static_cast<int64_t>(T) * top_k * I + 255) / 256 * 256;
}

extern "C" int64_t lx_moe_decode_workspace_bytes(int T, int I, int top_k) { return lx_moe_bf16x_workspace_bytes(T, I, top_k); }

extern "C" int lx_moe_experts_bf16x(const void* latent, const int32_t* ids, const float* weights, const void* gate_up,
                                    const void* down, float* out, void* workspace, int T, int L, int I, int top_k, void* stream) {
  if (T <= 0) return kOk;
  if (int bad = check_plain(latent, ids, weights, gate_up, down, out, workspace, L, I, top_k)) return bad;
  return plain_experts(LX_W_BF16X, latent, ids, weights, gate_up, down, out, workspace, T, L, I, top_k,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int lx_moe_experts_decode_bf16(const void* latent, const int32_t* ids, const float* weights, const void* gate_up,
                                          const void* down, float* out, void* workspace, int T, int L, int I, int top_k,
                                          void* stream) {
  if (T <= 0) return kOk;
  if (int bad = check_plain(latent, ids, weights, gate_up, down, out, workspace, L, I, top_k)) return bad;
  return plain_experts(LX_W_BF16, latent, ids, weights, gate_up, down, out, workspace, T, L, I, top_k,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int lx_moe_experts_decode(const void* latent, const int32_t* ids, const float* weights, const lx_weight* gate_up,
                                     const lx_weight* down, float* out, void* workspace, int T, int L, int I, int top_k,
                                     void* stream) {
  if (T <= 0) return kOk;
  if (T > kDecodeMaxT || top_k < 1 || top_k > kDecodeMaxTopK || L <= 0 || I <= 0) return kInvalid;
  if (!latent || !ids || !weights || !gate_up || !down || !out || !workspace) return kInvalid;
  if (!gate_up->data || !down->data) return kInvalid;
  if (gate_up->type == LX_W_BF16X || down->type == LX_W_BF16X) {
    // lossless stacks: both must be encoded, a mixed pair has no kernel (moe_decode.cu:404-409 of the reference)
    if (gate_up->type != LX_W_BF16X || down->type != LX_W_BF16X) return kNotSupported;
    return lx_moe_experts_bf16x(latent, ids, weights, gate_up->data, down->data, out, workspace, T, L, I, top_k, stream);
  }
  if (!whole_words(gate_up->type, L) || !whole_words(down->type, I)) return kInvalid;
  if (!aligned(workspace, 16)) return kInvalid;
  if ((gate_up->type != LX_W_BF16 && !gate_up->scale) || (down->type != LX_W_BF16 && !down->scale)) return kInvalid;
  const Stack gu = make_stack(gate_up->type, gate_up->data, gate_up->scale, gate_up->expert_global, gate_up->global, 2 * I, L);
  const Stack dn = make_stack(down->type, down->data, down->scale, down->expert_global, down->global, L, I);
  return decode_experts(latent, ids, weights, gate_up->type, gu, down->type, dn, out, workspace, T, L, I, top_k,
                        static_cast<cudaStream_t>(stream));
}

// bf16 stacks, any number of tokens, no caller workspace: the intermediates live in a stream-ordered allocation for
// the length of the call, as in the reference (moe.cu:288-310). Same kernels, so the decode entry points equal it bit
// for bit.
extern "C" int lx_moe_experts(const void* latent, const int32_t* ids, const float* weights, const void* gate_up, const void* down,
                              float* out, int T, int L, int I, int top_k, void* stream) {
  if (T <= 0) return kOk;
  if (L <= 0 || I <= 0 || top_k < 1 || !latent || !ids || !weights || !gate_up || !down || !out) return kInvalid;
  auto s = static_cast<cudaStream_t>(stream);
  void* mid = nullptr;
  const cudaError_t err = cudaMallocAsync(&mid, 2ll * T * top_k * I, s);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(err);
  }
  int e = kOk;
  // the grid's second extent carries at most 65535 pairs: longer batches go in slices of whole tokens
  const int slice = std::max(1, 65535 / top_k);
  for (int t0 = 0; t0 < T && !e; t0 += slice) {
    const int n = std::min(slice, T - t0);
    e = plain_experts(LX_W_BF16, static_cast<const uint16_t*>(latent) + static_cast<int64_t>(t0) * L, ids + static_cast<int64_t>(t0) * top_k,
                      weights + static_cast<int64_t>(t0) * top_k, gate_up, down, out + static_cast<int64_t>(t0) * L,
                      static_cast<uint16_t*>(mid) + static_cast<int64_t>(t0) * top_k * I, n, L, I, top_k, s);
  }
  cudaFreeAsync(mid, s);
  return e;
}
