// Mixture-of-experts entry points of the kernel ABI: lx_moe_route and the routed experts (lx_moe_experts_grouped,
// lx_moe_experts_decode and the bf16 / BF16X variants), lernex/dromos engine/cuda/kernels.h:203-225, 495-511, 603-611.
//
// Routed experts, for T tokens each with top_k (expert, weight) pairs:
//   1. group   the T * top_k pairs are sorted by expert, stably (ascending pair index inside an expert): one CTA, a
//              thread per expert walks the ids in order. Integer work only, so the grouping is exact.
//   2. gate_up the streaming kernel per (expert, 16 gate rows + the matching 16 up rows) with the expert's tokens as
//              columns; its epilogue writes mid = bf16(silu(gate) * up) in grouped order.
//   3. down    the streaming kernel per (expert, 32 output rows) on mid; its epilogue writes weight * row per pair.
//   4. sum     out[t] = the token's top_k rows added in k order.
// Every stage reads each chosen expert's weights once; no float atomics anywhere, so a token's bits do not depend on
// the batch or the run.
#include <algorithm>
#include <mutex>

#include "launch.cuh"
#include "scalar.cuh"

namespace b200 {
namespace {

constexpr int kMaxExperts = 1024;
constexpr int kMaxTopK = 32;

// ---- routing (one warp per token) ------------------------------------------------------------------------------
// One warp routes one row of logits (global or shared memory): softmax statistics of the whole row, top_k picks by
// logit + bias (descending, ties to the lower index), weights = softmax over the picks of their unbiased logits.
// Callers hand a row in shared memory where they can: it is read 3 + top_k times.
__device__ __forceinline__ void route_row(const float* row, const float* __restrict__ bias, int E, int top_k, int lane,
                                          int32_t* __restrict__ ids, float* __restrict__ weights, float* entropy, float* confidence) {
  float m = -INFINITY;
  for (int i = lane; i < E; i += 32) m = fmaxf(m, row[i]);
  m = warp_max(m);
  float z = 0.0f;
  for (int i = lane; i < E; i += 32) z += expf(row[i] - m);
  z = warp_sum(z);
  float h = 0.0f;
  for (int i = lane; i < E; i += 32) {
    const float p = expf(row[i] - m) / z;
    h -= p * logf(fmaxf(p, 1e-9f));
  }
  h = warp_sum(h);
  if (lane == 0) {
    if (entropy) *entropy = h;
    if (confidence) *confidence = 1.0f / z;
  }
  // top_k rounds of a warp arg-max over what is left. Lane l owns elements l, l + 32, ...: bit j of `taken` says that
  // element l + 32 j has been picked (the first 1024 experts; rarer ones beyond are looked up among the picks).
  int mine = -1;  // lane j keeps pick j
  float mine_logit = -INFINITY;
  uint32_t taken = 0;
  for (int r = 0; r < top_k; ++r) {
    float best = -INFINITY;
    int best_i = E;
    for (int base = 0, j = 0; base < E; base += 32, ++j) {  // the same trip count in every lane: the shuffle below needs them all
      const int i = base + lane;
      bool gone;
      if (j < 32) {
        gone = (taken >> j) & 1u;
      } else {  // beyond 1024 experts: compare with the picks so far, which lanes 0 .. r - 1 hold
        gone = false;
        for (int q = 0; q < r; ++q) gone |= __shfl_sync(0xffffffffu, mine, q) == i;
      }
      if (gone || i >= E) continue;
      const float v = row[i] + (bias ? bias[i] : 0.0f);
      if (v > best || (v == best && i < best_i)) best = v, best_i = i;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) best = ov, best_i = oi;
    }
    if (lane == r) mine = best_i, mine_logit = best_i < E ? row[best_i] : -INFINITY;
    if (best_i < 1024 && best_i < E && (best_i & 31) == lane) taken |= 1u << (best_i >> 5);
  }
  const bool live = lane < top_k && mine >= 0 && mine < E;
  const float lmax = warp_max(live ? mine_logit : -INFINITY);
  const float ex = live ? expf(mine_logit - lmax) : 0.0f;
  const float sum = warp_sum(ex);
  if (lane < top_k) {
    ids[lane] = live ? mine : 0;
    weights[lane] = live ? ex / sum : 0.0f;
  }
}

constexpr int kRouteStaged = 1024;
__global__ void __launch_bounds__(256) route_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                    int32_t* __restrict__ ids, float* __restrict__ weights,
                                                    float* __restrict__ entropy, float* __restrict__ confidence, int T,
                                                    int E, int top_k) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= T) return;
  // the warp's row, staged once (rows of more than kRouteStaged values are read where they are)
  __shared__ float staged[8][kRouteStaged];
  const float* row = logits + static_cast<int64_t>(t) * E;
  if (E <= kRouteStaged) {
    for (int i = lane; i < E; i += 32) staged[warp][i] = row[i];
    __syncwarp();
    row = staged[warp];
  }
  route_row(row, bias, E, top_k, lane, ids + static_cast<int64_t>(t) * top_k, weights + static_cast<int64_t>(t) * top_k, entropy ? entropy + t : nullptr,
            confidence ? confidence + t : nullptr);
}

// ---- the router of a decode-sized step in one launch (lx_router_route) ---------------------------------------------
// logits[m, e] = x[m, :] . w[e, :] + bias[e] for up to 8 rows, then the routing of route_row on those logits. One warp
// per expert: its lanes walk K in float4 steps, every row's partial in registers, a fixed shuffle tree, so a logit's
// bits depend on K only. The router weights are static and are in flight before the dependency wait. The block that
// counts itself last on the ticket (which it leaves at zero again) stages the logits in shared memory and routes
// them, one warp per row, with the arithmetic of lx_moe_route: every routing output equals that call on these logits
// bit for bit.
constexpr int kRouterRows = 8, kRouterMaxE = 1024, kRouterMaxK = 2048;
__global__ void __launch_bounds__(256) router_kernel(const float* __restrict__ x, int ld_x, const float* __restrict__ w,
                                                     const float* __restrict__ bias, float* __restrict__ logits,
                                                     const float* __restrict__ selection_bias, int32_t* __restrict__ ids,
                                                     float* __restrict__ weights, float* __restrict__ entropy,
                                                     float* __restrict__ confidence, int32_t* __restrict__ ticket, int M, int E, int K,
                                                     int top_k) {
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.x * 8 + warp;
  const bool vec = K % 4 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ld_x % 4 == 0;
  // this lane's weights of the expert's row: K <= 2048 is at most 16 float4 steps of the warp
  float4 wv[kRouterMaxK / 128];
  const float* wrow = w + static_cast<int64_t>(e < E ? e : 0) * K;
#pragma unroll
  for (int q = 0; q < kRouterMaxK / 128; ++q) {
    const int k = (q * 32 + lane) * 4;
    wv[q] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (k < K) {
      if (vec) wv[q] = __ldg(reinterpret_cast<const float4*>(wrow + k));
      else wv[q] = make_float4(wrow[k], k + 1 < K ? wrow[k + 1] : 0.0f, k + 2 < K ? wrow[k + 2] : 0.0f, k + 3 < K ? wrow[k + 3] : 0.0f);
    }
  }
  const float be = bias && e < E ? bias[e] : 0.0f;
  pdl_wait();  // the activations come from the kernel before this one
  for (int m = 0; m < M; ++m) {
    const float* xr = x + static_cast<int64_t>(m) * ld_x;
    float acc = 0.0f;
#pragma unroll
    for (int q = 0; q < kRouterMaxK / 128; ++q) {
      const int k = (q * 32 + lane) * 4;
      if (k >= K) continue;
      float4 xv;
      if (vec) xv = *reinterpret_cast<const float4*>(xr + k);
      else xv = make_float4(xr[k], k + 1 < K ? xr[k + 1] : 0.0f, k + 2 < K ? xr[k + 2] : 0.0f, k + 3 < K ? xr[k + 3] : 0.0f);
      acc = fmaf(xv.x, wv[q].x, acc);
      acc = fmaf(xv.y, wv[q].y, acc);
      acc = fmaf(xv.z, wv[q].z, acc);
      acc = fmaf(xv.w, wv[q].w, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0 && e < E) logits[static_cast<int64_t>(m) * E + e] = acc + be;
  }
  // publish this block's logits, then count it; the block that counts last routes every row
  __shared__ int last;
  __shared__ float rows[kRouterRows][kRouterMaxE];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(ticket, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (threadIdx.x == 0) *ticket = 0;
  for (int i = threadIdx.x; i < M * E; i += 256) rows[i / E][i % E] = __ldcg(logits + i);
  __syncthreads();
  if (warp < M)
    route_row(rows[warp], selection_bias, E, top_k, lane, ids + static_cast<int64_t>(warp) * top_k,
              weights + static_cast<int64_t>(warp) * top_k, entropy ? entropy + warp : nullptr, confidence ? confidence + warp : nullptr);
}

// ---- the f32 GEMV the router's logits are defined by (lx_spec_gemv_f32) --------------------------------------------
// y[m, n] = x[m, :] . w[n, :] + bias[n] for up to 8 rows and any K, in exactly the order router_kernel adds: one warp
// per output column, lane l takes the float4 steps l, l + 32, ... in ascending order (x, y, z, w inside a step, one
// fmaf chain per row), then the fixed shuffle tree, then the bias. A row's bits depend on K alone, and for K <= 2048
// they are router_kernel's logits bit for bit.
__global__ void __launch_bounds__(256) rows_gemv_f32_kernel(const float* __restrict__ x, int ld_x, const float* __restrict__ w,
                                                            const float* __restrict__ bias, float* __restrict__ y, int ld_y, int M, int N,
                                                            int K) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const bool vec = K % 4 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ld_x % 4 == 0;
  const float* wrow = w + static_cast<int64_t>(n) * K;
  float acc[kRouterRows];
#pragma unroll
  for (int m = 0; m < kRouterRows; ++m) acc[m] = 0.0f;
  for (int k = lane * 4; k < K; k += 128) {
    float4 wv;
    if (vec) wv = __ldg(reinterpret_cast<const float4*>(wrow + k));
    else wv = make_float4(wrow[k], k + 1 < K ? wrow[k + 1] : 0.0f, k + 2 < K ? wrow[k + 2] : 0.0f, k + 3 < K ? wrow[k + 3] : 0.0f);
#pragma unroll
    for (int m = 0; m < kRouterRows; ++m) {
      if (m >= M) break;
      const float* xr = x + static_cast<int64_t>(m) * ld_x;
      float4 xv;
      if (vec) xv = *reinterpret_cast<const float4*>(xr + k);
      else xv = make_float4(xr[k], k + 1 < K ? xr[k + 1] : 0.0f, k + 2 < K ? xr[k + 2] : 0.0f, k + 3 < K ? xr[k + 3] : 0.0f);
      acc[m] = fmaf(xv.x, wv.x, acc[m]);
      acc[m] = fmaf(xv.y, wv.y, acc[m]);
      acc[m] = fmaf(xv.z, wv.z, acc[m]);
      acc[m] = fmaf(xv.w, wv.w, acc[m]);
    }
  }
  const float b = bias ? bias[n] : 0.0f;
#pragma unroll
  for (int m = 0; m < kRouterRows; ++m) {
    if (m >= M) break;
    const float sum = warp_sum(acc[m]);
    if (lane == 0) y[static_cast<int64_t>(m) * ld_y + n] = sum + b;
  }
}

// ---- grouping --------------------------------------------------------------------------------------------------
// offsets[e] = pairs of experts below e; pairs[offsets[e] + j] = the j-th pair (ascending) that chose expert e.
// One CTA of 1024 threads, thread e walks the ids (staged in shared memory when there are at most 8192 of them: the
// walk is then ~P shared-memory reads, not P dependent global loads); E <= 1024.
constexpr int kGroupStaged = 8192;
// own0 .. own1 - 1: the experts whose rows get chunks (all of them on one GPU; a rank's own experts when the experts are
// split over ranks, and then a chunk names its expert by its index in the rank's stack). Rows of the other experts get
// chunk -1: nothing is prepared or multiplied for them.
__global__ void __launch_bounds__(1024) group_kernel(const int32_t* __restrict__ ids, int P, int E,
                                                     int32_t* __restrict__ offsets, int32_t* __restrict__ pairs,
                                                     const ExpertChunkTables chunks, int own0, int own1) {
  pdl_trigger();
  pdl_wait();
  __shared__ int32_t start[kMaxExperts + 1];
  __shared__ int32_t staged[kGroupStaged];
  const int e = threadIdx.x;
  const bool in_smem = P <= kGroupStaged;
  if (in_smem) {
    for (int p = e; p < P; p += 1024) staged[p] = ids[p];
    __syncthreads();
  }
  const int32_t* src = in_smem ? staged : ids;
  int count = 0;
  if (e < E)
    for (int p = 0; p < P; ++p) count += src[p] == e;
  start[e] = e < E ? count : 0;
  __syncthreads();
  if (e == 0) {
    int run = 0;
    for (int i = 0; i < E; ++i) {
      const int c = start[i];
      start[i] = run;
      run += c;
    }
    start[E] = run;
  }
  __syncthreads();
  if (e <= E) offsets[e] = start[e];
  if (e == 0) offsets[E] = start[E];  // with E equal to the thread count no thread has e == E
  const int row0 = e < E ? start[e] : 0, rows = count;
  if (e < E) {
    int at = row0;
    for (int p = 0; p < P && count > 0; ++p)
      if (src[p] == e) pairs[at++] = p, --count;
  }
  // The chunk tables of the tensor-core expert kernels: expert e's rows cut into chunks of up to 16.
  if (chunks.n_chunks) {
    __syncthreads();  // everyone has read start[]; it now holds each expert's chunk count
    const bool own = e >= own0 && e < own1;
    const int mine = own ? (rows + kExpertChunkRows - 1) / kExpertChunkRows : 0;
    if (e < E && !own)
      for (int m = 0; m < rows; ++m) chunks.pos_chunk[row0 + m] = -1;
    start[e] = e < E ? mine : 0;
    __syncthreads();
    int base = 0;
    for (int q = 0; q < e && q < E; ++q) base += start[q];
    if (e == E - 1) *chunks.n_chunks = base + mine;
    for (int j = 0; j < mine; ++j) {
      const int c = base + j, first = row0 + j * kExpertChunkRows, n = min(kExpertChunkRows, rows - j * kExpertChunkRows);
      chunks.chunk_expert[c] = e - own0, chunks.chunk_row0[c] = first, chunks.chunk_rows[c] = n;
      for (int m = 0; m < n; ++m) chunks.pos_chunk[first + m] = c, chunks.pos_col[first + m] = m;
    }
  }
}

// The same tables for up to 1024 pairs (every decode-sized call), a thread per pair instead of a thread per expert
// walking all ids: a pair's place among its expert's pairs is how many earlier pairs chose the same expert (a scan of
// the staged ids, broadcast reads), the experts' counts are scanned by the whole block, and every thread writes its
// own table entries. (The thread-per-expert kernel above took 22 us of a 233 us step at 256 pairs.)
__device__ __forceinline__ int block_exclusive_scan_1024(int x, int* warp_totals, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int v = x;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) warp_totals[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = warp_totals[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    warp_totals[lane] = w;  // inclusive
  }
  __syncthreads();
  const int before = warp ? warp_totals[warp - 1] : 0;
  if (total) *total = warp_totals[31];
  __syncthreads();  // warp_totals may be reused by the caller
  return before + v - x;
}

static_assert(kMaxExperts == 1024, "group_pairs_kernel zeroes one count per thread of its 1024");
__global__ void __launch_bounds__(1024) group_pairs_kernel(const int32_t* __restrict__ ids, int P, int E,
                                                           int32_t* __restrict__ offsets, int32_t* __restrict__ pairs,
                                                           const ExpertChunkTables chunks, int own0, int own1) {
  pdl_trigger();
  pdl_wait();
  __shared__ __align__(16) int32_t sid[1024];
  __shared__ int32_t count[kMaxExperts], start[kMaxExperts], chunk0[kMaxExperts];
  __shared__ int warp_totals[32];
  const int p = threadIdx.x;
  const int mine = p < P ? ids[p] : -1;
  sid[p] = mine;
  count[p] = 0;  // kMaxExperts == the block size
  __syncthreads();
  int rank = 0;
  const bool valid = p < P && mine >= 0 && mine < E;  // a pair with an id outside the experts is left out of the tables
  if (valid) {
    const int4* v = reinterpret_cast<const int4*>(sid);
    const int whole = p >> 2;
    for (int q = 0; q < whole; ++q) {
      const int4 w = v[q];
      rank += (w.x == mine) + (w.y == mine) + (w.z == mine) + (w.w == mine);
    }
    for (int q = whole * 4; q < p; ++q) rank += sid[q] == mine;
    atomicAdd(&count[mine], 1);
  }
  __syncthreads();
  const int e = threadIdx.x;
  const int rows = e < E ? count[e] : 0;
  int total = 0;
  const int first = block_exclusive_scan_1024(rows, warp_totals, &total);
  start[e] = first;
  if (e < E) offsets[e] = first;
  if (e == 0) offsets[E] = total;
  const bool own = e >= own0 && e < own1;
  int n_chunks = 0;
  if (chunks.n_chunks) {
    const int c0 = block_exclusive_scan_1024(own && e < E ? (rows + kExpertChunkRows - 1) / kExpertChunkRows : 0, warp_totals, &n_chunks);
    chunk0[e] = c0;
    if (e == 0) *chunks.n_chunks = n_chunks;
  }
  __syncthreads();
  if (!valid) return;
  const int u = start[mine] + rank;  // the pair's sorted position: stable, ascending pair index inside an expert
  pairs[u] = p;
  if (chunks.n_chunks) {
    if (mine >= own0 && mine < own1) {
      const int c = chunk0[mine] + rank / kExpertChunkRows, col = rank % kExpertChunkRows;
      chunks.pos_chunk[u] = c, chunks.pos_col[u] = col;
      if (col == 0)
        chunks.chunk_expert[c] = mine - own0, chunks.chunk_row0[c] = u, chunks.chunk_rows[c] = min(kExpertChunkRows, count[mine] - rank);
    } else {
      chunks.pos_chunk[u] = -1;
    }
  }
}

// Picks the kernel by the number of pairs.
int launch_group(const int32_t* ids, int P, int E, int32_t* offsets, int32_t* pairs, const ExpertChunkTables& chunks, int own0, int own1,
                 cudaStream_t s) {
  if (P <= 1024) return launch_kernel(group_pairs_kernel, dim3(1), dim3(1024), 0, s, ids, P, E, offsets, pairs, chunks, own0, own1);
  return launch_kernel(group_kernel, dim3(1), dim3(1024), 0, s, ids, P, E, offsets, pairs, chunks, own0, own1);
}

// Grouping without knowing E (the decode entry points): the distinct experts of the ids in ascending order.
// groups[g] = expert, offsets[g], pairs as above; unused groups get empty ranges. One CTA; P <= 1024.
__global__ void __launch_bounds__(1024) group_small_kernel(const int32_t* __restrict__ ids, int P,
                                                           int32_t* __restrict__ group_expert,
                                                           int32_t* __restrict__ offsets, int32_t* __restrict__ pairs) {
  pdl_trigger();
  pdl_wait();
  __shared__ int32_t sid[1024];
  __shared__ int32_t first[1024];  // 1 when pair p is the first (lowest p) with its expert
  __shared__ int32_t rank[1024];
  const int p = threadIdx.x;
  sid[p] = p < P ? ids[p] : 0x7fffffff;
  __syncthreads();
  int is_first = p < P;
  int smaller = 0;  // distinct experts below mine = my group index (counted on first occurrences)
  int before = 0;   // pairs of my expert before me
  if (p < P) {
    for (int q = 0; q < p; ++q) {
      if (sid[q] == sid[p]) is_first = 0, ++before;
    }
  }
  first[p] = is_first;
  __syncthreads();
  int members = 0;  // pairs of my expert
  if (p < P) {
    for (int q = 0; q < P; ++q) {
      smaller += first[q] && sid[q] < sid[p];
      members += sid[q] == sid[p];
    }
  }
  rank[p] = smaller;
  // pairs with a smaller expert id than mine = where my group starts
  int below = 0;
  if (p < P)
    for (int q = 0; q < P; ++q) below += sid[q] < sid[p];
  if (p < P) {
    pairs[below + before] = p;
    if (is_first) {
      group_expert[smaller] = sid[p];
      offsets[smaller] = below;
    }
  }
  __syncthreads();
  // groups past the last distinct expert: empty, starting at P
  int groups = 0;
  for (int q = 0; q < P; ++q) groups += first[q];
  if (p <= P && p >= groups) offsets[p] = P;
  if (p < P && p >= groups) group_expert[p] = 0;
}

// out[t, l] = sum over k, in order, of rows[t * top_k + k, l]
__global__ void __launch_bounds__(256) ordered_sum_kernel(const float* __restrict__ rows, float* __restrict__ out, int T,
                                                          int L, int top_k) {
  pdl_trigger();
  pdl_wait();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= static_cast<int64_t>(T) * L) return;
  const int64_t t = i / L, l = i % L;
  float acc = 0.0f;
  for (int k = 0; k < top_k; ++k) acc += rows[(t * top_k + k) * L + l];
  out[i] = acc;
}

// ---- scalar expert stages (shapes the streaming kernel does not take): one warp per output value --------------------
// mid[p, i] = bf16(silu(s_g * gate_i . x) * (s_u * up_i . x)) for pair p = t * top_k + k, rows by pair index.
template <int F>
__global__ void __launch_bounds__(256) scalar_gate_up_kernel(const StreamParams P, const int32_t* __restrict__ ids, int pairs) {
  pdl_trigger();
  pdl_wait();
  const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (w >= static_cast<int64_t>(pairs) * P.I) return;
  const int p = static_cast<int>(w / P.I), i = static_cast<int>(w % P.I), lane = threadIdx.x & 31;
  const int e = ids[p];
  const uint16_t* x = static_cast<const uint16_t*>(P.x) + static_cast<int64_t>(p / P.top_k) * P.ld_x;
  const int64_t ng = static_cast<int64_t>(e) * P.N + i, nu = ng + P.I;
  float g = 0.0f, u = 0.0f;
  for (int k = lane; k < P.K; k += 32) {
    const float xv = bf16_bits_to_f32(x[k]);
    g = fmaf(xv, weight_element<F>(P, ng, k), g);
    u = fmaf(xv, weight_element<F>(P, nu, k), u);
  }
  g = warp_sum(g) * scalar_row_factor<F>(P, ng, e);
  u = warp_sum(u) * scalar_row_factor<F>(P, nu, e);
  if (lane == 0) static_cast<uint16_t*>(P.moe_out)[w] = static_cast<uint16_t>(f32_to_bf16_bits(g / (1.0f + expf(-g)) * u));
}

// rows[p, l] = weight[p] * (s_l * down_l . mid[p])
template <int F>
__global__ void __launch_bounds__(256) scalar_down_kernel(const StreamParams P, const int32_t* __restrict__ ids, int pairs) {
  pdl_trigger();
  pdl_wait();
  const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (w >= static_cast<int64_t>(pairs) * P.N) return;
  const int p = static_cast<int>(w / P.N), l = static_cast<int>(w % P.N), lane = threadIdx.x & 31;
  const int e = ids[p];
  const uint16_t* x = static_cast<const uint16_t*>(P.x) + static_cast<int64_t>(p) * P.ld_x;
  const int64_t n = static_cast<int64_t>(e) * P.N + l;
  float acc = 0.0f;
  for (int k = lane; k < P.K; k += 32) acc = fmaf(bf16_bits_to_f32(x[k]), weight_element<F>(P, n, k), acc);
  acc = warp_sum(acc);
  if (lane == 0) static_cast<float*>(P.moe_out)[w] = P.route_w[p] * (scalar_row_factor<F>(P, n, e) * acc);
}

template <int F>
int launch_scalar_stage(bool gate_up, const StreamParams& P, const int32_t* ids, int pairs, cudaStream_t s) {
  const int64_t warps = static_cast<int64_t>(pairs) * (gate_up ? P.I : P.N);
  const dim3 grid(static_cast<unsigned>((warps + 7) / 8));
  return gate_up ? launch_kernel(scalar_gate_up_kernel<F>, grid, dim3(256), 0, s, P, ids, pairs)
                 : launch_kernel(scalar_down_kernel<F>, grid, dim3(256), 0, s, P, ids, pairs);
}
int launch_scalar_stage(bool gate_up, int type, const StreamParams& P, const int32_t* ids, int pairs, cudaStream_t s) {
  switch (type) {
    case LX_W_BF16: return launch_scalar_stage<LX_W_BF16>(gate_up, P, ids, pairs, s);
    case LX_W_INT8: return launch_scalar_stage<LX_W_INT8>(gate_up, P, ids, pairs, s);
    case LX_W_FP8: return launch_scalar_stage<LX_W_FP8>(gate_up, P, ids, pairs, s);
    case LX_W_NVFP4: return launch_scalar_stage<LX_W_NVFP4>(gate_up, P, ids, pairs, s);
    case LX_W_BF16X: return launch_scalar_stage<LX_W_BF16X>(gate_up, P, ids, pairs, s);
  }
  return kInvalid;
}

int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

struct Layout {
  int64_t offsets, group_expert, pairs, mid, rows, total;
};
// groups: the number of expert groups the tables hold (E, or P when E is not known)
Layout layout(int P, int groups, int L, int I) {
  Layout l{};
  int64_t o = 0;
  auto take = [&](int64_t bytes) {
    const int64_t at = o;
    o = round_up(o + bytes, 256);
    return at;
  };
  l.offsets = take(4ll * (groups + 1));
  l.group_expert = take(4ll * groups);
  l.pairs = take(4ll * P);
  l.mid = take(2ll * P * I);
  l.rows = take(4ll * P * L);
  l.total = o;
  return l;
}

int row_bytes_of(int type, int K) {
  switch (type) {
    case LX_W_BF16: return 2 * K;
    case LX_W_NVFP4: return K / 2;
    case LX_W_BF16X: return static_cast<int>(x16::row_bytes(K));
    default: return K;
  }
}

bool stack_streams(const lx_weight& w, int K) {
  switch (w.type) {
    case LX_W_BF16: return K % 32 == 0 && aligned(w.data, 16);
    case LX_W_INT8:
    case LX_W_FP8: return K % 64 == 0 && aligned(w.data, 16);
    case LX_W_NVFP4: return K % 256 == 0 && aligned(w.data, 16) && aligned(w.scale, 16);
    case LX_W_BF16X: return K % 32 == 0 && aligned(w.data, 8);
    default: return false;
  }
}

template <int MODE>
int launch_expert_stage(const StreamParams& P, int type, cudaStream_t s, int64_t stack_rows) {
  switch (type) {
    case LX_W_BF16: return launch_stream<LX_W_BF16, 8, 1, 2, 2, 2, 4, 32, MODE>(P, s, stack_rows);
    case LX_W_INT8: return launch_stream<LX_W_INT8, 8, 1, 2, 2, 2, 4, 32, MODE>(P, s, stack_rows);
    case LX_W_FP8: return launch_stream<LX_W_FP8, 8, 1, 2, 2, 2, 4, 32, MODE>(P, s, stack_rows);
    case LX_W_NVFP4: return launch_stream<LX_W_NVFP4, 8, 1, 2, 2, 2, 4, 32, MODE>(P, s, stack_rows);
    case LX_W_BF16X: return launch_stream<LX_W_BF16X, 8, 1, 2, 2, 2, 4, 32, MODE>(P, s, stack_rows);
  }
  return kInvalid;
}

// Stages 2-4 on grouping tables already in the workspace. groups = grid extent over expert groups.
int run_experts(const void* latent, const int32_t* ids, const float* weights, const lx_weight& gate_up, const lx_weight& down,
                float* out,
                uint8_t* ws, const Layout& l, bool indirect, int groups, int experts, int T, int L, int I, int top_k,
                cudaStream_t s, int* status = nullptr, bool quantized = false) {
  StreamParams g{};
  g.w = static_cast<const uint8_t*>(gate_up.data);
  g.scale = static_cast<const uint8_t*>(gate_up.scale);
  g.global = gate_up.global;
  g.expert_global = gate_up.type == LX_W_NVFP4 ? gate_up.expert_global : nullptr;
  g.row_bytes = row_bytes_of(gate_up.type, L);
  g.N = 2 * I, g.K = L;
  g.x = latent, g.x_dtype = LX_BF16, g.ld_x = L, g.M = T;
  g.x_vec = aligned(latent, 16) && L % 8 == 0;
  g.groups = groups;
  g.offsets = reinterpret_cast<const int32_t*>(ws + l.offsets);
  g.group_expert = indirect ? reinterpret_cast<const int32_t*>(ws + l.group_expert) : nullptr;
  g.pairs = reinterpret_cast<const int32_t*>(ws + l.pairs);
  g.route_w = weights;
  g.top_k = top_k, g.I = I;
  g.moe_out = ws + l.mid;
  g.status = status ? status : status_word();
  // Both stacks in a format the tensor core reads as stored: the tcgen05 kernels (their tables and activation blocks
  // sit behind this layout in the workspace), then the same ordered sum.
  if (!indirect && experts_tc_ok(gate_up, down, L, I)) {
    if (int e = experts_tc(latent, weights, gate_up, down, reinterpret_cast<const int32_t*>(ws + l.offsets),
                           reinterpret_cast<const int32_t*>(ws + l.pairs), reinterpret_cast<uint16_t*>(ws + l.mid),
                           reinterpret_cast<float*>(ws + l.rows), ws, l.total, T, L, I, experts, top_k, g.status, s, quantized))
      return e;
    const int64_t n = static_cast<int64_t>(T) * L;
    return launch_kernel(ordered_sum_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s,
                         reinterpret_cast<const float*>(ws + l.rows), out, T, L, top_k);
  }
  if (quantized) return kNotSupported;  // the low-precision maths exist on the tensor-core kernels only
  // weights the streaming kernel cannot take run both stages on the scalar kernels (intermediate rows by pair index)
  const bool fast_gu = stack_streams(gate_up, L) && stack_streams(down, I), fast_dn = fast_gu;
  if (int e = fast_gu ? launch_expert_stage<kGateUp>(g, gate_up.type, s, static_cast<int64_t>(experts) * 2 * I)
                      : launch_scalar_stage(true, gate_up.type, g, ids, T * top_k, s))
    return e;

  StreamParams d = g;
  d.w = static_cast<const uint8_t*>(down.data);
  d.scale = static_cast<const uint8_t*>(down.scale);
  d.global = down.global;
  d.expert_global = down.type == LX_W_NVFP4 ? down.expert_global : nullptr;
  d.row_bytes = row_bytes_of(down.type, I);
  d.N = L, d.K = I;
  d.x = ws + l.mid, d.ld_x = I;
  d.x_vec = I % 8 == 0;
  d.moe_out = ws + l.rows;
  if (int e = fast_dn ? launch_expert_stage<kDown>(d, down.type, s, static_cast<int64_t>(experts) * L)
                      : launch_scalar_stage(false, down.type, d, ids, T * top_k, s))
    return e;

  const int64_t n = static_cast<int64_t>(T) * L;
  return launch_kernel(ordered_sum_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s,
                       reinterpret_cast<const float*>(ws + l.rows), out, T, L, top_k);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int lx_moe_route(const float* logits, const float* selection_bias, int32_t* ids, float* weights,
                            float* entropy, float* confidence, int T, int E, int top_k, void* stream) {
  if (T <= 0) return kOk;
  if (top_k < 1 || top_k > kMaxTopK || top_k > E || !logits || !ids || !weights) return kInvalid;
  return launch_kernel(route_kernel, dim3((T + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), logits,
                       selection_bias, ids, weights, entropy, confidence, T, E, top_k);
}

extern "C" int lx_router_route(const float* x, int ld_x, const float* w, const float* bias, float* logits,
                               const float* selection_bias, int32_t* ids, float* weights, float* entropy, float* confidence,
                               int32_t* ticket, int M, int E, int K, int top_k, void* stream) {
  if (M <= 0) return kOk;
  if (M > kRouterRows || E < 1 || E > kRouterMaxE || K < 1 || K > kRouterMaxK || top_k < 1 || top_k > kMaxTopK || top_k > E)
    return kInvalid;
  if (!x || !w || !logits || !ids || !weights || !ticket || ld_x < K) return kInvalid;
  return launch_kernel(router_kernel, dim3((E + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), x, ld_x, w, bias, logits,
                       selection_bias, ids, weights, entropy, confidence, ticket, M, E, K, top_k);
}

extern "C" int lx_spec_gemv_f32(const float* x, int ld_x, const float* w, const float* bias, float* y, int ld_y, int M, int N, int K,
                                void* stream) {
  if (M == 0 || N == 0) return kOk;
  if (M < 0 || M > kRouterRows || K <= 0 || ld_x < K || ld_y < N || !x || !w || !y) return kInvalid;
  return launch_kernel(rows_gemv_f32_kernel, dim3((N + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), x, ld_x, w, bias, y, ld_y, M,
                       N, K);
}

extern "C" int64_t lx_moe_grouped_workspace_bytes(int T, int L, int I, int E, int top_k, lx_math math) {
  (void)math;
  if (T <= 0 || L <= 0 || I <= 0 || E <= 0 || top_k <= 0) return 0;
  // the grouping tables and buffers, then what the tensor-core path adds (chunk tables, activation blocks)
  return experts_tc_workspace(layout(T * top_k, E, L, I).total, T * top_k, E, L, I);
}

extern "C" int lx_moe_experts_grouped(const void* latent, const int32_t* ids, const float* weights,
                                      const lx_weight* gate_up, const lx_weight* down, lx_math math, float* out,
                                      void* workspace, int T, int L, int I, int E, int top_k, void* stream) {
  if (T < 0 || L <= 0 || I <= 0 || E <= 0 || top_k <= 0 || top_k > E || !gate_up || !down) return kInvalid;
  if (math < LX_MATH_BF16 || math > LX_MATH_FP4) return kInvalid;
  if (T == 0) return kOk;
  if (!latent || !ids || !weights || !out || !workspace || !gate_up->data || !down->data) return kInvalid;
  // formats this entry point does not take (the lossless BF16X among them) are "not supported", whatever their scale pointers
  if (gate_up->type < LX_W_BF16 || gate_up->type > LX_W_NVFP4 || down->type < LX_W_BF16 || down->type > LX_W_NVFP4)
    return kNotSupported;
  if ((gate_up->type != LX_W_BF16 && !gate_up->scale) || (down->type != LX_W_BF16 && !down->scale)) return kInvalid;
  if (E > kMaxExperts || static_cast<int64_t>(T) * top_k > (1ll << 30)) return kNotSupported;
  // One math for both stages, admitted per stack as lx_gemm_w admits it (engine/cuda/moe_grouped.cu:400-402).
  const bool quantized = math != LX_MATH_BF16;
  if (int e = math_admitted(math, gate_up->type)) return e;
  if (int e = math_admitted(math, down->type)) return e;
  if (quantized && !experts_tc_ok(*gate_up, *down, L, I)) return kNotSupported;
  if (I % 8 != 0 || L % 8 != 0) return kNotSupported;
  if (gate_up->type == LX_W_NVFP4 && (L % 16 != 0 || I % 16 != 0)) return kInvalid;
  auto s = static_cast<cudaStream_t>(stream);
  const int P = T * top_k;
  const Layout l = layout(P, E, L, I);
  auto* ws = static_cast<uint8_t*>(workspace);
  const ExpertChunkTables chunks = experts_tc_ok(*gate_up, *down, L, I) ? expert_chunk_tables(ws, l.total, P, E, L, I) : ExpertChunkTables{};
  if (int e = launch_group(ids, P, E, reinterpret_cast<int32_t*>(ws + l.offsets), reinterpret_cast<int32_t*>(ws + l.pairs), chunks, 0, E, s))
    return e;
  return run_experts(latent, ids, weights, *gate_up, *down, out, ws, l, false, E, E, T, L, I, top_k, s, nullptr, quantized);
}

// ---- routed experts split over ranks (no counterpart in the reference, which is single-GPU) ----------------------------
// Routing is replicated (every rank routes the same logits), and so are the tokens: at decode sizes the latent is a few
// hundred KB, less than a dispatch would cost. A rank holds the stacks of its own experts only and computes the
// weighted rows of the pairs that chose them (lx_b200_moe_experts_owned: grouping with an owned range, the two expert
// stages); the rows then travel to every rank as flag-in-data packets (lx_b200_moe_exchange_rows) and every rank adds
// each token's rows in k order (lx_b200_moe_sum_rows), exactly what one GPU with all experts adds: the result does not
// depend on how the experts are split. Nothing here reads a device value on the host, so the three calls can be
// captured in a graph.
extern "C" int lx_b200_moe_experts_owned(const void* latent, const int32_t* ids, const float* weights, const lx_weight* gate_up,
                                         const lx_weight* down, lx_math math, float* rows, void* workspace, int T, int L, int I,
                                         int E, int own0, int own1, int top_k, void* stream) {
  if (T < 0 || L <= 0 || I <= 0 || E <= 0 || top_k <= 0 || top_k > E) return kInvalid;
  if (own0 < 0 || own1 < own0 || own1 > E) return kInvalid;
  if (math < LX_MATH_BF16 || math > LX_MATH_FP4) return kInvalid;
  if (T == 0) return kOk;
  if (!ids || !workspace) return kInvalid;
  if (E > kMaxExperts || static_cast<int64_t>(T) * top_k > (1ll << 30)) return kNotSupported;
  if (I % 8 != 0 || L % 8 != 0) return kNotSupported;
  auto s = static_cast<cudaStream_t>(stream);
  const int P = T * top_k;
  const Layout l = layout(P, E, L, I);
  auto* ws = static_cast<uint8_t*>(workspace);
  // The grouping tables are written whatever the owned range is: the row exchange reads them on every rank, also on a
  // rank that owns no expert (more ranks than experts) and therefore holds no stacks.
  const ExpertChunkTables chunks = expert_chunk_tables(ws, l.total, P, E, L, I);
  if (int e = launch_group(ids, P, E, reinterpret_cast<int32_t*>(ws + l.offsets), reinterpret_cast<int32_t*>(ws + l.pairs), chunks, own0, own1, s))
    return e;
  if (own1 == own0) return kOk;
  if (!gate_up || !down || !latent || !weights || !rows || !gate_up->data || !down->data) return kInvalid;
  if (gate_up->type < LX_W_BF16 || gate_up->type > LX_W_NVFP4 || down->type < LX_W_BF16 || down->type > LX_W_NVFP4)
    return kNotSupported;
  if ((gate_up->type != LX_W_BF16 && !gate_up->scale) || (down->type != LX_W_BF16 && !down->scale)) return kInvalid;
  if (int e = math_admitted(math, gate_up->type)) return e;
  if (int e = math_admitted(math, down->type)) return e;
  if (!experts_tc_ok(*gate_up, *down, L, I)) return kNotSupported;  // the tensor-core kernels only
  return experts_tc(latent, weights, *gate_up, *down, reinterpret_cast<const int32_t*>(ws + l.offsets),
                    reinterpret_cast<const int32_t*>(ws + l.pairs), reinterpret_cast<uint16_t*>(ws + l.mid), rows, ws, l.total, T, L, I, E,
                    top_k, status_word(), s, math != LX_MATH_BF16, own1 - own0);
}

namespace b200 {
namespace {
constexpr int kStatusRowsPoll = 8;  // a peer's rows did not arrive in time

struct RowPacketParams {
  float* rows;              // f32 [P, L] by pair index
  const int32_t* offsets;   // [E + 1] sorted position of every expert's first pair
  const int32_t* pairs;     // [P] the pair at every sorted position
  uint4* box[8];            // every rank's receive buffer: two halves of P * L / 2 packets, indexed like rows
  int64_t half_packets;     // packets per half
  int bound[9];             // rank r owns experts bound[r] .. bound[r + 1] - 1
  uint32_t* seq;
  int* done;
  int ranks, self, L;
  int* status;
  uint64_t budget_ns;
};

// As exchange_packets_kernel (exchange.cu), for rows picked by the grouping tables: a rank sends the rows of the sorted
// positions of its own experts and polls those of every other rank's experts; a packet's place in the buffer is the
// place of its 8 bytes in `rows`.
__global__ void __launch_bounds__(256) exchange_rows_kernel(const RowPacketParams P) {
  pdl_trigger();
  pdl_wait();
  uint32_t seq;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seq) : "l"(P.seq) : "memory");
  const int64_t half = static_cast<int64_t>(seq & 1u) * P.half_packets;  // the half this call's parity names, on every rank alike
  seq += 1;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x, nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int units = P.L / 2;
  {
    const int u0 = P.offsets[P.bound[P.self]], u1 = P.offsets[P.bound[P.self + 1]];
    const int64_t total = static_cast<int64_t>(u1 - u0) * units;
    for (int64_t i = tid; i < total; i += nthreads) {
      const int u = u0 + static_cast<int>(i / units);
      const int64_t at = static_cast<int64_t>(P.pairs[u]) * units + (i % units);
      const uint2 d = reinterpret_cast<const uint2*>(P.rows)[at];
      for (int r = 0; r < P.ranks; ++r)
        if (r != P.self)
          asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(P.box[r] + half + at), "r"(d.x), "r"(seq), "r"(d.y), "r"(seq) : "memory");
    }
  }
  const uint64_t t0 = global_timer_ns();
  bool gave_up = false;
  for (int r = 0; r < P.ranks && !gave_up; ++r) {
    if (r == P.self) continue;
    const int u0 = P.offsets[P.bound[r]], u1 = P.offsets[P.bound[r + 1]];
    const int64_t total = static_cast<int64_t>(u1 - u0) * units;
    for (int64_t i = tid; i < total && !gave_up; i += nthreads) {
      const int u = u0 + static_cast<int>(i / units);
      const int64_t at = static_cast<int64_t>(P.pairs[u]) * units + (i % units);
      uint32_t a, fa, b, fb;
      for (int spin = 0;; ++spin) {
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(fa), "=r"(b), "=r"(fb) : "l"(P.box[P.self] + half + at) : "memory");
        if (fa == seq && fb == seq) break;
        if ((spin & 63) == 63 && global_timer_ns() - t0 > P.budget_ns) {
          gave_up = true;
          break;
        }
      }
      if (gave_up) break;
      reinterpret_cast<uint2*>(P.rows)[at] = make_uint2(a, b);
    }
  }
  if (gave_up && P.status) atomicExch(P.status, kStatusRowsPoll);
  __syncthreads();
  if (threadIdx.x != 0) return;
  __threadfence();
  int before;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(before) : "l"(P.done) : "memory");
  if (before != static_cast<int>(gridDim.x) - 1) return;
  asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(P.done), "r"(0) : "memory");
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(P.seq), "r"(seq) : "memory");
}
}  // namespace
}  // namespace b200

// workspace: the one lx_b200_moe_experts_owned just used with the same T, L, I, E, top_k (its grouping tables are read).
// boxes: every rank's receive buffer of 2 * half_packets packets of 16 bytes (peer-mapped, zeroed once), half_packets >=
// T * top_k * L / 2: a call uses the half its sequence number's parity names. seq, done: two zeroed words of this rank's
// memory that belong to the buffers; bounds: ranks + 1 expert indices.
extern "C" int lx_b200_moe_exchange_rows(float* rows, const void* workspace, void* const* boxes, int64_t half_packets, uint32_t* seq,
                                         int* done, int ranks, int rank, const int* bounds, int T, int L, int I, int E, int top_k,
                                         void* stream) {
  if (!rows || !workspace || !boxes || !seq || !done || !bounds || ranks < 1 || ranks > 8 || rank < 0 || rank >= ranks) return kInvalid;
  if (T <= 0) return kOk;
  if (L <= 0 || L % 2 != 0 || I <= 0 || E <= 0 || top_k <= 0 || !aligned(rows, 8)) return kInvalid;
  RowPacketParams P{};
  for (int r = 0; r <= ranks; ++r) {
    if (bounds[r] < 0 || bounds[r] > E || (r > 0 && bounds[r] < bounds[r - 1])) return kInvalid;
    P.bound[r] = bounds[r];
  }
  if (bounds[0] != 0 || bounds[ranks] != E) return kInvalid;
  for (int r = 0; r < ranks; ++r) {
    if (!boxes[r] || !aligned(boxes[r], 16)) return kInvalid;
    P.box[r] = static_cast<uint4*>(boxes[r]);
  }
  const int Pn = T * top_k;
  if (half_packets < static_cast<int64_t>(Pn) * (L / 2)) return kInvalid;
  P.half_packets = half_packets;
  const Layout l = layout(Pn, E, L, I);
  const auto* ws = static_cast<const uint8_t*>(workspace);
  P.rows = rows;
  P.offsets = reinterpret_cast<const int32_t*>(ws + l.offsets);
  P.pairs = reinterpret_cast<const int32_t*>(ws + l.pairs);
  P.seq = seq, P.done = done;
  P.ranks = ranks, P.self = rank, P.L = L;
  P.status = status_word();
  uint64_t ms = 1000;  // LX_B200_WAIT_MS: how long the polls may last (default 1000; read on every call)
  if (const char* v = std::getenv("LX_B200_WAIT_MS")) ms = static_cast<uint64_t>(std::max(1, std::min(10000, atoi(v))));
  P.budget_ns = ms * 1000000ull;
  const int64_t most = static_cast<int64_t>(Pn) * (L / 2);
  const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(148, (most + 1023) / 1024)));
  return launch_kernel(exchange_rows_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), P);
}

// out[t, :] = rows[t * top_k + 0, :] + rows[t * top_k + 1, :] + ... in that order (the last stage of lx_moe_experts_grouped).
extern "C" int lx_b200_moe_sum_rows(const float* rows, float* out, int T, int L, int top_k, void* stream) {
  if (T <= 0) return kOk;
  if (!rows || !out || L <= 0 || top_k <= 0) return kInvalid;
  const int64_t n = static_cast<int64_t>(T) * L;
  return launch_kernel(ordered_sum_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream), rows,
                       out, T, L, top_k);
}

// ---- the same routed experts with no allocation anywhere -------------------------------------------------------------
// Some callers cannot let a library allocate: a server that has already handed every free byte of device memory to its
// own arena (so a later cudaMalloc fails or evicts), or a decode loop that is forbidden to enter the driver's allocator
// because that takes a device-wide lock at an unpredictable moment. For them the scratch of lx_moe_experts_grouped
// (grouping tables, the bf16 intermediate, the per-pair rows) lives in a fixed array inside the library image instead of
// a caller workspace. Every GPU that loads the library holds these kStaticScratchBytes until the process exits.
constexpr int64_t kStaticScratchBytes = 8ll << 20;
constexpr int64_t kStaticHeaderBytes = 256;  // the first bytes hold this entry point's kernel status word
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
std::mutex g_static_mu;
uint8_t* g_static_base[64] = {};
// In host code `g_static_scratch` is only a handle: the address kernels can use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
int static_scratch(uint8_t** ptr) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return static_cast<int>(cudaGetLastError());
  dev &= 63;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_base[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return static_cast<int>(e);
    }
    g_static_base[dev] = static_cast<uint8_t*>(p);
  }
  *ptr = g_static_base[dev];
  return kOk;
}
}  // namespace

namespace b200 {
int* static_scratch_status() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_static_mu);
  return reinterpret_cast<int*>(g_static_base[dev & 63]);
}
}  // namespace b200

extern "C" int64_t lx_b200_moe_static_scratch_bytes(void) { return kStaticScratchBytes - kStaticHeaderBytes; }

extern "C" void* lx_b200_moe_static_scratch_ptr(void) {
  uint8_t* base = nullptr;
  return static_scratch(&base) == kOk ? base : nullptr;
}

extern "C" int lx_b200_moe_experts_grouped_static(const void* latent, const int32_t* ids, const float* weights,
                                                  const lx_weight* gate_up, const lx_weight* down, lx_math math, float* out,
                                                  int T, int L, int I, int E, int top_k, void* stream) {
  if (T < 0 || L <= 0 || I <= 0 || E <= 0 || top_k <= 0 || top_k > E || !gate_up || !down) return kInvalid;
  if (math < LX_MATH_BF16 || math > LX_MATH_FP4) return kInvalid;
  if (T == 0) return kOk;
  if (!latent || !ids || !weights || !out || !gate_up->data || !down->data) return kInvalid;
  if ((gate_up->type != LX_W_BF16 && !gate_up->scale) || (down->type != LX_W_BF16 && !down->scale)) return kInvalid;
  if (E > kMaxExperts || static_cast<int64_t>(T) * top_k > (1ll << 30)) return kNotSupported;
  if (gate_up->type < LX_W_BF16 || gate_up->type > LX_W_NVFP4 || down->type < LX_W_BF16 || down->type > LX_W_NVFP4)
    return kNotSupported;
  if (math != LX_MATH_BF16) return kNotSupported;
  if (I % 8 != 0 || L % 8 != 0) return kNotSupported;
  if (gate_up->type == LX_W_NVFP4 && (L % 16 != 0 || I % 16 != 0)) return kInvalid;
  const int P = T * top_k;
  const Layout l = layout(P, E, L, I);
  if (experts_tc_workspace(l.total, P, E, L, I) > kStaticScratchBytes - kStaticHeaderBytes) return LX_B200_ERR_SCRATCH;  // larger than the fixed array
  uint8_t* base = nullptr;
  if (int e = static_scratch(&base)) return e;
  auto s = static_cast<cudaStream_t>(stream);
  uint8_t* ws = base + kStaticHeaderBytes;
  const ExpertChunkTables chunks = experts_tc_ok(*gate_up, *down, L, I) ? expert_chunk_tables(ws, l.total, P, E, L, I) : ExpertChunkTables{};
  if (int e = launch_group(ids, P, E, reinterpret_cast<int32_t*>(ws + l.offsets), reinterpret_cast<int32_t*>(ws + l.pairs), chunks, 0, E, s))
    return e;
  return run_experts(latent, ids, weights, *gate_up, *down, out, ws, l, false, E, E, T, L, I, top_k, s,
                     reinterpret_cast<int*>(base));
}
