// The two grouped products of the routed experts on the 5th-generation tensor cores: gate/up with SwiGLU, then down.
//
// After the pairs (token, pick) have been sorted by expert, an expert's rows are cut into CHUNKS of up to 16 rows (the
// grouping kernel writes the chunk tables with its own). A
// tile is one chunk x R weight rows of its expert x all of K: the weight tile is the A operand of tcgen05.mma exactly
// as it lands in shared memory (128-byte-swizzled 2-D TMA boxes addressed in the stack [E, N, K]), the chunk's rows are
// the B operand as digit columns (BF16: bf16; FP8: two e4m3 digits; INT8: three int8 digits), prepared once per stage
// by a small kernel that also gathers the rows (the latent row of the pair's token, or the pair's intermediate row).
// The tiles of the call, n_chunks x tiles per expert, known only on the device, are dealt to the CTAs in equal
// contiguous ranges, so the work is spread over all SMs whatever the routing was (an expert nobody picked has no
// chunk, an expert with 40 rows has three and streams its weights three times).
//
//   gate/up: a tile is R gate rows and the R up rows of the same indices: two products per K step into two accumulators
//            in tensor memory, so that thread r of the epilogue holds gate[i] and up[i] for the same i and writes
//            mid = bf16(silu(gate) * up) without any exchange.
//   down:    a tile is R rows of down[e]; the epilogue multiplies by the pair's routing weight and writes the pair's
//            f32 row; the k-ordered sum over a token's picks is a kernel of its own (moe.cu).
//
// Roles, rings, bounded waits and the two accumulators in tensor memory are those of the dense kernel (gemm_tc.cu).
// Here every role waits for the previous kernel first: which weights a CTA streams depends on the routing.
#include "tc.cuh"

namespace b200 {
namespace {

constexpr int kChunkRows = kExpertChunkRows;  // rows of one expert a tile multiplies at once
constexpr int kExpertThreads = 192;  // warps 0-3 epilogue, warp 4 producers, warp 5 MMA issuer
constexpr int kDBuf = 256;           // two accumulator sets, 256 TMEM columns apart

struct ExpertTables {
  const int* n_chunks;      // how many chunks this call has
  const int* chunk_expert;  // per chunk: its expert,
  const int* chunk_row0;    //   the sorted position of its first row,
  const int* chunk_rows;    //   and how many rows (1..16)
  const int* pairs;         // sorted position -> pair index t * top_k + k
};

struct ExpertParams {
  ExpertTables tab;
  const uint8_t* scale;        // f32 per weight row of the stack (INT8 / FP8)
  int rows_per_expert;         // 2 I (gate/up) or L (down)
  int out_rows;                // rows a tile's index runs over: I (gate/up) or L (down)
  int K;
  int R, box_bytes, tiles_per_expert;
  int NC, planes;
  float digit;
  const uint8_t* xprep;        // per chunk: n_stages blocks of x_bytes
  int x_bytes;
  int64_t chunk_stride;
  const float* inv_scales;     // per sorted position
  uint16_t* mid;               // gate/up: bf16 [P, I] by sorted position
  float* rows;                 // down: f32 [P, L] by pair index
  const float* route_w;        // down: the pair's routing weight
  int* status;
  int SW, SX;
};

// ---- activation blocks of the chunks -----------------------------------------------------------------------------------
// Block (k piece, sorted position u): as tc_prep_kernel, but the row is gathered (src row = pairs[u] / top_k for the
// latent, u itself for the intermediate rows) and goes to column pos_col[u] of its chunk's blocks.
// QUANT: one plane of per-row quantized values (the low-precision maths) instead of exact digits.
template <int ACT, bool QUANT = false>
__global__ void __launch_bounds__(128) expert_prep_kernel(const uint16_t* __restrict__ src, int ld, int top_k_or_0, int K, int NC,
                                                          const int32_t* __restrict__ pairs, const int32_t* __restrict__ pos_chunk,
                                                          const int32_t* __restrict__ pos_col, uint8_t* __restrict__ out, int64_t chunk_stride,
                                                          float* __restrict__ inv_scales, int n_stages) {
  constexpr int kElem = act_elem(ACT), V = 16 / kElem, kKS = ks_of(ACT);
  pdl_trigger();
  pdl_wait();
  __shared__ float part[4];
  const int u = blockIdx.y, tid = threadIdx.x;
  if (pos_chunk[u] < 0) return;  // a row of an expert another rank owns (the whole block leaves together)
  const int k0 = (blockIdx.x * 128 + tid) * V;
  const bool in_range = k0 < n_stages * kKS;
  const int64_t row = static_cast<int64_t>(top_k_or_0 ? pairs[u] / top_k_or_0 : u) * ld;
  const bool aligned16 = (reinterpret_cast<uintptr_t>(src) & 15) == 0 && ld % 8 == 0;
  float v[V];
  if (in_range) load_values<true, V>(src, row, k0, K, aligned16, v);
  float sc = 1.0f, back = 1.0f;
  if constexpr (ACT != kActBf16) {
    float a = warp_max(row_max_share<true>(src, row, K, aligned16, tid, 128));
    if ((tid & 31) == 0) part[tid >> 5] = a;
    __syncthreads();
    a = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
    if constexpr (QUANT) {
      quant_scales<ACT>(a, sc, back);
    } else {
      sc = scale_of<ACT>(a);
      back = 1.0f / sc;
    }
  }
  if (blockIdx.x == 0 && tid == 0) inv_scales[u] = back;
  if (!in_range) return;
  uint32_t w[3][4];
  if constexpr (QUANT) quantize_plane<ACT>(v, sc, w[0]);
  else make_planes<ACT, true, V>(v, sc, w);
  uint8_t* block = out + pos_chunk[u] * chunk_stride + static_cast<size_t>(k0 / kKS) * (static_cast<size_t>(NC) * kKS * kElem);
  const int kb = (k0 % kKS) * kElem, col = pos_col[u];
  constexpr int planes = QUANT ? 1 : ACT == kActS8 ? 3 : ACT == kActE4m3 ? 2 : 1;
#pragma unroll
  for (int j = 0; j < planes; ++j)
    *reinterpret_cast<uint4*>(block + block_offset(NC, kb, j * kChunkRows + col)) = make_uint4(w[j][0], w[j][1], w[j][2], w[j][3]);
}

// ---- the product kernel ------------------------------------------------------------------------------------------------
enum { kGateUpStage = 0, kDownStage = 1 };

template <int F, int MODE>
__global__ void __launch_bounds__(kExpertThreads, 1) tc_expert_kernel(const __grid_constant__ CUtensorMap wmap, const ExpertParams P) {
  using Fm = TcFmt<F>;
  constexpr int kAct = Fm::kAct, kKS = ks_of(kAct);
  constexpr int kBoxes = Fm::kRowBytes / 128;      // 128-byte-wide tile copies per stage and operand
  constexpr int kSets = MODE == kGateUpStage ? 2 : 1;  // weight tiles per stage: gate and up, or one
  extern __shared__ __align__(1024) uint8_t smem[];
  const int NC = P.NC, SW = P.SW, SX = P.SX;
  const int x_bytes = P.x_bytes, box_bytes = P.box_bytes;
  const int set_bytes = kBoxes * box_bytes, w_stage = kSets * set_bytes;
  uint8_t* const xring = smem + static_cast<size_t>(SW) * w_stage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(xring + static_cast<size_t>(SX) * x_bytes);
  const uint32_t bar0 = smem_u32(bars);
  auto w_full = [&](int s) { return bar0 + 8u * s; };
  auto w_empty = [&](int s) { return bar0 + 8u * (SW + s); };
  auto x_full = [&](int s) { return bar0 + 8u * (2 * SW + s); };
  auto x_empty = [&](int s) { return bar0 + 8u * (2 * SW + SX + s); };
  auto d_full = [&](int b) { return bar0 + 8u * (2 * SW + 2 * SX + b); };
  auto d_empty = [&](int b) { return bar0 + 8u * (2 * SW + 2 * SX + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SW + 2 * SX + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_stages = (P.K + kKS - 1) / kKS;

  if (tid == 0) {
    for (int s = 0; s < SW; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), 1);
    }
    for (int s = 0; s < SX; ++s) {
      mbar_init(x_full(s), 1);
      mbar_init(x_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(d_full(b), 1);
      mbar_init(d_empty(b), 4);
    }
    mbar_init_fence();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(tmem_slot), kTmemColumns);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4 && lane == 0) pdl_trigger();
  // The chunk table, the activation blocks and their scales all come from earlier kernels of this call.
  pdl_wait();
  const int n_tiles = *P.tab.n_chunks * P.tiles_per_expert;
  const int tile_begin = static_cast<int>(static_cast<int64_t>(n_tiles) * blockIdx.x / gridDim.x);
  const int tile_end = static_cast<int>(static_cast<int64_t>(n_tiles) * (blockIdx.x + 1) / gridDim.x);

  if (warp == 4) {
    // ================================ producers ================================
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
      Ring w;
      bool ok = true, wrapped = false;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        const int chunk = tile / P.tiles_per_expert, tt = tile - chunk * P.tiles_per_expert;
        const int y0 = P.tab.chunk_expert[chunk] * P.rows_per_expert + tt * P.R;  // first weight row of the tile in the stack
        for (int s = 0; s < n_stages; ++s) {
          if (wrapped && !tc_wait(w_empty(w.slot), w.lap ^ 1u, P.status)) {
            ok = false;
            break;
          }
          const uint32_t dst = smem_u32(smem) + static_cast<uint32_t>(w.slot) * w_stage;
          mbar_arrive_expect_tx(w_full(w.slot), kSets * kBoxes * P.R * 128);
#pragma unroll
          for (int set = 0; set < kSets; ++set)
#pragma unroll
            for (int b = 0; b < kBoxes; ++b)
              tile_g2s(dst + set * set_bytes + b * box_bytes, &wmap, (s * Fm::kRowBytes + b * 128) / 4, y0 + set * P.out_rows, w_full(w.slot));
          w.advance(SW);
          wrapped |= w.slot == 0;
        }
      }
    } else if (lane == 1) {
      Ring x;
      bool ok = true, wrapped = false;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        const uint8_t* blocks = P.xprep + (tile / P.tiles_per_expert) * P.chunk_stride;
        for (int s = 0; s < n_stages; ++s) {
          if (wrapped && !tc_wait(x_empty(x.slot), x.lap ^ 1u, P.status)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(x_full(x.slot), x_bytes);
          bulk_g2s(smem_u32(xring) + static_cast<uint32_t>(x.slot) * x_bytes, blocks + static_cast<size_t>(s) * x_bytes, x_bytes, x_full(x.slot));
          x.advance(SX);
          wrapped |= x.slot == 0;
        }
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t cfmt = kAct == kActS8 ? 2u : 1u, abfmt = kAct == kActE4m3 ? 0u : 1u;
      const uint32_t idesc = (cfmt << 4) | (abfmt << 7) | (abfmt << 10) | (static_cast<uint32_t>(NC >> 3) << 17) |
                             (static_cast<uint32_t>(kBM >> 4) << 24);
      const uint32_t lbo = static_cast<uint32_t>(NC / 8) * 128, sbo = 128;
      Ring w, x;
      bool ok = true;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        const int t = tile - tile_begin, buf = t & 1;
        const uint32_t d_tmem = tmem_base + buf * kDBuf;
        if (t >= 2) {
          if (!tc_wait(d_empty(buf), ((t >> 1) - 1) & 1, P.status)) break;
          tc_fence_after();
        }
        for (int s = 0; s < n_stages; ++s) {
          if (!tc_wait(w_full(w.slot), w.lap, P.status) || !tc_wait(x_full(x.slot), x.lap, P.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t wb = smem_u32(smem) + static_cast<uint32_t>(w.slot) * w_stage;
          const uint32_t xb = smem_u32(xring) + static_cast<uint32_t>(x.slot) * x_bytes;
#pragma unroll
          for (int b = 0; b < kBoxes; ++b) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const int c = b * 4 + ks;  // 32 bytes of K per instruction
              const uint64_t bdesc = smem_desc(xb + static_cast<uint32_t>(2 * c) * lbo, lbo, sbo);
#pragma unroll
              for (int set = 0; set < kSets; ++set)
                umma_ss<kAct>(d_tmem + set * NC, smem_desc_sw128(wb + set * set_bytes + b * box_bytes + ks * 32), bdesc, idesc, (s | c) ? 1u : 0u);
            }
          }
          umma_commit(w_empty(w.slot));
          umma_commit(x_empty(x.slot));
          w.advance(SW);
          x.advance(SX);
        }
        if (ok) umma_commit(d_full(buf));
      }
    }
  } else {
    // ================================ epilogue ================================
    const int r = tid;  // row of the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    for (int tile = tile_begin; tile < tile_end; ++tile) {
      const int t = tile - tile_begin, buf = t & 1;
      const int chunk = tile / P.tiles_per_expert, tt = tile - chunk * P.tiles_per_expert;
      const int e = P.tab.chunk_expert[chunk], row0 = P.tab.chunk_row0[chunk], n_rows = P.tab.chunk_rows[chunk];
      const int i = tt * P.R + r;  // the output index inside the expert: 0 .. I - 1 (gate/up) or 0 .. L - 1 (down)
      const bool live = r < P.R && i < P.out_rows;
      float rf0 = 1.0f, rf1 = 1.0f;
      if (live && (F == LX_W_INT8 || F == LX_W_FP8)) {
        const float* sc = reinterpret_cast<const float*>(P.scale) + static_cast<int64_t>(e) * P.rows_per_expert;
        rf0 = sc[i];
        if (MODE == kGateUpStage) rf1 = sc[P.out_rows + i];
      }
      const float inv_mine = lane < n_rows ? P.inv_scales[row0 + lane] : 0.0f;                       // lane l: row l of the chunk
      const float rw_mine = (MODE == kDownStage && lane < n_rows) ? P.route_w[P.tab.pairs[row0 + lane]] : 0.0f;
      const int pair_mine = (MODE == kDownStage && lane < n_rows) ? P.tab.pairs[row0 + lane] : 0;
      if (!tc_wait(d_full(buf), (t >> 1) & 1, P.status)) break;
      tc_fence_after();
      const uint32_t d_addr = lane_addr + buf * kDBuf;
#pragma unroll
      for (int c8 = 0; c8 < kChunkRows / 8; ++c8) {
        uint32_t raw[kSets][3][8];
#pragma unroll
        for (int set = 0; set < kSets; ++set)
#pragma unroll
          for (int p = 0; p < 3; ++p)
            if (p < P.planes) tmem_ld8(d_addr + set * NC + p * kChunkRows + c8 * 8, raw[set][p]);
        tmem_wait_ld();
        if (c8 == kChunkRows / 8 - 1) {  // the accumulators have been read
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(d_empty(buf));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int m = c8 * 8 + j;
          const float inv = __shfl_sync(0xffffffffu, inv_mine, m);
          const float rw = __shfl_sync(0xffffffffu, rw_mine, m);
          const int pair = __shfl_sync(0xffffffffu, pair_mine, m);
          if (!live || m >= n_rows) continue;
          float sum[kSets];
#pragma unroll
          for (int set = 0; set < kSets; ++set) {
            float acc = 0.0f, digit = 1.0f;
#pragma unroll
            for (int p = 0; p < 3; ++p) {
              if (p >= P.planes) break;
              const float v = kAct == kActS8 ? static_cast<float>(static_cast<int>(raw[set][p][j])) : __uint_as_float(raw[set][p][j]);
              acc += v * digit;
              digit *= P.digit;
            }
            sum[set] = acc * inv;
          }
          if constexpr (MODE == kGateUpStage) {
            const float g = rf0 * sum[0], u = rf1 * sum[kSets - 1];
            const float h = g / (1.0f + __expf(-g)) * u;
            P.mid[static_cast<int64_t>(row0 + m) * P.out_rows + i] = static_cast<uint16_t>(f32_to_bf16_bits(h));
          } else {
            P.rows[static_cast<int64_t>(pair) * P.out_rows + i] = rw * (rf0 * sum[0]);
          }
        }
      }
    }
  }
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, kTmemColumns);
}

// Rows per tile for an expert's `out_rows` outputs when about `chunks` chunks are expected: the multiple of 8 between 64
// and r_max (what lets three stages fit in shared memory, at most 128) that leaves the busiest SM the fewest rows.
int expert_tile_rows(int out_rows, int chunks, int sms, int r_max) {
  int best = r_max;
  int64_t best_cost = -1;
  for (int R = r_max; R >= std::min(64, r_max); R -= 8) {
    const int64_t tiles = static_cast<int64_t>(chunks) * ((out_rows + R - 1) / R);
    const int64_t cost = (tiles + sms - 1) / sms * R;
    if (best_cost < 0 || cost < best_cost) best = R, best_cost = cost;
  }
  return std::min(best, std::max(8, (out_rows + 7) / 8 * 8));
}

template <int F, int MODE>
int launch_expert(const lx_weight& w, ExpertParams P, int64_t stack_rows, int chunks_expected, cudaStream_t stream) {
  using Fm = TcFmt<F>;
  constexpr int kBoxes = Fm::kRowBytes / 128, kSets = MODE == kGateUpStage ? 2 : 1;
  const int sms = sm_count();
  if (!sms) return kInvalid;
  constexpr int kBudget = 204 * 1024;
  P.SX = 3;
  const int r_max = std::min(128, (kBudget - P.SX * P.x_bytes) / 3 / (kSets * kBoxes * 128) / 8 * 8);
  if (r_max < 8) return kNotSupported;
  P.R = expert_tile_rows(P.out_rows, chunks_expected, sms, r_max);
  P.tiles_per_expert = (P.out_rows + P.R - 1) / P.R;
  P.box_bytes = (P.R + 7) / 8 * 1024;
  const int w_stage = kSets * kBoxes * P.box_bytes;
  P.SW = std::min(12, (kBudget - P.SX * P.x_bytes) / w_stage);
  if (P.SW < 2) return kNotSupported;
  const size_t smem = std::max<size_t>(static_cast<size_t>(P.SW) * w_stage + std::max(P.SX * P.x_bytes, 16 * 1024) + 1024, 120 * 1024);
  alignas(64) CUtensorMap wmap;
  memset(&wmap, 0, sizeof(wmap));
  const int64_t row_bytes = F == LX_W_BF16 ? 2ll * P.K : P.K;
  if (int e = make_tile_map(&wmap, w.data, row_bytes, stack_rows, 128, P.R, 4, true)) return e;
  if (int e = allow_big_smem<100 + F * 2 + MODE>(tc_expert_kernel<F, MODE>)) return e;
  return launch_kernel(tc_expert_kernel<F, MODE>, dim3(sms), dim3(kExpertThreads), smem, stream, wmap, P);
}

int64_t round256(int64_t v) { return (v + 255) / 256 * 256; }

}  // namespace

// Where the tensor-core path keeps its tables and blocks, behind the `base` bytes of the grouping tables and buffers.
struct ExpertTcLayout {
  int64_t n_chunks, chunk_expert, chunk_row0, chunk_rows, pos_chunk, pos_col, inv, xprep, total;
  int max_chunks;
  ExpertTcLayout(int64_t base, int P, int E, int L, int I) {
    max_chunks = std::min(P, E + P / kChunkRows);
    int64_t o = round256(base);
    auto take = [&](int64_t bytes) {
      const int64_t at = o;
      o = round256(o + bytes);
      return at;
    };
    n_chunks = take(4);
    chunk_expert = take(4ll * max_chunks), chunk_row0 = take(4ll * max_chunks), chunk_rows = take(4ll * max_chunks);
    pos_chunk = take(4ll * P), pos_col = take(4ll * P);
    inv = take(4ll * P);
    // the blocks of one stage at a time (gate/up, then down): the widest columns (int8: 48) and the longer K
    const int64_t stages = (std::max(L, I) + 255) / 256;
    xprep = take(static_cast<int64_t>(max_chunks) * stages * 48 * 256);  // int8: 48 columns x 256 bytes; bf16: 16 x 512
    total = o;
  }
};

int64_t experts_tc_workspace(int64_t base, int P, int E, int L, int I) { return ExpertTcLayout(base, P, E, L, I).total; }

ExpertChunkTables expert_chunk_tables(uint8_t* ws, int64_t base, int P, int E, int L, int I) {
  const ExpertTcLayout lay(base, P, E, L, I);
  return ExpertChunkTables{reinterpret_cast<int32_t*>(ws + lay.n_chunks),  reinterpret_cast<int32_t*>(ws + lay.chunk_expert),
                           reinterpret_cast<int32_t*>(ws + lay.chunk_row0), reinterpret_cast<int32_t*>(ws + lay.chunk_rows),
                           reinterpret_cast<int32_t*>(ws + lay.pos_chunk), reinterpret_cast<int32_t*>(ws + lay.pos_col)};
}

// Can the routed experts run on the tensor-core kernels? Both stacks of the same directly readable format, rows of
// whole 16-byte pieces.
bool experts_tc_ok(const lx_weight& gate_up, const lx_weight& down, int L, int I) {
  if (!tc_enabled() || gate_up.type != down.type) return false;
  if (gate_up.type != LX_W_BF16 && gate_up.type != LX_W_INT8 && gate_up.type != LX_W_FP8) return false;
  const int elem = gate_up.type == LX_W_BF16 ? 2 : 1;
  if ((L * elem) % 16 != 0 || (I * elem) % 16 != 0 || L % 8 != 0 || I % 8 != 0) return false;
  return (reinterpret_cast<uintptr_t>(gate_up.data) & 15) == 0 && (reinterpret_cast<uintptr_t>(down.data) & 15) == 0;
}

// offsets / pairs: the grouping tables (sorted by expert); mid: bf16 [P, I]; rows: f32 [P, L] by pair, both in the
// caller's workspace like `tc_ws`, the region ExpertTcLayout describes.
int experts_tc(const void* latent, const float* weights, const lx_weight& gate_up, const lx_weight& down, const int32_t* offsets,
               const int32_t* pairs, uint16_t* mid, float* rows, uint8_t* ws, int64_t base, int T, int L, int I, int E, int top_k,
               int* status, cudaStream_t stream, bool quantized, int stack_experts) {
  const int P = T * top_k;
  if (stack_experts <= 0) stack_experts = E;  // experts the two stacks hold (a rank's own when the experts are split over ranks)
  const ExpertTcLayout lay(base, P, E, L, I);
  int32_t* n_chunks = reinterpret_cast<int32_t*>(ws + lay.n_chunks);
  int32_t* chunk_expert = reinterpret_cast<int32_t*>(ws + lay.chunk_expert);
  int32_t* chunk_row0 = reinterpret_cast<int32_t*>(ws + lay.chunk_row0);
  int32_t* chunk_rows = reinterpret_cast<int32_t*>(ws + lay.chunk_rows);
  int32_t* pos_chunk = reinterpret_cast<int32_t*>(ws + lay.pos_chunk);
  int32_t* pos_col = reinterpret_cast<int32_t*>(ws + lay.pos_col);
  float* inv = reinterpret_cast<float*>(ws + lay.inv);
  uint8_t* xprep = ws + lay.xprep;
  (void)offsets;  // the chunk tables were written together with the grouping tables (group_kernel)
  const int act = act_of(gate_up.type), elem = act_elem(act), KS = ks_of(act);
  if (quantized && act != kActS8 && act != kActE4m3) return kNotSupported;
  const int planes = quantized ? 1 : act_planes(act, true);
  ExpertParams Pm{};
  Pm.tab = ExpertTables{n_chunks, chunk_expert, chunk_row0, chunk_rows, pairs};
  Pm.planes = planes;
  Pm.digit = act == kActS8 ? 0.0078125f : act == kActE4m3 ? 0.0625f : 1.0f;
  Pm.NC = (planes * kChunkRows + 15) / 16 * 16;
  Pm.x_bytes = Pm.NC * KS * elem;
  Pm.xprep = xprep, Pm.inv_scales = inv;
  Pm.mid = mid, Pm.rows = rows, Pm.route_w = weights;
  Pm.status = status;
  const int chunks_expected = std::min(P, E);
  auto prep = [&](const uint16_t* src, int ld, int gather_top_k, int K, int n_stages) {
    const int per_block = 128 * 16 / elem;
    const dim3 grid((n_stages * KS + per_block - 1) / per_block, P);
    const int64_t stride = static_cast<int64_t>(n_stages) * Pm.x_bytes;
    if (quantized) {
      if (act == kActS8)
        return launch_kernel(expert_prep_kernel<kActS8, true>, grid, dim3(128), 0, stream, src, ld, gather_top_k, K, Pm.NC,
                             static_cast<const int32_t*>(pairs), static_cast<const int32_t*>(pos_chunk), static_cast<const int32_t*>(pos_col),
                             xprep, stride, inv, n_stages);
      return launch_kernel(expert_prep_kernel<kActE4m3, true>, grid, dim3(128), 0, stream, src, ld, gather_top_k, K, Pm.NC,
                           static_cast<const int32_t*>(pairs), static_cast<const int32_t*>(pos_chunk), static_cast<const int32_t*>(pos_col),
                           xprep, stride, inv, n_stages);
    }
    switch (act) {
      case kActBf16:
        return launch_kernel(expert_prep_kernel<kActBf16>, grid, dim3(128), 0, stream, src, ld, gather_top_k, K, Pm.NC,
                             static_cast<const int32_t*>(pairs), static_cast<const int32_t*>(pos_chunk), static_cast<const int32_t*>(pos_col),
                             xprep, stride, inv, n_stages);
      case kActE4m3:
        return launch_kernel(expert_prep_kernel<kActE4m3>, grid, dim3(128), 0, stream, src, ld, gather_top_k, K, Pm.NC,
                             static_cast<const int32_t*>(pairs), static_cast<const int32_t*>(pos_chunk), static_cast<const int32_t*>(pos_col),
                             xprep, stride, inv, n_stages);
      default:
        return launch_kernel(expert_prep_kernel<kActS8>, grid, dim3(128), 0, stream, src, ld, gather_top_k, K, Pm.NC,
                             static_cast<const int32_t*>(pairs), static_cast<const int32_t*>(pos_chunk), static_cast<const int32_t*>(pos_col),
                             xprep, stride, inv, n_stages);
    }
  };
  // ---- gate/up ----
  {
    const int n_stages = (L + KS - 1) / KS;
    if (int e = prep(static_cast<const uint16_t*>(latent), L, top_k, L, n_stages)) return e;
    ExpertParams G = Pm;
    G.scale = static_cast<const uint8_t*>(gate_up.scale);
    G.rows_per_expert = 2 * I, G.out_rows = I, G.K = L;
    G.chunk_stride = static_cast<int64_t>(n_stages) * Pm.x_bytes;
    int e;
    switch (gate_up.type) {
      case LX_W_BF16: e = launch_expert<LX_W_BF16, kGateUpStage>(gate_up, G, static_cast<int64_t>(stack_experts) * 2 * I, chunks_expected, stream); break;
      case LX_W_INT8: e = launch_expert<LX_W_INT8, kGateUpStage>(gate_up, G, static_cast<int64_t>(stack_experts) * 2 * I, chunks_expected, stream); break;
      default: e = launch_expert<LX_W_FP8, kGateUpStage>(gate_up, G, static_cast<int64_t>(stack_experts) * 2 * I, chunks_expected, stream); break;
    }
    if (e) return e;
  }
  // ---- down ----
  {
    const int n_stages = (I + KS - 1) / KS;
    if (int e = prep(mid, I, 0, I, n_stages)) return e;
    ExpertParams D = Pm;
    D.scale = static_cast<const uint8_t*>(down.scale);
    D.rows_per_expert = L, D.out_rows = L, D.K = I;
    D.chunk_stride = static_cast<int64_t>(n_stages) * Pm.x_bytes;
    int e;
    switch (down.type) {
      case LX_W_BF16: e = launch_expert<LX_W_BF16, kDownStage>(down, D, static_cast<int64_t>(stack_experts) * L, chunks_expected, stream); break;
      case LX_W_INT8: e = launch_expert<LX_W_INT8, kDownStage>(down, D, static_cast<int64_t>(stack_experts) * L, chunks_expected, stream); break;
      default: e = launch_expert<LX_W_FP8, kDownStage>(down, D, static_cast<int64_t>(stack_experts) * L, chunks_expected, stream); break;
    }
    if (e) return e;
  }
  return kOk;
}

}  // namespace b200
