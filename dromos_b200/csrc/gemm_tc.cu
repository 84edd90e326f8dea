// The batched-decode product on the 5th-generation tensor cores: y[m, n] = sum_k x[m, k] * w[n, k] for 9..64 activation
// rows per pass, weights streamed once in their stored format.
//
// The weight tile is the A operand of tcgen05.mma (128 weight rows = the 128 lanes of the accumulator in tensor memory),
// the activations are the B operand (one accumulator column per activation row and digit), K advances 32 bytes per
// instruction. An instruction costs the tensor pipe at least ~46 cycles whatever the column count, so what matters is
// instructions per byte of weights, and that decides the math per format:
//
//   BF16   kind::f16, A = the bf16 weights as they land in shared memory (128-byte swizzled TMA boxes, read through a
//          shared-memory descriptor), B = bf16 activations; f32 activations as a high and a low bf16 column.
//   FP8    kind::f8f6f4, A = the e4m3 weights as they land, B = the scaled activations as two (bf16 x) or three (f32 x)
//          e4m3 digits in base 16; the digit columns are recombined in the epilogue.
//   INT8   kind::i8, A = the int8 weights as they land, B = the scaled activations as three int8 digits in base 128;
//          the s32 sums are exact.
//   NVFP4  no kind multiplies e2m1 * e4m3-block-scale weights by wider activations, so eight converter warps expand each
//          stage to f16 in registers (exact) and write it with tcgen05.st into tensor memory as the A operand of
//          kind::f16 (K = 16 per instruction); B = activations as f16 after a per-row power-of-two scaling.
//
// Roles (one CTA per SM): a weight producer thread (2-D TMA tile copies, no multicast, ring of stages with one mbarrier
// each), an activation producer thread (1-D bulk copies of prepared blocks through a second, shallower ring), one MMA
// issuer thread, and the epilogue warps (tcgen05.ld, lane = weight row; row factor, activation scale, bias, alpha /
// beta, store). The direct formats keep two accumulators in tensor memory so that the next tile's products run while
// the epilogue of the last one is still reading.
//
// Work is split by ROWS: a tile is R <= 128 weight rows with R chosen so that the tiles divide evenly among the SMs
// (N = 14336 on 148 SMs: 148 tiles of 97 rows), and a CTA streams its tiles whole, all of K. The tensor core always
// multiplies 128 rows; the lanes past R hold whatever shared memory held and are never read. Every output element
// is thus the work of one CTA: no partial sums, no counters, and the same bits whatever the grid.
//
// Activations are prepared once per call by a small kernel into the caller's workspace, in the K-major core-matrix
// order the B descriptor reads.
//
// Every wait is bounded; a wait that gives up writes a code to the status word and the kernel still frees its TMEM.
#include "tc.cuh"

namespace b200 {
namespace {

struct TcParams {
  const uint8_t* scale;   // f32 [N] (INT8 / FP8); NVFP4 block scales come through the tensor map
  float global;
  int N, K, M;            // M: activation rows of this pass
  int R;                  // weight rows per tile
  int box_bytes;          // shared memory one 128-byte-wide tile copy takes: R rounded up to 8, times 128
  int NC;                 // accumulator columns, a multiple of 16: column j * Mp + m is digit j of row m
  int Mp;                 // M rounded up to 8
  int planes;             // digits (or halves) per activation row
  float digit;            // weight of a plane relative to the one before it
  const uint8_t* xprep;   // prepared activations: n_stages blocks of x_bytes
  int x_bytes;            // NC * 256 * bytes per element
  const float* inv_scales;  // M f32: what each row's sum is multiplied by
  const void* x;          // the activations themselves, for CTAs that prepare their own (up to 8 rows)
  int ld_x;
  const void* bias;
  int bias_dtype;
  void* y;
  int y_dtype, ld_y;
  // All-gather epilogue (peers > 0): the tile's outputs go to column col0 + n of every rank's copy of the whole y
  // (peer-mapped pointers, this rank's own among them) instead of P.y; the last epilogue warp of the whole grid to
  // finish then adds one to every rank's arrival counter.
  void* y_peer[8];
  int* flag_peer[8];
  int* done_local;  // this rank's count of finished epilogue warps (word 1 of its own counter pair)
  int peers;
  int64_t col0;
  float alpha, beta;
  int* status;
  int SW, SX;             // depth of the weight ring and of the activation ring
  int SA, slot_bytes;     // (NVFP4 through shared memory) A slots, and the bytes of a weight slot (box + block scales)
  int tmem_cols, dstride; // TMEM columns the CTA takes (a power of two >= 32) and the distance between its two accumulators
};

// Where the parts of the workspace begin, for a pass of NC columns of the activation math `act` over n_stages stages.
struct TcLayout {
  int64_t scales, total;
  TcLayout(int NC, int act, int64_t n_stages) {
    scales = n_stages * NC * ks_of(act) * act_elem(act);
    total = scales + 256;
  }
};

// Block (chunk, u): 128 threads, each 16 bytes of K of every plane of activation row u. The row's largest magnitude
// is found by every block of the row again (the row is a few KB, from L2), which saves a second kernel. Plane j of
// row u is column j * Mp + u. k past K is written as zero up to the end of the last stage; columns that no row owns
// are never written (their accumulator columns are never read).
// MODE kPrepQuant (int8 / e4m3 only): the low-precision maths of lx_gemm_w. The row is quantized once, as
// lx_quantize_act does (scale = max|x| / 127 or / 448, values rounded to nearest even and clamped; engine/cuda/quant.cu),
// into ONE plane, and the row's sums are multiplied by that scale.
// MODE kPrepRound (f32 activations): every value is rounded to bf16 first and then treated as a bf16 activation, which
// is what lx_gemm_w does with f32 activations under BF16 math (engine/cuda/gemm_w.cu:239-252: "a bf16 copy").
enum { kPrepExact = 0, kPrepQuant = 1, kPrepRound = 2 };
template <int ACT, bool XBF, int MODE = kPrepExact>
__global__ void __launch_bounds__(128) tc_prep_kernel(const void* __restrict__ x, int ld_x, int rows, int K, int NC, int Mp, int planes,
                                                      uint8_t* __restrict__ out, float* __restrict__ inv_scales, int n_stages) {
  constexpr int kElem = act_elem(ACT), V = 16 / kElem, kKS = ks_of(ACT);
  pdl_trigger();
  pdl_wait();  // the kernel before this one may still be reading the workspace
  __shared__ float part[4];
  const int u = blockIdx.y, tid = threadIdx.x;
  const int k0 = (blockIdx.x * 128 + tid) * V;
  const bool in_range = k0 < n_stages * kKS;
  const int64_t row = static_cast<int64_t>(u) * ld_x;
  const bool aligned16 = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ld_x % (XBF ? 8 : 4) == 0;
  // this thread's values first (the loads are in flight while the row's largest magnitude is found)
  constexpr bool QUANT = MODE == kPrepQuant;
  constexpr bool AS_BF16 = XBF || MODE == kPrepRound;  // the values are bf16 by the time they are split
  static_assert(MODE != kPrepRound || !XBF, "only f32 activations are rounded");
  float v[V];
  if (in_range) {
    load_values<XBF, V>(x, row, k0, K, aligned16, v);
    if constexpr (MODE == kPrepRound) {
#pragma unroll
      for (int i = 0; i < V; ++i) v[i] = bf16_bits_to_f32(f32_to_bf16_bits(v[i]));
    }
  }
  float sc = 1.0f, back = 1.0f;
  if constexpr (ACT != kActBf16) {
    float a = warp_max(row_max_share<XBF>(x, row, K, aligned16, tid, 128));
    if ((tid & 31) == 0) part[tid >> 5] = a;
    __syncthreads();
    a = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
    if constexpr (MODE == kPrepRound) a = bf16_bits_to_f32(f32_to_bf16_bits(a));  // rounding is monotonic: the largest rounded value
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
  else make_planes<ACT, AS_BF16, V>(v, sc, w);
  uint8_t* block = out + static_cast<size_t>(k0 / kKS) * (static_cast<size_t>(NC) * kKS * kElem);
  const int kb = (k0 % kKS) * kElem;
  for (int j = 0; j < planes; ++j) *reinterpret_cast<uint4*>(block + block_offset(NC, kb, j * Mp + u)) = make_uint4(w[j][0], w[j][1], w[j][2], w[j][3]);
}

// ---- expanding NVFP4 -------------------------------------------------------------------------------------------------
// 16 e2m1 values (8 bytes) times one e4m3 block scale
__device__ __forceinline__ void expand_nvfp4(uint32_t w0, uint32_t w1, uint32_t scale_byte, uint32_t (&p)[8]) {
  uint32_t s2;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(s2) : "r"(scale_byte & 0xffu));
  const uint32_t s = __byte_perm(s2, s2, 0x1010);
  const uint32_t w[2] = {w0, w1};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t v0, v1, v2, v3;
    asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0; cvt.rn.f16x2.e2m1x2 %1, b1; cvt.rn.f16x2.e2m1x2 %2, b2; cvt.rn.f16x2.e2m1x2 %3, b3; }"
        : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
        : "r"(w[i]));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v0) : "r"(s));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v1) : "r"(s));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v2) : "r"(s));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(v3) : "r"(s));
    p[4 * i] = v0, p[4 * i + 1] = v1, p[4 * i + 2] = v2, p[4 * i + 3] = v3;
  }
}

// ---- the epilogue of a tile ---------------------------------------------------------------------------------------------
template <int kAct, bool kPeers>
__device__ __forceinline__ void combine_and_store(const TcParams& P, const uint32_t (&raw)[3][8], const float (&inv)[8], int m0, int n, float rf,
                                                  float bias) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int m = m0 + j;
    if (m >= P.M) continue;
    float sum = 0.0f, digit = 1.0f;
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      if (p >= P.planes) break;
      const float v = kAct == kActS8 ? static_cast<float>(static_cast<int>(raw[p][j])) : __uint_as_float(raw[p][j]);
      sum += v * digit;
      digit *= P.digit;
    }
    sum *= inv[j];
    float out = P.alpha * (rf * sum + bias);
    const int64_t at = static_cast<int64_t>(m) * P.ld_y + n;
    if constexpr (kPeers) {
      for (int g = 0; g < P.peers; ++g) store_from_f32(P.y_peer[g], P.y_dtype, at + P.col0, out);
      continue;
    }
    if (P.beta != 0.0f) out = fmaf(P.beta, load_f32(P.y, P.y_dtype, at), out);
    store_from_f32(P.y, P.y_dtype, at, out);
  }
}

// What a thread needs for its row of a tile besides the accumulator; loaded before the wait for the accumulator.
struct RowTerms {
  int n;
  bool live;
  float rf, bias;
};
template <int F>
__device__ __forceinline__ RowTerms row_terms(const TcParams& P, int tile, int r) {
  RowTerms t;
  t.n = tile * P.R + r;
  t.live = r < P.R && t.n < P.N;
  t.rf = 1.0f, t.bias = 0.0f;
  if (t.live) {  // the weight's scales and the bias are static, like the weight
    if constexpr (F == LX_W_INT8 || F == LX_W_FP8) t.rf = reinterpret_cast<const float*>(P.scale)[t.n];
    if constexpr (F == LX_W_NVFP4) t.rf = P.global;
    if (P.bias) t.bias = load_f32(P.bias, P.bias_dtype, t.n);
  }
  return t;
}

// The calling thread owns row r of the tile (accumulator lane r, its warp's lane quarter already in d_addr) and the
// 8-row chunks of activations chunk0, chunk0 + chunk_step, ... inv_lo / inv_hi: lane l holds the inverse activation
// scale of rows l and 32 + l. release_bar (0 = none) gets one arrival per warp as soon as the warp has read the
// accumulator.
// kPeers: the all-gather epilogue (stores into every rank's y) instead of the usual one (into P.y).
template <int F, bool kPeers>
__device__ __forceinline__ void finish_tile(const TcParams& P, const RowTerms& T, uint32_t d_addr, int lane, int chunk0, int chunk_step,
                                            float inv_lo, float inv_hi, uint32_t release_bar) {
  constexpr int kAct = TcFmt<F>::kAct;
  const int Mp = P.Mp, chunks = Mp / 8;
  auto release = [&]() {
    tc_fence_before();
    __syncwarp();
    if (release_bar && lane == 0) mbar_arrive(release_bar);
  };
  uint32_t raw[3][8];
  for (int c = chunk0; c < chunks; c += chunk_step) {
#pragma unroll
    for (int p = 0; p < 3; ++p)
      if (p < P.planes) tmem_ld8(d_addr + p * Mp + c * 8, raw[p]);
    float inv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) inv[j] = __shfl_sync(0xffffffffu, c < 4 ? inv_lo : inv_hi, (c * 8 + j) & 31);
    tmem_wait_ld();
    if (c + chunk_step >= chunks) release();
    if (T.live) combine_and_store<kAct, kPeers>(P, raw, inv, c * 8, T.n, T.rf, T.bias);
  }
  if (chunk0 >= chunks) release();
}

// The all-gather epilogue's hand-off. Every epilogue warp, once what it stored to the peers' buffers is visible
// system-wide, counts itself in shared memory; the CTA's last warp counts the CTA on this GPU's own counter; the CTA
// that finds it is the last of the grid puts that counter back to zero and adds ONE arrival to every rank's semaphore.
// (Atomics on one word serialise: a remote atomic per warp, 1184 per product at two ranks, cost more than the product,
// and even 592 local ones showed; now it is 148 local and one remote per rank.) cta_count: a zeroed word of shared memory.
__device__ __forceinline__ void signal_peers(const TcParams& P, int lane, int* cta_count) {
  if (P.peers <= 0) return;
  __threadfence_system();
  __syncwarp();
  if (lane == 0) {
    if (atomicAdd(cta_count, 1) != 3) return;  // not the CTA's last epilogue warp
    __threadfence();
    int before;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(before) : "l"(P.done_local) : "memory");
    if (before == static_cast<int>(gridDim.x) - 1) {
      asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(P.done_local), "r"(0) : "memory");
      __threadfence_system();
      for (int g = 0; g < P.peers; ++g) asm volatile("red.relaxed.sys.global.add.s32 [%0], 1;" ::"l"(P.flag_peer[g]) : "memory");  // ordered by the fence above
    }
  }
}

// Stages of raw activations a CTA that prepares its own keeps in flight (32 bytes per thread and stage for bf16, 64 for f32).
constexpr int own_depth(bool x_bf16) { return x_bf16 ? 1 : 1; }  // iterations (of two stages) per group of preparing warps; there are two groups
constexpr int own_staging_bytes(bool x_bf16) { return 2 * own_depth(x_bf16) * 2 * 128 * 16 * (x_bf16 ? 2 : 4); }  // groups x depth x stages per iteration x threads x unit

// ---- BF16 / FP8 / INT8: weights go from shared memory straight into the tensor core ------------------------------------
constexpr int kDirectThreads = 192;   // warps 0-3 epilogue, warp 4 producers, warp 5 MMA issuer
constexpr int kOwnThreads = 320;      // ... and warps 6-9, the second group that prepares activation blocks

// XMODE 0: activation blocks come prepared from the workspace (bulk copies). XMODE 1 / 2: up to 8 rows of bf16 / f32
// activations, which the CTA's epilogue warps turn into blocks themselves, stage by stage, straight into the ring: no
// preparation kernel, no workspace, one launch.
// PEERS: the epilogue stores into every rank's y and signals (the all-gather epilogue) instead of storing into P.y; its
// own instantiations, so that the usual kernels carry none of it (their code size shows when kernels alternate).
template <int F, int XMODE, bool PEERS>
__global__ void __launch_bounds__(XMODE ? kOwnThreads : kDirectThreads, XMODE ? 1 : 2) tc_direct_kernel(const __grid_constant__ CUtensorMap wmap, const TcParams P) {
  using Fm = TcFmt<F>;
  constexpr int kAct = Fm::kAct, kKS = ks_of(kAct);
  constexpr bool kOwn = XMODE != 0, kXBF = XMODE == 1;
  constexpr int kBoxes = Fm::kRowBytes / 128;    // 128-byte-wide tile copies per stage
  extern __shared__ __align__(1024) uint8_t smem[];
  const int NC = P.NC, SW = P.SW, SX = P.SX;
  const int x_bytes = P.x_bytes, box_bytes = P.box_bytes;
  const int w_stage = kBoxes * box_bytes;        // a multiple of 1024
  // The tensor core reads 128 rows from every box, whatever R is: behind the weight ring come at least 16 KB of this
  // CTA's own shared memory (the activation ring and padding).
  uint8_t* const xring = smem + static_cast<size_t>(SW) * w_stage;
  // (kOwn) behind the activation ring: the threads' private pieces for raw activations in flight
  uint64_t* bars = reinterpret_cast<uint64_t*>(xring + static_cast<size_t>(SX) * x_bytes + (kOwn ? own_staging_bytes(kXBF) : 0));
  const uint32_t bar0 = smem_u32(bars);
  auto w_full = [&](int s) { return bar0 + 8u * s; };                     // weight stage landed
  auto w_empty = [&](int s) { return bar0 + 8u * (SW + s); };             // its products are done
  // CTAs that prepare their own blocks into a ring of the weights' depth count them on the weights' barrier: the issuer
  // waits once per stage
  const bool one_full = kOwn && SW == SX;
  auto x_full = [&](int s) { return one_full ? w_full(s) : bar0 + 8u * (2 * SW + s); };  // activation block landed
  auto x_empty = [&](int s) { return SW == SX ? w_empty(s) : bar0 + 8u * (2 * SW + SX + s); };  // its products are done (rings of one depth share the weights' barrier)
  auto d_full = [&](int b) { return bar0 + 8u * (2 * SW + 2 * SX + b); };       // accumulator b is complete
  auto d_empty = [&](int b) { return bar0 + 8u * (2 * SW + 2 * SX + 2 + b); };  // accumulator b has been read
  const uint32_t group_bar = bar0 + 8u * (2 * SW + 2 * SX + 4);           // the epilogue warps meet here
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SW + 2 * SX + 5);
  int* cta_count = reinterpret_cast<int*>(tmem_slot + 1);                  // (PEERS) epilogue warps of this CTA that are done
  float* row_scale = reinterpret_cast<float*>(tmem_slot + 2);             // (kOwn) at 16 + 8 w + m: warp w's share of row m's largest magnitude

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_stages = (P.K + kKS - 1) / kKS;
  const int n_tiles = (P.N + P.R - 1) / P.R;
  const int tile_begin = static_cast<int>(static_cast<int64_t>(n_tiles) * blockIdx.x / gridDim.x);
  const int tile_end = static_cast<int>(static_cast<int64_t>(n_tiles) * (blockIdx.x + 1) / gridDim.x);

  if (tid == 0) {
    for (int s = 0; s < SW; ++s) {
      mbar_init(w_full(s), one_full ? 5 : 1);  // the tile copies' bytes (and the four preparing warps)
      mbar_init(w_empty(s), 1);
    }
    for (int s = 0; s < SX; ++s) {
      if (!one_full) mbar_init(x_full(s), kOwn ? 4 : 1);  // the four preparing warps, or the bulk copy's bytes
      if (SW != SX) mbar_init(x_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(d_full(b), 1);
      mbar_init(d_empty(b), 4);
    }
    mbar_init(group_bar, kOwn ? 8 : 4);
    *cta_count = 0;
    mbar_init_fence();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(tmem_slot), P.tmem_cols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ================================ producers ================================
    pdl_trigger();
    const int total = (tile_end - tile_begin) * n_stages;
    if (lane == 0) {
      // Weights are static (nothing earlier in the stream is still writing them: the contract of the reference's
      // kernels, which also load them before their wait), so they stream while the preparation kernel still runs.
      asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
      Ring w;
      bool ok = true, wrapped = false;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        for (int s = 0; s < n_stages; ++s) {
          if (wrapped && !tc_wait(w_empty(w.slot), w.lap ^ 1u, P.status)) {
            ok = false;
            break;
          }
          const uint32_t dst = smem_u32(smem) + static_cast<uint32_t>(w.slot) * w_stage;
          mbar_arrive_expect_tx(w_full(w.slot), kBoxes * P.R * 128);
#pragma unroll
          for (int b = 0; b < kBoxes; ++b)
            tile_g2s(dst + b * box_bytes, &wmap, (s * Fm::kRowBytes + b * 128) / 4, tile * P.R, w_full(w.slot));
          w.advance(SW);
          wrapped |= w.slot == 0;
        }
      }
    } else if (lane == 1 && !kOwn) {
      pdl_wait();  // the prepared activations come from the kernel before this one
      Ring x;
      bool wrapped = false;
      int s = 0;
      for (int i = 0; i < total; ++i) {
        if (wrapped && !tc_wait(x_empty(x.slot), x.lap ^ 1u, P.status)) break;
        mbar_arrive_expect_tx(x_full(x.slot), x_bytes);
        bulk_g2s(smem_u32(xring) + static_cast<uint32_t>(x.slot) * x_bytes, P.xprep + static_cast<size_t>(s) * x_bytes, x_bytes, x_full(x.slot));
        x.advance(SX);
        wrapped |= x.slot == 0;
        if (++s == n_stages) s = 0;
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      // c format (f32 = 1, s32 = 2), a / b format (bf16 = 1 in kind::f16, e4m3 = 0 in kind::f8f6f4, signed = 1 in
      // kind::i8), both operands K-major, N / 8, M / 16
      const uint32_t cfmt = kAct == kActS8 ? 2u : 1u, abfmt = kAct == kActE4m3 ? 0u : 1u;
      const uint32_t idesc = (cfmt << 4) | (abfmt << 7) | (abfmt << 10) | (static_cast<uint32_t>(NC >> 3) << 17) |
                             (static_cast<uint32_t>(kBM >> 4) << 24);
      const uint32_t lbo = static_cast<uint32_t>(NC / 8) * 128, sbo = 128;
      // the descriptors' halves (smem_desc_sw128 / smem_desc): the high words never change, the low words carry the address
      const uint32_t a_hi = (1024u >> 4) | (1u << 14) | (2u << 29), b_hi = (sbo >> 4) | (1u << 14);
      const uint32_t a_lo0 = ((smem_u32(smem) & 0x3ffffu) >> 4) | (1u << 16);
      const uint32_t b_lo0 = ((smem_u32(xring) & 0x3ffffu) >> 4) | ((lbo >> 4) << 16);
      const uint32_t w_stage16 = static_cast<uint32_t>(w_stage) >> 4, x_bytes16 = static_cast<uint32_t>(x_bytes) >> 4;
      const uint32_t box16 = static_cast<uint32_t>(box_bytes) >> 4, b_step = (2u * lbo) >> 4;
      const bool one_ring = SW == SX;  // one barrier per stage frees both the weights and the activation block
      Ring w, x;
      bool ok = true;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        const int t = tile - tile_begin, buf = t & 1;
        const uint32_t d_tmem = tmem_base + buf * P.dstride;
        if (t >= 2) {  // the epilogue of the tile before last has read this accumulator
          if (!tc_wait(d_empty(buf), ((t >> 1) - 1) & 1, P.status)) break;
          tc_fence_after();
        }
        for (int s = 0; s < n_stages; ++s) {
          if (!tc_wait(w_full(w.slot), w.lap, P.status) || (!one_full && !tc_wait(x_full(x.slot), x.lap, P.status))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(w.slot) * w_stage16;
          const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(x.slot) * x_bytes16;
#pragma unroll
          for (int b = 0; b < kBoxes; ++b) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const int c = b * 4 + ks;  // 32 bytes of K per instruction
              umma_ss_halves<kAct>(d_tmem, a_lo + b * box16 + ks * 2, a_hi, b_lo + c * b_step, b_hi, idesc, c ? 1u : (s ? 1u : 0u));
            }
          }
          umma_commit(w_empty(w.slot));
          if (!one_ring) umma_commit(x_empty(x.slot));
          w.advance(SW);
          x.advance(SX);
        }
        if (ok) umma_commit(d_full(buf));
      }
    }
  } else {
    // ================================ epilogue (and, if kOwn, the activation blocks) ================================
    // kOwn: two groups of four warps (0-3 and 6-9) prepare the activation blocks of alternate stages; the first group
    // also runs the epilogue, its thread r owning accumulator lane r.
    const int group = warp >= 6 ? 1 : 0;
    const int gtid = group ? tid - 192 : tid, gwarp = gtid >> 5;
    const int r = gtid;  // weight row of the tile = TMEM lane (group 0)
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(gwarp * 32) << 16);
    pdl_wait();  // the activations (or their prepared form) and y come from earlier kernels
    if constexpr (!kOwn) {
      const float inv_lo = lane < P.M ? P.inv_scales[lane] : 0.0f, inv_hi = 32 + lane < P.M ? P.inv_scales[32 + lane] : 0.0f;
      for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int t = tile - tile_begin, buf = t & 1;
        const RowTerms T = row_terms<F>(P, tile, r);
        if (!tc_wait(d_full(buf), (t >> 1) & 1, P.status)) break;
        tc_fence_after();
        finish_tile<F, PEERS>(P, T, lane_addr + buf * P.dstride, lane, 0, 1, inv_lo, inv_hi, d_empty(buf));
      }
      if constexpr (PEERS) signal_peers(P, lane, cta_count);  // (a CTA whose wait gave up still counts itself: nobody hangs, the status word tells)
    } else {
      static_assert(act_elem(kAct) == 1, "CTAs prepare their own activations for the 8-bit maths only");
      constexpr int V = 16;
      constexpr int kPiece = kXBF ? 8 : 4;  // activations per 16 bytes
      constexpr int kUnitBytes = V * (kXBF ? 2 : 4);
      constexpr int D = own_depth(kXBF);
      const bool aligned16 = (reinterpret_cast<uintptr_t>(P.x) & 15) == 0 && P.ld_x % kPiece == 0;
      bool ok = true;
      // Thread (m = gtid % 8, kg = gtid / 8) owns, in each of its group's stages, the 16 values k = 16 kg .. 16 kg + 15
      // of activation row m: 16 bytes of each plane. Its raw activations travel from global memory into a private piece
      // of shared memory with cp.async, D iterations ahead. A group takes two consecutive stages per iteration (group 0:
      // stages 0, 1, 4, 5, ...; group 1: 2, 3, 6, 7, ...): the fixed cost of an iteration (about a microsecond of waits,
      // proxy fence and arrivals, measured) is paid once for both.
      constexpr int B = 2;
      const int m = gtid & 7, kg = gtid >> 3;
      const bool row_live = m < P.M;
      const uint8_t* xrow = static_cast<const uint8_t*>(P.x) + static_cast<int64_t>(m) * P.ld_x * (kXBF ? 2 : 4);
      uint8_t* const staging = xring + static_cast<size_t>(SX) * x_bytes + static_cast<size_t>(group) * D * B * 128 * kUnitBytes;
      const int row_bytes = P.K * (kXBF ? 2 : 4);
      // stage s of a tile (or nothing, s < 0) into piece b of staging slot d
      auto fetch = [&](int s, int d, int b) {
        if (!row_live || s < 0) return;
        uint8_t* dst = staging + ((static_cast<size_t>(d) * B + b) * 128 + gtid) * kUnitBytes;
        const int k0 = s * kKS + kg * V;
        const int at = k0 * (kXBF ? 2 : 4);  // byte offset of the unit in its row
        if (aligned16) {
#pragma unroll
          for (int q = 0; q < kUnitBytes / 16; ++q) {
            const int left = min(16, max(0, row_bytes - (at + 16 * q)));  // bytes of the row in this piece; the rest reads as zero
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst + 16 * q)), "l"(xrow + (left ? at + 16 * q : 0)),
                         "r"(left)
                         : "memory");
          }
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) {
            if constexpr (kXBF) reinterpret_cast<uint16_t*>(dst)[i] = k0 + i < P.K ? reinterpret_cast<const uint16_t*>(xrow)[k0 + i] : uint16_t(0);
            else reinterpret_cast<float*>(dst)[i] = k0 + i < P.K ? reinterpret_cast<const float*>(xrow)[k0 + i] : 0.0f;
          }
        }
      };
      const int total = (tile_end - tile_begin) * n_stages;
      // The next stages to fetch: CTA stage ahead_i (and ahead_i + 1), which is stage ahead_s of its tile.
      int ahead_i = B * group, ahead_s = (B * group) % n_stages;
      auto issue = [&](int d) {  // always one cp.async group
#pragma unroll
        for (int b = 0; b < B; ++b) {
          int sb = ahead_s + b;
          if (sb >= n_stages) sb -= n_stages;
          fetch(ahead_i + b < total ? sb : -1, d, b);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        ahead_i += 2 * B;
        ahead_s += 2 * B;
        while (ahead_s >= n_stages) ahead_s -= n_stages;
      };
      // the first fetches go out before the row maxima are known: they do not depend on them
      for (int d = 0; d < D; ++d) issue(d);
      // ---- first pass: the largest magnitude of every row, by all 256 preparing threads ----
      {
        const int t256 = group * 128 + gtid;
        float a[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) a[m] = 0.0f;
        if (aligned16) {
          const int pieces = P.K / kPiece;  // whole 16-byte pieces per row
          for (int p0 = t256; p0 < pieces; p0 += 512) {
            uint4 q[2][8];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int m = 0; m < 8; ++m) {
                q[h][m] = make_uint4(0, 0, 0, 0);
                const int p = p0 + 256 * h;
                if (m < P.M && p < pieces)
                  q[h][m] = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(P.x) +
                                                            (static_cast<int64_t>(m) * P.ld_x + static_cast<int64_t>(p) * kPiece) * (kXBF ? 2 : 4));
              }
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int m = 0; m < 8; ++m) {
                const uint32_t w[4] = {q[h][m].x, q[h][m].y, q[h][m].z, q[h][m].w};
#pragma unroll
                for (int z = 0; z < 4; ++z) {
                  if constexpr (kXBF) a[m] = fmaxf(a[m], fmaxf(fabsf(__uint_as_float(w[z] << 16)), fabsf(__uint_as_float(w[z] & 0xffff0000u))));
                  else a[m] = fmaxf(a[m], fabsf(__uint_as_float(w[z])));
                }
              }
          }
          for (int m = 0; m < P.M; ++m)
            for (int k = pieces * kPiece + t256; k < P.K; k += 256)
              a[m] = fmaxf(a[m], fabsf(load_f32(P.x, kXBF ? LX_BF16 : LX_F32, static_cast<int64_t>(m) * P.ld_x + k)));
        } else {
          for (int m = 0; m < P.M; ++m)
            for (int k = t256; k < P.K; k += 256)
              a[m] = fmaxf(a[m], fabsf(load_f32(P.x, kXBF ? LX_BF16 : LX_F32, static_cast<int64_t>(m) * P.ld_x + k)));
        }
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const float v = warp_max(a[m]);
          if (lane == 0) row_scale[(group * 4 + gwarp) * 8 + m] = v;  // this warp's share of row m
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(group_bar);
        ok = tc_wait(group_bar, 0, P.status);
      }
      auto row_scale_of = [&](int row) {
        float v = 0.0f;
#pragma unroll
        for (int w8 = 0; w8 < 8; ++w8) v = fmaxf(v, row_scale[w8 * 8 + row]);
        return scale_of<kAct>(v);
      };
      // ---- second pass: the digits, two stages per iteration into the ring ----
      const float sc = row_live ? row_scale_of(m) : 1.0f;
      const float inv = lane < P.M ? 1.0f / row_scale_of(lane) : 0.0f;  // lane l: row l (finish_tile's layout)
      auto wait_landed = [&]() { asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory"); };
      // piece b of staging slot d as f32 (after wait_landed)
      auto take = [&](int d, int b, float (&v)[V]) {
        const uint8_t* src = staging + ((static_cast<size_t>(d) * B + b) * 128 + gtid) * kUnitBytes;
        if constexpr (kXBF) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const uint4 t = *reinterpret_cast<const uint4*>(src + 16 * q);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int z = 0; z < 4; ++z) {
              v[8 * q + 2 * z] = __uint_as_float(w[z] << 16);
              v[8 * q + 2 * z + 1] = __uint_as_float(w[z] & 0xffff0000u);
            }
          }
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 t = *reinterpret_cast<const float4*>(src + 16 * q);
            v[4 * q] = t.x, v[4 * q + 1] = t.y, v[4 * q + 2] = t.z, v[4 * q + 3] = t.w;
          }
        }
      };
      int next_finish = tile_begin;  // (group 0) the first tile whose accumulator has not been read yet
      auto finish = [&](int tile) {
        const int t = tile - tile_begin, buf = t & 1;
        const RowTerms T = row_terms<F>(P, tile, r);
        if (!tc_wait(d_full(buf), (t >> 1) & 1, P.status)) return false;
        tc_fence_after();
        finish_tile<F, PEERS>(P, T, lane_addr + buf * P.dstride, lane, 0, 1, inv, 0.0f, d_empty(buf));
        return true;
      };
      Ring x[B];
#pragma unroll
      for (int b = 0; b < B; ++b)
        for (int a = 0; a < B * group + b; ++a) x[b].advance(SX);
      int d = 0, tile = tile_begin, s = B * group;  // the iteration's first stage: stage s of `tile`
      while (s >= n_stages) s -= n_stages, ++tile;
      for (int i = B * group; ok; i += 2 * B) {
        const bool draining = i >= total;  // past the last stage: group 0 reads the accumulators that are left
        if (group == 0) {
          // The products of a stage's tile need the accumulator of the tile two before it: that one must have been
          // read by now (the iteration's second stage may already belong to the next tile). The one before, as soon as
          // it happens to be complete. (One call site: the epilogue is 9 KB of code, and code size shows whenever the
          // stream alternates between kernels.)
          const int tile_hi = s + 1 >= n_stages ? tile + 1 : tile;
          for (;;) {
            const bool must = draining ? next_finish < tile_end : next_finish <= tile_hi - 2;
            bool go = must;
            if (!go && !draining && next_finish < tile)
              go = mbar_try_wait(d_full((next_finish - tile_begin) & 1), ((next_finish - tile_begin) >> 1) & 1);
            if (!go) break;
            ok = finish(next_finish++);
            if (!ok || !must) break;
          }
          if (!ok) break;
        }
        if (draining) break;
        wait_landed();  // the oldest group in flight, this iteration's
        uint32_t w[B][3][4];
#pragma unroll
        for (int b = 0; b < B; ++b) {
          float v[V];
          take(d, b, v);
          make_planes<kAct, kXBF, V>(v, sc, w[b]);
        }
        issue(d);
        if (++d == D) d = 0;
#pragma unroll
        for (int b = 0; b < B; ++b) {
          if (i + b >= total) break;
          if (i + b >= SX && !tc_wait(x_empty(x[b].slot), x[b].lap ^ 1u, P.status)) {
            ok = false;
            break;
          }
          uint8_t* block = xring + static_cast<size_t>(x[b].slot) * x_bytes;
          if (row_live) {
#pragma unroll
            for (int j = 0; j < 3; ++j)
              if (j < P.planes)
                *reinterpret_cast<uint4*>(block + block_offset(NC, kg * 16, j * P.Mp + m)) = make_uint4(w[b][j][0], w[b][j][1], w[b][j][2], w[b][j][3]);
          }
        }
        if (!ok) break;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads what these threads wrote
        __syncwarp();
#pragma unroll
        for (int b = 0; b < B; ++b) {
          if (lane == 0 && i + b < total) mbar_arrive(x_full(x[b].slot));
#pragma unroll
          for (int a = 0; a < 2 * B; ++a) x[b].advance(SX);
        }
        s += 2 * B;
        while (s >= n_stages) s -= n_stages, ++tile;
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      if (group == 0) {
        if constexpr (PEERS) signal_peers(P, lane, cta_count);
      }
    }
  }
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, P.tmem_cols);
}

// ---- NVFP4: converter warps expand the stage into tensor memory ---------------------------------------------------------
constexpr int kKS4 = ks_of(kActF16);  // values of K per stage
constexpr int kChunks = kKS4 / 16;   // tcgen05.mma instructions per stage (K = 16 each)
constexpr int kASlots = 3;           // A-operand slots in TMEM, one stage each (kKS4 / 2 columns)
constexpr int kAColumns = kKS4 / 2;
constexpr int kDColumn = kASlots * kAColumns;  // the accumulator's first TMEM column (128 columns remain for it)
// Eight or sixteen converter warps (kConvWarps = 8 or 16) were both measured on the 28672 x 8192 matrix: 76.9 / 82.2 us
// at M = 16 / 64 with eight, 80.1 / 86.2 us with sixteen, so the converters' instruction stream is not what bounds a stage
// (ncu: 30 % of issue slots, tensor pipe 6 %). A stage writes 64 KB of f16 into tensor memory for 16 KB of weights, and
// 2375 cycles per stage is 27 bytes per cycle and SM of tcgen05.st.
constexpr int kConvWarps = 8, kConvParts = kConvWarps / 4;  // a part: the share of a stage's K one converter thread expands for its row
constexpr int kConvPieces = 8 / kConvParts;                  // 16-byte pieces (32 values, two block scales) per thread and stage
constexpr int kProducerWarp = kConvWarps, kIssuerWarp = kConvWarps + 1;
constexpr int kConvThreads = (kConvWarps + 2) * 32;  // converter warps, then the producer warp, then the MMA issuer

__global__ void __launch_bounds__(kConvThreads, 1)
    tc_nvfp4_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap, const TcParams P) {
  constexpr int F = LX_W_NVFP4;
  using Fm = TcFmt<F>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int NC = P.NC, SW = P.SW, SX = P.SX;
  const int x_bytes = P.x_bytes, box_bytes = P.box_bytes;
  // a slot is the stage's box (R rows of 128 bytes, 1024-aligned) and, box_bytes further, its 16 block scales per row
  uint8_t* const xring = smem + static_cast<size_t>(SW) * box_bytes * 2;
  uint64_t* bars = reinterpret_cast<uint64_t*>(xring + static_cast<size_t>(SX) * x_bytes);
  const uint32_t bar0 = smem_u32(bars);
  auto w_full = [&](int s) { return bar0 + 8u * s; };                               // weight stage landed
  auto w_empty = [&](int s) { return bar0 + 8u * (SW + s); };                       // read by all converter warps
  auto x_full = [&](int s) { return bar0 + 8u * (2 * SW + s); };                    // activation block landed
  auto x_empty = [&](int s) { return bar0 + 8u * (2 * SW + SX + s); };              // its products are done
  auto a_full = [&](int a) { return bar0 + 8u * (2 * SW + 2 * SX + a); };           // A slot written
  auto a_empty = [&](int a) { return bar0 + 8u * (2 * SW + 2 * SX + kASlots + a); };// A slot consumed
  const uint32_t d_full = bar0 + 8u * (2 * SW + 2 * SX + 2 * kASlots);              // the tile's accumulator is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SW + 2 * SX + 2 * kASlots + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_stages = (P.K + kKS4 - 1) / kKS4;
  const int n_tiles = (P.N + P.R - 1) / P.R;
  const int tile_begin = static_cast<int>(static_cast<int64_t>(n_tiles) * blockIdx.x / gridDim.x);
  const int tile_end = static_cast<int>(static_cast<int64_t>(n_tiles) * (blockIdx.x + 1) / gridDim.x);
  const int total = (tile_end - tile_begin) * n_stages;
  const int slot_bytes = 2 * box_bytes;

  if (tid == 0) {
    for (int s = 0; s < SW; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), kConvWarps);
    }
    for (int s = 0; s < SX; ++s) {
      mbar_init(x_full(s), 1);
      mbar_init(x_empty(s), 1);
    }
    for (int a = 0; a < kASlots; ++a) {
      mbar_init(a_full(a), kConvWarps);
      mbar_init(a_empty(a), 1);
    }
    mbar_init(d_full, 1);
    mbar_init_fence();
  }
  if (warp == kIssuerWarp) {
    tmem_alloc(smem_u32(tmem_slot), kTmemColumns);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kProducerWarp) {
    // ================================ producers ================================
    pdl_trigger();
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&smap) : "memory");
    }
    if (lane == 0) {  // weights and their scales are static: no wait
      Ring w;
      bool ok = true, wrapped = false;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        for (int s = 0; s < n_stages; ++s) {
          if (wrapped && !tc_wait(w_empty(w.slot), w.lap ^ 1u, P.status)) {
            ok = false;
            break;
          }
          const uint32_t dst = smem_u32(smem) + static_cast<uint32_t>(w.slot) * slot_bytes;
          mbar_arrive_expect_tx(w_full(w.slot), P.R * (128 + 16));
          tile_g2s(dst, &wmap, (s * Fm::kRowBytes) / 4, tile * P.R, w_full(w.slot));
          tile_g2s(dst + box_bytes, &smap, s * 16, tile * P.R, w_full(w.slot));
          w.advance(SW);
          wrapped |= w.slot == 0;
        }
      }
    } else if (lane == 1) {
      pdl_wait();  // the prepared activations come from the kernel before this one
      Ring x;
      bool wrapped = false;
      int s = 0;
      for (int i = 0; i < total; ++i) {
        if (wrapped && !tc_wait(x_empty(x.slot), x.lap ^ 1u, P.status)) break;
        mbar_arrive_expect_tx(x_full(x.slot), x_bytes);
        bulk_g2s(smem_u32(xring) + static_cast<uint32_t>(x.slot) * x_bytes, P.xprep + static_cast<size_t>(s) * x_bytes, x_bytes, x_full(x.slot));
        x.advance(SX);
        wrapped |= x.slot == 0;
        if (++s == n_stages) s = 0;
      }
    }
  } else if (warp == kIssuerWarp) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(NC >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);  // f16 x f16 -> f32
      const uint32_t lbo = static_cast<uint32_t>(NC / 8) * 128, sbo = 128;
      Ring x, a;
      int s = 0;
      for (int i = 0; i < total; ++i) {
        // the activations of this stage are in shared memory, the converted weights in tensor memory
        if (!tc_wait(x_full(x.slot), x.lap, P.status) || !tc_wait(a_full(a.slot), a.lap, P.status)) break;
        tc_fence_after();
        const uint32_t xb = smem_u32(xring) + static_cast<uint32_t>(x.slot) * x_bytes;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          const uint64_t bdesc = smem_desc(xb + static_cast<uint32_t>(2 * c) * lbo, lbo, sbo);
          umma_ts(tmem_base + kDColumn, tmem_base + a.slot * kAColumns + c * 8, bdesc, idesc, (s | c) ? 1u : 0u);
        }
        umma_commit(a_empty(a.slot));    // the A slot may be overwritten once these products are done
        umma_commit(x_empty(x.slot));    // and so may the activation block
        // A tile ends here: its accumulator is complete when everything issued so far is. The next tile's first
        // product overwrites it, but waits for an A slot the converters fill only after they have read the accumulator.
        if (++s == n_stages) {
          s = 0;
          umma_commit(d_full);
        }
        x.advance(SX);
        a.advance(kASlots);
      }
    }
  } else {
    // ================================ converters, then epilogue ================================
    const int quarter = warp & 3, part = warp >> 2;
    const int r = quarter * 32 + lane;  // weight row of the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    Ring w, a;
    int s = 0, t = 0;
    bool a_wrapped = false;
    for (int i = 0; i < total; ++i) {
      if (!tc_wait(w_full(w.slot), w.lap, P.status) || (a_wrapped && !tc_wait(a_empty(a.slot), a.lap ^ 1u, P.status))) break;
      tc_fence_after();
      // Rows past R read what shared memory holds behind the box (this CTA's own, see tc_launch); their lanes are
      // never read back.
      const uint8_t* stage = smem + static_cast<size_t>(w.slot) * slot_bytes;
      const uint32_t a_addr = lane_addr + a.slot * kAColumns + part * (kAColumns / kConvParts);
      const int sw = r & 7;
      // this part's pieces kConvPieces * part .. of the row's eight 16-byte pieces (32 values each), two block scales per piece
      const uint8_t* box = stage + r * 128;
      uint4 q[kConvPieces];
#pragma unroll
      for (int j = 0; j < kConvPieces; ++j) q[j] = *reinterpret_cast<const uint4*>(box + (((kConvPieces * part + j) ^ sw) << 4));
      uint32_t sc[(kConvPieces + 1) / 2];
#pragma unroll
      for (int j = 0; j < (kConvPieces + 1) / 2; ++j)
        sc[j] = *reinterpret_cast<const uint32_t*>(stage + box_bytes + r * 16 + part * (2 * kConvPieces) + 4 * j);
      static_assert(kConvPieces % 2 == 0, "a thread's scale bytes are read as whole words");
#pragma unroll
      for (int j = 0; j < kConvPieces; ++j) {
        uint32_t p[8];
        const uint32_t sword = sc[j / 2];
        expand_nvfp4(q[j].x, q[j].y, sword >> (16 * (j & 1)), p);
        tmem_st8(a_addr + (2 * j) * 8, p);
        expand_nvfp4(q[j].z, q[j].w, sword >> (16 * (j & 1) + 8), p);
        tmem_st8(a_addr + (2 * j + 1) * 8, p);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(w_empty(w.slot));  // the bytes are in registers / tensor memory: the stage may be refilled
        mbar_arrive(a_full(a.slot));
      }
      w.advance(SW);
      a.advance(kASlots);
      a_wrapped |= a.slot == 0;
      if (++s != n_stages) continue;
      s = 0;
      // ---- the tile is over ----
      const RowTerms T = row_terms<F>(P, tile_begin + t, r);
      if (!tc_wait(d_full, t & 1, P.status)) break;
      tc_fence_after();
      pdl_wait();  // y and the activation scales come from earlier kernels
      const float inv_lo = lane < P.M ? P.inv_scales[lane] : 0.0f, inv_hi = 32 + lane < P.M ? P.inv_scales[32 + lane] : 0.0f;
      finish_tile<F, false>(P, T, lane_addr + kDColumn, lane, part, kConvParts, inv_lo, inv_hi, 0u);
      ++t;
    }
  }
  __syncthreads();
  if (warp == kIssuerWarp) tmem_dealloc(tmem_base, kTmemColumns);
}

// ---- NVFP4 with the expanded weights in shared memory ---------------------------------------------------------------
// The kernel above is bound by tcgen05.st (27 bytes per cycle and SM measured; a stage writes 64 KB). Here the converter
// warps write the f16 expansion into shared memory instead (st.shared takes 128 bytes per cycle), in the layout a
// 128-byte-swizzled tile copy would have left it, and the products read both operands from shared memory like the
// kernels of the formats that need no conversion. A weight stage (256 values of K per row, as above) is converted in two
// halves of 128 values; an A slot holds one half: two boxes of 128 rows x 128 bytes. Converter thread (row r, part p)
// expands kSsPieces 16-byte pieces (32 values, two block scales each) of its row per half.
//
// Measured on the 28672 x 8192 matrix at M = 16 / 64: 72.3 / 80.9 us, against 79.1 / 87.3 us for the kernel above in the
// same run. Variants measured and dropped: quarter-stage slots (86 us: the per-slot handshakes cost more than the finer
// overlap gives), sixteen converter warps (75 us), block scales fetched for four stages per copy (75 / 91 us: the 32 KB
// they take leave fewer weight stages). Switching the conversion off (raw bytes stored) gives 67 us and issuing one
// product in eight gives 66 us: two bounds of nearly the same height. The converters execute ~2080 warp instructions
// per stage on dependent chains; and the sixteen products of a stage take ~2050 cycles whatever their column count: the
// tensor core takes its 4 KB A tile (128 rows x 32 bytes) at about 32 bytes per cycle, and the f16 expansion is four
// times the stored bytes. A faster NVFP4 product needs the weights as the B operand (256 rows per product) or a kind
// that reads e2m1 as stored.
constexpr int kSsWarps = 8, kSsParts = kSsWarps / 4, kSsPieces = 4 / kSsParts;
constexpr int kSsProducer = kSsWarps, kSsIssuer = kSsWarps + 1, kSsThreads = (kSsWarps + 2) * 32;
constexpr int kSsSlotBytes = 2 * kBM * 128;  // one half stage of f16: 128 rows x 128 values

__global__ void __launch_bounds__(kSsThreads, 1)
    tc_nvfp4_ss_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap, const TcParams P) {
  constexpr int F = LX_W_NVFP4;
  using Fm = TcFmt<F>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int NC = P.NC, SW = P.SW, SX = P.SX, SA = P.SA;
  const int x_bytes = P.x_bytes, box_bytes = P.box_bytes, slot_bytes = P.slot_bytes;
  uint8_t* const aring = smem + static_cast<size_t>(SW) * slot_bytes;
  uint8_t* const xring = aring + static_cast<size_t>(SA) * kSsSlotBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(xring + static_cast<size_t>(SX) * x_bytes);
  const uint32_t bar0 = smem_u32(bars);
  auto w_full = [&](int s) { return bar0 + 8u * s; };
  auto w_empty = [&](int s) { return bar0 + 8u * (SW + s); };
  auto x_full = [&](int s) { return bar0 + 8u * (2 * SW + s); };
  auto x_empty = [&](int s) { return bar0 + 8u * (2 * SW + SX + s); };
  auto a_full = [&](int a) { return bar0 + 8u * (2 * SW + 2 * SX + a); };
  auto a_empty = [&](int a) { return bar0 + 8u * (2 * SW + 2 * SX + SA + a); };
  const uint32_t d_full = bar0 + 8u * (2 * SW + 2 * SX + 2 * SA);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SW + 2 * SX + 2 * SA + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_stages = (P.K + kKS4 - 1) / kKS4;
  const int n_tiles = (P.N + P.R - 1) / P.R;
  const int tile_begin = static_cast<int>(static_cast<int64_t>(n_tiles) * blockIdx.x / gridDim.x);
  const int tile_end = static_cast<int>(static_cast<int64_t>(n_tiles) * (blockIdx.x + 1) / gridDim.x);
  const int total = (tile_end - tile_begin) * n_stages;

  if (tid == 0) {
    for (int s = 0; s < SW; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), kSsWarps);
    }
    for (int s = 0; s < SX; ++s) {
      mbar_init(x_full(s), 1);
      mbar_init(x_empty(s), 1);
    }
    for (int a = 0; a < SA; ++a) {
      mbar_init(a_full(a), kSsWarps);
      mbar_init(a_empty(a), 1);
    }
    mbar_init(d_full, 1);
    mbar_init_fence();
  }
  if (warp == kSsIssuer) {
    tmem_alloc(smem_u32(tmem_slot), kTmemColumns);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kSsProducer) {
    // ================================ producers ================================
    pdl_trigger();
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&smap) : "memory");
    }
    if (lane == 0) {  // weights and their scales are static: no wait
      Ring w;
      bool ok = true, wrapped = false;
      for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
        for (int s = 0; s < n_stages; ++s) {
          if (wrapped && !tc_wait(w_empty(w.slot), w.lap ^ 1u, P.status)) {
            ok = false;
            break;
          }
          const uint32_t dst = smem_u32(smem) + static_cast<uint32_t>(w.slot) * slot_bytes;
          mbar_arrive_expect_tx(w_full(w.slot), P.R * (128 + 16));
          tile_g2s(dst, &wmap, (s * Fm::kRowBytes) / 4, tile * P.R, w_full(w.slot));
          tile_g2s(dst + box_bytes, &smap, s * 16, tile * P.R, w_full(w.slot));
          w.advance(SW);
          wrapped |= w.slot == 0;
        }
      }
    } else if (lane == 1) {
      pdl_wait();  // the prepared activations come from the kernel before this one
      Ring x;
      bool wrapped = false;
      int s = 0;
      for (int i = 0; i < total; ++i) {
        if (wrapped && !tc_wait(x_empty(x.slot), x.lap ^ 1u, P.status)) break;
        mbar_arrive_expect_tx(x_full(x.slot), x_bytes);
        bulk_g2s(smem_u32(xring) + static_cast<uint32_t>(x.slot) * x_bytes, P.xprep + static_cast<size_t>(s) * x_bytes, x_bytes, x_full(x.slot));
        x.advance(SX);
        wrapped |= x.slot == 0;
        if (++s == n_stages) s = 0;
      }
    }
  } else if (warp == kSsIssuer) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(NC >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);  // f16 x f16 -> f32
      const uint32_t lbo = static_cast<uint32_t>(NC / 8) * 128, sbo = 128;
      const uint32_t a_hi = (1024u >> 4) | (1u << 14) | (2u << 29), b_hi = (sbo >> 4) | (1u << 14);
      const uint32_t a_lo0 = ((smem_u32(aring) & 0x3ffffu) >> 4) | (1u << 16);
      const uint32_t b_lo0 = ((smem_u32(xring) & 0x3ffffu) >> 4) | ((lbo >> 4) << 16);
      const uint32_t b_step = (2u * lbo) >> 4;
      Ring x, a;
      int s = 0;
      bool ok = true;
      for (int i = 0; i < total && ok; ++i) {
        if (!tc_wait(x_full(x.slot), x.lap, P.status)) break;
        const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(x.slot) * (static_cast<uint32_t>(x_bytes) >> 4);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!tc_wait(a_full(a.slot), a.lap, P.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(a.slot) * (kSsSlotBytes >> 4);
#pragma unroll
          for (int b = 0; b < 2; ++b) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const int c = 8 * h + 4 * b + ks;  // 16 values of K per instruction
              umma_ss_halves<kActF16>(tmem_base, a_lo + b * ((kSsSlotBytes / 2) >> 4) + ks * 2, a_hi, b_lo + c * b_step, b_hi, idesc, (s | c) ? 1u : 0u);
            }
          }
          umma_commit(a_empty(a.slot));  // the half stage may be overwritten once these products are done
          a.advance(SA);
        }
        if (!ok) break;
        umma_commit(x_empty(x.slot));
        if (++s == n_stages) {
          s = 0;
          umma_commit(d_full);  // the tile's accumulator is complete when everything issued so far is
        }
        x.advance(SX);
      }
    }
  } else {
    // ================================ converters, then epilogue ================================
    const int quarter = warp & 3, part = warp >> 2;
    const int r = quarter * 32 + lane;  // weight row of the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int sw = r & 7;
    Ring w, a;
    int s = 0, t = 0;
    bool a_wrapped = false, ok = true;
    // The arrival for a slot is sent one half later, after the next half has been expanded into registers: the proxy
    // fence waits for the slot's stores to complete, and that wait is what the expansion of the next half hides.
    int owed_a = -1, owed_w = -1;  // the A slot (and, after a stage's second half, the weight slot) whose arrival is still owed
    auto settle = [&]() {
      if (owed_a < 0) return;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads what these threads wrote
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(a_full(owed_a));
        if (owed_w >= 0) mbar_arrive(w_empty(owed_w));  // both halves have been read and used: the stage may be refilled
      }
      owed_a = owed_w = -1;
    };
    for (int i = 0; i < total && ok; ++i) {
      if (!tc_wait(w_full(w.slot), w.lap, P.status)) break;
      // Rows past R read what shared memory holds behind the box (this CTA's own); their lanes are never read back.
      const uint8_t* stage = smem + static_cast<size_t>(w.slot) * slot_bytes;
      const uint8_t* box = stage + r * 128;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint4 q[kSsPieces];
#pragma unroll
        for (int j = 0; j < kSsPieces; ++j) q[j] = *reinterpret_cast<const uint4*>(box + (((4 * h + kSsPieces * part + j) ^ sw) << 4));
        uint32_t sc[kSsPieces];  // two scale bytes per piece
#pragma unroll
        for (int j = 0; j < kSsPieces; ++j)
          sc[j] = *reinterpret_cast<const uint16_t*>(stage + box_bytes + r * 16 + 2 * (4 * h + kSsPieces * part + j));
        uint32_t p[kSsPieces][16];
#pragma unroll
        for (int j = 0; j < kSsPieces; ++j) {
          uint32_t lo[8], hi[8];
          expand_nvfp4(q[j].x, q[j].y, sc[j], lo);
          expand_nvfp4(q[j].z, q[j].w, sc[j] >> 8, hi);
#pragma unroll
          for (int z = 0; z < 8; ++z) p[j][z] = lo[z], p[j][8 + z] = hi[z];
        }
        settle();
        if (a_wrapped && !tc_wait(a_empty(a.slot), a.lap ^ 1u, P.status)) {
          ok = false;
          break;
        }
        uint8_t* arow = aring + static_cast<size_t>(a.slot) * kSsSlotBytes + r * 128;
#pragma unroll
        for (int j = 0; j < kSsPieces; ++j) {
          const int g = kSsPieces * part + j;  // the piece's place in the half: box g / 2, chunks 4 (g % 2) ..
          uint8_t* dst = arow + (g >> 1) * (kSsSlotBytes / 2);
          const int c0 = 4 * (g & 1);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(dst + (((c0 + c) ^ sw) << 4)) = make_uint4(p[j][4 * c], p[j][4 * c + 1], p[j][4 * c + 2], p[j][4 * c + 3]);
        }
        owed_a = a.slot, owed_w = h == 1 ? w.slot : -1;
        a.advance(SA);
        a_wrapped |= a.slot == 0;
      }
      if (!ok) break;
      w.advance(SW);
      if (++s != n_stages) continue;
      s = 0;
      // ---- the tile is over ----
      settle();
      const RowTerms T = row_terms<F>(P, tile_begin + t, r);
      if (!tc_wait(d_full, t & 1, P.status)) break;
      tc_fence_after();
      pdl_wait();  // y and the activation scales come from earlier kernels
      const float inv_lo = lane < P.M ? P.inv_scales[lane] : 0.0f, inv_hi = 32 + lane < P.M ? P.inv_scales[32 + lane] : 0.0f;
      finish_tile<F, false>(P, T, lane_addr, lane, part, kSsParts, inv_lo, inv_hi, 0u);
      ++t;
    }
  }
  __syncthreads();
  if (warp == kSsIssuer) tmem_dealloc(tmem_base, kTmemColumns);
}

// LX_B200_NVFP4_TMEM=1 keeps the kernel that expands into tensor memory.
bool nvfp4_through_tmem() {
  static const bool on = [] {
    const char* v = std::getenv("LX_B200_NVFP4_TMEM");
    return v && v[0] == '1';
  }();
  return on;
}

// ---- launching -------------------------------------------------------------------------------------------------------
// LX_B200_TC_SMALL=1 lets products whose rings fit take small CTAs (two per SM); LX_B200_TC_SMALL_STAGES sets the fewest
// weight stages a small CTA must keep (default 3). Off by default: measured on C2, a product between small neighbours
// gains 5 % (the next product's first stages arrive while this one drains; it cannot start multiplying before this one
// has finished, whose output its activations may be), but a stream that alternates small and large CTAs loses more
// than that.
bool small_ctas() {
  static const bool on = [] {
    const char* v = std::getenv("LX_B200_TC_SMALL");
    return v && v[0] == '1';
  }();
  return on;
}
int small_min_stages() {
  static const int n = [] {
    const char* v = std::getenv("LX_B200_TC_SMALL_STAGES");
    return v ? std::max(2, atoi(v)) : 3;
  }();
  return n;
}

// Rows per tile: the fewest whole tiles per SM that keep a tile within 128 rows, then the rows that spread N evenly
// over that many tiles.
int tile_rows(int N, int sms) {
  const int per_sm = (N + kBM * sms - 1) / (kBM * sms);
  const int rows = (N + per_sm * sms - 1) / (per_sm * sms);
  return std::min(kBM, std::max(kMinTileRows, rows));
}

template <int F, int XMODE>
int tc_launch(const lx_weight& w, TcParams P, cudaStream_t stream, int* grid_out = nullptr) {
  using Fm = TcFmt<F>;
  constexpr int kBoxes = Fm::kRowBytes / 128;
  const int sms = sm_count();
  if (!sms) return kInvalid;
  P.R = tile_rows(P.N, sms);
  P.box_bytes = (P.R + 7) / 8 * 1024;
  // NVFP4 keeps a stage's box and its block scales in a slot of twice the box, so that every box starts 1024-aligned.
  const int w_stage = F == LX_W_NVFP4 ? 2 * P.box_bytes : kBoxes * P.box_bytes;
  constexpr int kStaging = XMODE == 0 ? 0 : own_staging_bytes(XMODE == 1);
  // Two sizes of CTA. Small: at most half of an SM's shared memory and tensor memory, so that the CTAs of the NEXT kernel
  // in the stream (launched programmatically, their weights static) move in beside this kernel's and fill their rings
  // while these drain: the weight stream never stops between products. Measured on plain tile copies of a 58 MB weight,
  // back to back: 12.7 us per pass with one CTA per SM and no overlap, 8.2 us with the next kernel's CTAs resident.
  // Large (one CTA per SM, deeper rings): for activation blocks that leave a small CTA fewer than two weight stages,
  // or more than 256 accumulator columns.
  constexpr int kSmall = 113 * 1024 - 512, kLarge = 204 * 1024;  // large: room for the 16 KB the tensor core may read past the last box
  constexpr int kBars = 1024;
  P.dstride = P.NC;
  P.tmem_cols = 32;
  while (P.tmem_cols < 2 * P.NC) P.tmem_cols *= 2;
  const int small_sw = small_ctas() && F != LX_W_NVFP4 && P.tmem_cols <= 256 ? (kSmall - kBars - std::max(2 * P.x_bytes + kStaging, 16 * 1024)) / w_stage : 0;
  const bool small = small_sw >= small_min_stages();
  size_t smem;
  if (small) {
    P.SX = 2;
    P.SW = std::min(12, small_sw);
    smem = static_cast<size_t>(P.SW) * w_stage + std::max(P.SX * P.x_bytes + kStaging, 16 * 1024) + kBars;
  } else {
    if (XMODE) {
      // CTAs that prepare their own (small) activation blocks keep one ring: a block per weight stage, one barrier for both
      P.SW = P.SX = std::min(12, (kLarge - kStaging) / (w_stage + P.x_bytes));
    } else if (F != LX_W_NVFP4 && kLarge / (w_stage + P.x_bytes) >= 4) {
      P.SW = P.SX = std::min(12, kLarge / (w_stage + P.x_bytes));  // one ring again: one commit per stage
    } else {
      // Large activation blocks (64 rows of two digits are 32 KB per stage): measured at M = 64 on the 28672 x 8192 FP8
      // matrix, three, four or five weight stages make no difference (57.9-58.2 us) while a third activation slot gives
      // 54.8 us and a single one 95.7 us: a block is asked for only when the products that used its slot are done, then
      // travels from L2 for a microsecond, so the activation ring is what is latency-bound (a fourth slot at the price of
      // a weight stage: 56.3 us). Up to three activation slots as long as three weight stages stay, the rest to the weights.
      constexpr int kRoom = 222 * 1024 - kBars;
      P.SX = std::max(2, std::min(3, (kRoom - 3 * w_stage - kStaging) / P.x_bytes));
      P.SW = std::min(12, (kRoom - P.SX * P.x_bytes - kStaging) / w_stage);
    }
    if (P.SW < 2) return kNotSupported;
    P.tmem_cols = kTmemColumns, P.dstride = 256;
    // all of tensor memory: exactly one CTA may live on an SM, so ask for more than half of its shared memory
    smem = std::max<size_t>(static_cast<size_t>(P.SW) * w_stage + std::max(P.SX * P.x_bytes + kStaging, 16 * 1024) + kBars, 120 * 1024);
  }
  alignas(64) CUtensorMap wmap, smap;
  memset(&wmap, 0, sizeof(wmap));
  memset(&smap, 0, sizeof(smap));
  const int64_t row_bytes = F == LX_W_BF16 ? 2ll * P.K : F == LX_W_NVFP4 ? P.K / 2 : P.K;
  if (int e = make_tile_map(&wmap, w.data, row_bytes, P.N, 128, P.R, 4, true)) return e;
  const int tiles = (P.N + P.R - 1) / P.R;
  const int grid = std::min(tiles, sms);
  if (grid_out) *grid_out = grid;
  if constexpr (F == LX_W_NVFP4) {
    static_assert(XMODE == 0, "NVFP4 takes prepared activations");
    if (int e = make_tile_map(&smap, w.scale, P.K / 16, P.N, 16, P.R, 1, false)) return e;
    if (!nvfp4_through_tmem()) {
      // weight slots of the box and 128 rows of scales; two or three half-stage A slots; two activation blocks
      constexpr int kBudget = 224 * 1024;
      const int slot = (P.box_bytes + kBM * 16 + 1023) / 1024 * 1024;
      P.SX = 2;
      int sa = 3;
      int sw_fit = (kBudget - kBars - P.SX * P.x_bytes - sa * kSsSlotBytes) / slot;
      if (sw_fit < 5) sa = 2, sw_fit = (kBudget - kBars - P.SX * P.x_bytes - sa * kSsSlotBytes) / slot;
      if (sw_fit >= 2) {
        P.SW = std::min(12, sw_fit);
        P.SA = sa, P.slot_bytes = slot;
        const size_t bytes = static_cast<size_t>(P.SW) * slot + static_cast<size_t>(sa) * kSsSlotBytes + P.SX * P.x_bytes + kBars;
        if (int e = allow_big_smem<F * 4 + 1>(tc_nvfp4_ss_kernel)) return e;
        return launch_kernel(tc_nvfp4_ss_kernel, dim3(grid), dim3(kSsThreads), bytes, stream, wmap, smap, P);
      }
    }
    if (int e = allow_big_smem<F * 4>(tc_nvfp4_kernel)) return e;
    return launch_kernel(tc_nvfp4_kernel, dim3(grid), dim3(kConvThreads), smem, stream, wmap, smap, P);
  } else {
    if (P.peers > 0) {
      if (int e = allow_big_smem<64 + F * 4 + XMODE>(tc_direct_kernel<F, XMODE, true>)) return e;
      return launch_kernel(tc_direct_kernel<F, XMODE, true>, dim3(grid), dim3(XMODE ? kOwnThreads : kDirectThreads), smem, stream, wmap, P);
    }
    if (int e = allow_big_smem<F * 4 + XMODE>(tc_direct_kernel<F, XMODE, false>)) return e;
    return launch_kernel(tc_direct_kernel<F, XMODE, false>, dim3(grid), dim3(XMODE ? kOwnThreads : kDirectThreads), smem, stream, wmap, P);
  }
}

// Activation rows one pass takes: the block of one stage stays within 48 KB.
int rows_per_pass(int act, bool x_bf16) { return (act == kActBf16 && !x_bf16) ? 32 : kMaxRows; }

// Fills what every pass shares.
TcParams base_params(const lx_weight& w, const void* bias, int bias_dtype, int y_dtype, int ld_y, int N, int K, float alpha, float beta,
                     int act, bool x_bf16, int rows, bool quantized = false) {
  TcParams P{};
  P.scale = static_cast<const uint8_t*>(w.scale);
  P.global = w.global;
  P.N = N, P.K = K, P.M = rows;
  P.planes = quantized ? 1 : act_planes(act, x_bf16);
  P.digit = act == kActS8 ? 0.0078125f : act == kActE4m3 ? 0.0625f : 1.0f;
  P.Mp = (rows + 7) / 8 * 8;
  P.NC = (P.planes * P.Mp + 15) / 16 * 16;
  P.x_bytes = P.NC * ks_of(act) * act_elem(act);
  P.bias = bias, P.bias_dtype = bias_dtype;
  P.y_dtype = y_dtype, P.ld_y = ld_y;
  P.alpha = alpha, P.beta = beta;
  P.status = status_word();
  return P;
}

}  // namespace

bool tc_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LX_B200_TC");
    return !(v && v[0] == '0');
  }();
  return on;
}

// Can up to 8 activation rows go through the tensor-core product without a workspace? INT8 and FP8 weights whose
// tiles come out at 40 rows or more (smaller ones leave the tensor pipe's instruction rate, not HBM, as the bound),
// rows of whole 16-byte pieces. The answer depends on the weight and its shape only, never on the row count, so that
// a row's bits do not depend on its batch. (BF16 stays with the streaming kernel, whose bits the lossless BF16X
// format must reproduce.)
bool tc_rows_shape_ok(int wtype, int N, int K) {
  if (!tc_enabled() || (wtype != LX_W_INT8 && wtype != LX_W_FP8) || K % 16 != 0) return false;
  const int sms = sm_count();
  return sms > 0 && tile_rows(N, sms) >= 40;
}
bool tc_rows_ok(const lx_weight& w, int N, int K) {
  return tc_rows_shape_ok(w.type, N, K) && (reinterpret_cast<uintptr_t>(w.data) & 15) == 0;
}

// Up to 8 activation rows, prepared by the product kernel itself: one launch, no workspace.
int tc_product_rows(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype, void* y, int y_dtype,
                    int ld_y, int M, int N, int K, float alpha, float beta, cudaStream_t stream) {
  const bool x_bf16 = x_dtype == LX_BF16;
  TcParams P = base_params(w, bias, bias_dtype, y_dtype, ld_y, N, K, alpha, beta, act_of(w.type), x_bf16, M);
  P.x = x, P.ld_x = ld_x;
  P.y = y;
  if (w.type == LX_W_INT8) return x_bf16 ? tc_launch<LX_W_INT8, 1>(w, P, stream) : tc_launch<LX_W_INT8, 2>(w, P, stream);
  if (w.type == LX_W_FP8) return x_bf16 ? tc_launch<LX_W_FP8, 1>(w, P, stream) : tc_launch<LX_W_FP8, 2>(w, P, stream);
  return kNotSupported;
}

// The product, in passes of at most 64 activation rows. workspace: at least tc_workspace_bytes. quantized (INT8 and
// FP8 weights only): activations quantized per row to the weight's number type instead of split into exact digits.
int tc_product(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype, void* y, int y_dtype,
               int ld_y, int M, int N, int K, float alpha, float beta, void* workspace, cudaStream_t stream, bool quantized) {
  const bool x_bf16 = x_dtype == LX_BF16;
  if (quantized && w.type != LX_W_INT8 && w.type != LX_W_FP8) return kNotSupported;
  const int act = act_of(w.type), elem = act_elem(act), kKS = ks_of(act);
  const int per_pass = rows_per_pass(act, true);  // f32 activations become bf16 (or quantized) values: as many planes as bf16
  const int n_stages = (K + kKS - 1) / kKS;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  for (int m0 = 0; m0 < M; m0 += per_pass) {
    const int rows = std::min(per_pass, M - m0);
    TcParams P = base_params(w, bias, bias_dtype, y_dtype, ld_y, N, K, alpha, beta, act, true, rows, quantized);
    const TcLayout L(P.NC, act, n_stages);
    P.xprep = ws;
    P.inv_scales = reinterpret_cast<const float*>(ws + L.scales);
    P.y = static_cast<uint8_t*>(y) + static_cast<int64_t>(m0) * ld_y * (y_dtype == LX_BF16 ? 2 : 4);
    const uint8_t* xrow = static_cast<const uint8_t*>(x) + static_cast<int64_t>(m0) * ld_x * (x_bf16 ? 2 : 4);
    const int per_block = 128 * 16 / elem;
    const dim3 prep_grid((n_stages * kKS + per_block - 1) / per_block, rows);
    auto prep = [&](auto kernel) {
      return launch_kernel(kernel, prep_grid, dim3(128), 0, stream, static_cast<const void*>(xrow), ld_x, rows, K, P.NC, P.Mp, P.planes, ws,
                           reinterpret_cast<float*>(ws + L.scales), n_stages);
    };
    int pe;
    if (quantized) {
      if (act == kActS8) pe = x_bf16 ? prep(tc_prep_kernel<kActS8, true, kPrepQuant>) : prep(tc_prep_kernel<kActS8, false, kPrepQuant>);
      else pe = x_bf16 ? prep(tc_prep_kernel<kActE4m3, true, kPrepQuant>) : prep(tc_prep_kernel<kActE4m3, false, kPrepQuant>);
    } else {
      switch (act * 2 + (x_bf16 ? 1 : 0)) {
        case kActBf16 * 2: pe = prep(tc_prep_kernel<kActBf16, false, kPrepRound>); break;
        case kActBf16 * 2 + 1: pe = prep(tc_prep_kernel<kActBf16, true>); break;
        case kActF16 * 2: pe = prep(tc_prep_kernel<kActF16, false, kPrepRound>); break;
        case kActF16 * 2 + 1: pe = prep(tc_prep_kernel<kActF16, true>); break;
        case kActE4m3 * 2: pe = prep(tc_prep_kernel<kActE4m3, false, kPrepRound>); break;
        case kActE4m3 * 2 + 1: pe = prep(tc_prep_kernel<kActE4m3, true>); break;
        case kActS8 * 2: pe = prep(tc_prep_kernel<kActS8, false, kPrepRound>); break;
        default: pe = prep(tc_prep_kernel<kActS8, true>); break;
      }
    }
    if (pe) return pe;
    int e;
    switch (w.type) {
      case LX_W_BF16: e = tc_launch<LX_W_BF16, 0>(w, P, stream); break;
      case LX_W_INT8: e = tc_launch<LX_W_INT8, 0>(w, P, stream); break;
      case LX_W_FP8: e = tc_launch<LX_W_FP8, 0>(w, P, stream); break;
      case LX_W_NVFP4: e = tc_launch<LX_W_NVFP4, 0>(w, P, stream); break;
      default: e = kNotSupported;
    }
    if (e) return e;
  }
  return kOk;
}

// ---- the product with an all-gather epilogue ---------------------------------------------------------------------------
// A counting semaphore: waits (bounded) until the counter holds at least `total` arrivals, then takes them. Arrivals of
// a later round that come early stay in the counter, and nothing here depends on how often the call has run before, so
// a captured graph can be replayed.
__global__ void wait_arrivals_kernel(int* counter, int total, int* status, uint64_t budget_ns) {
  pdl_trigger();
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    if (v >= total) break;
    if (global_timer_ns() - t0 > budget_ns) {  // a peer that never arrives: give up (after a second by default) and say so
      if (status) atomicExch(status, kStatusTcWait);
      return;
    }
  }
  asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(counter), "r"(-total) : "memory");
}

// LX_B200_WAIT_MS: how long a wait for peers may last before it gives up (default 1000; read on every call).
int tc_wait_arrivals(int* counter, int total, cudaStream_t stream) {
  uint64_t ms = 1000;
  if (const char* v = std::getenv("LX_B200_WAIT_MS")) ms = static_cast<uint64_t>(std::max(1, std::min(10000, atoi(v))));
  return launch_kernel(wait_arrivals_kernel, dim3(1), dim3(1), 0, stream, counter, total, status_word(), ms * 1000000ull);
}

// One pass (M <= 64 rows for bf16 activations) of BF16 / INT8 / FP8 weights whose outputs go straight into every rank's
// y. *arrivals_added: what this launch adds to each rank's semaphore when it is done.
int tc_product_allgather(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype,
                         const PeerTargets& T, int y_dtype, int ld_y, int M, int N, int K, float alpha, void* workspace,
                         int* arrivals_added, cudaStream_t stream) {
  if (!tc_enabled() || T.ranks < 1 || T.ranks > 8 || T.self < 0 || T.self >= T.ranks) return kNotSupported;
  if (w.type != LX_W_BF16 && w.type != LX_W_INT8 && w.type != LX_W_FP8) return kNotSupported;
  const bool x_bf16 = x_dtype == LX_BF16;
  const int act = act_of(w.type);
  const bool own = M <= 8 && tc_rows_ok(w, N, K);
  if (!own && (!workspace || M > rows_per_pass(act, x_bf16))) return kNotSupported;
  TcParams P = base_params(w, bias, bias_dtype, y_dtype, ld_y, N, K, alpha, 0.0f, act, x_bf16, M);
  P.peers = T.ranks, P.col0 = T.col0;
  for (int g = 0; g < T.ranks; ++g) P.y_peer[g] = T.y_all[g], P.flag_peer[g] = T.arrivals[g];
  P.done_local = T.arrivals[T.self] + 1;
  int grid = 0, e;
  if (own) {
    P.x = x, P.ld_x = ld_x;
    if (w.type == LX_W_INT8) e = x_bf16 ? tc_launch<LX_W_INT8, 1>(w, P, stream, &grid) : tc_launch<LX_W_INT8, 2>(w, P, stream, &grid);
    else e = x_bf16 ? tc_launch<LX_W_FP8, 1>(w, P, stream, &grid) : tc_launch<LX_W_FP8, 2>(w, P, stream, &grid);
  } else {
    const int elem = act_elem(act), kKS = ks_of(act), n_stages = (K + kKS - 1) / kKS;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    const TcLayout L(P.NC, act, n_stages);
    P.xprep = ws;
    P.inv_scales = reinterpret_cast<const float*>(ws + L.scales);
    const int per_block = 128 * 16 / elem;
    const dim3 prep_grid((n_stages * kKS + per_block - 1) / per_block, M);
    auto prep = [&](auto kernel) {
      return launch_kernel(kernel, prep_grid, dim3(128), 0, stream, x, ld_x, M, K, P.NC, P.Mp, P.planes, ws, reinterpret_cast<float*>(ws + L.scales),
                           n_stages);
    };
    int pe;
    switch (act * 2 + (x_bf16 ? 1 : 0)) {
      case kActBf16 * 2: pe = prep(tc_prep_kernel<kActBf16, false>); break;
      case kActBf16 * 2 + 1: pe = prep(tc_prep_kernel<kActBf16, true>); break;
      case kActE4m3 * 2: pe = prep(tc_prep_kernel<kActE4m3, false>); break;
      case kActE4m3 * 2 + 1: pe = prep(tc_prep_kernel<kActE4m3, true>); break;
      case kActS8 * 2: pe = prep(tc_prep_kernel<kActS8, false>); break;
      default: pe = prep(tc_prep_kernel<kActS8, true>); break;
    }
    if (pe) return pe;
    switch (w.type) {
      case LX_W_BF16: e = tc_launch<LX_W_BF16, 0>(w, P, stream, &grid); break;
      case LX_W_INT8: e = tc_launch<LX_W_INT8, 0>(w, P, stream, &grid); break;
      default: e = tc_launch<LX_W_FP8, 0>(w, P, stream, &grid); break;
    }
  }
  if (e) return e;
  (void)grid;
  if (arrivals_added) *arrivals_added = 1;  // the grid's last epilogue warp signals once
  return kOk;
}

// Bytes of workspace the product needs for M activation rows, whatever the weight format and activation dtype.
int64_t tc_workspace_bytes(int M, int K) {
  const int rows = std::min(M, kMaxRows);
  int64_t need = 0;
  for (int act = 0; act < 4; ++act)
    for (int bf = 0; bf < 2; ++bf) {
      const int r = std::min(rows, rows_per_pass(act, bf != 0));
      const int NC = (act_planes(act, bf != 0) * ((r + 7) / 8 * 8) + 15) / 16 * 16;
      need = std::max(need, TcLayout(NC, act, (K + ks_of(act) - 1) / ks_of(act)).total);
    }
  return need;
}

}  // namespace b200
