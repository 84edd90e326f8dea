// Host-side launch helpers: every kernel of the library is launched through launch_kernel, which counts the launch,
// marks it for programmatic dependent launch (the kernel may start while its predecessor in the stream drains; it
// calls griddepcontrol.wait before reading anything the predecessor wrote) and returns the launch status.
#pragma once

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "stream.cuh"

namespace b200 {

// LX_PDL=0 turns programmatic dependent launch off (plain stream order), as in the reference's common.cuh switch.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LX_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

// LX_B200_FORCE_SCALAR=1 sends every dense product down the scalar kernel (a second implementation to test against).
inline bool force_scalar() {
  const char* v = std::getenv("LX_B200_FORCE_SCALAR");
  return v && v[0] == '1';
}

template <typename... KArgs, typename... Args>
int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(e);
  }
  return kOk;
}

// Scratch for the stage-granular split of dense products: per device, a few regions handed out in turn (consecutive
// launches never share one), each holding kSplitMaxCtas partial-sum slots of kSplitBytesPerCta bytes and their flags.
// Allocated on first use and kept for the life of the process; the flags are zero whenever no kernel is running.
constexpr int kSplitMaxCtas = 1024;
constexpr int kSplitBytesPerCta = 8192;
constexpr int kSplitRegions = 4;
int split_scratch(float** partials, int** flags);
// Off unless LX_B200_SPLIT_K=1: measured on B200, the hand-off between CTAs (fence, flag, partial loads, about 3 us)
// costs more than the better balance wins at decode sizes, so by default every tile stays whole in one CTA.
inline bool split_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LX_B200_SPLIT_K");
    return v && v[0] == '1';
  }();
  return on;
}

// cuTensorMapEncodeTiled, fetched from the driver through the runtime (the library does not link libcuda).
using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encoder();

// A 2-D map over `rows` rows of `row_bytes` bytes each (row pitch = row_bytes, a multiple of 16; base 16-byte aligned),
// copied in boxes of box_rows x box_bytes. elem_bytes (1 or 4) is the unit the kernel gives x coordinates in. With
// swizzle128 (boxes 128 bytes wide) the 16-byte pieces of row r land at piece ^ (r % 8).
inline int make_tile_map(CUtensorMap* map, const void* base, int64_t row_bytes, int64_t rows, int box_bytes, int box_rows,
                         int elem_bytes, bool swizzle128 = false) {
  TensorMapEncodeFn encode = tensor_map_encoder();
  if (!encode) return kNotSupported;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes / elem_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes / elem_bytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_INT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kInvalid;
}

// Launches the persistent streaming kernel: as many CTAs as the device holds at once (or one per tile when there are
// fewer tiles). stack_rows: rows of the whole weight the kernel may address (N, or E * N for a stack of experts).
template <int F, int NW, int RT, int WR, int NT, int U, int S, int XKB, int MODE>
int launch_stream(StreamParams P, cudaStream_t stream, int64_t stack_rows) {
  using C = StreamCfg<F, NW, RT, WR, NT, U, S, XKB>;
  auto kernel = stream_kernel<F, NW, RT, WR, NT, U, S, XKB, MODE>;
  const size_t smem = stream_smem_bytes<F, NW, RT, WR, NT, U, S, XKB>(P.K);
  if (smem > 226 * 1024) return kNotSupported;
  // The opt-in to more than 48 KB of dynamic shared memory is per device and per kernel; set it once per device,
  // with the whole of the SM's L1 given to shared memory so that as many CTAs fit as their sizes allow.
  static std::mutex mu;
  static int ctas_per_sm[64] = {};  // per device ordinal; 0 = not set up yet
  static int sm_count[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!ctas_per_sm[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      int n = 0, sms = 0;
      if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, C::kThreads, smem);
      if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) {
        cudaGetLastError();
        return static_cast<int>(e);
      }
      if (n < 1) return kNotSupported;
      ctas_per_sm[dev] = n;
      sm_count[dev] = sms;
    }
  }
  alignas(64) CUtensorMap wmap, smap;
  memset(&wmap, 0, sizeof(wmap));
  memset(&smap, 0, sizeof(smap));
  // BF16X records come as tiles when they and their data start on 16-byte boundaries; every other format always does
  // (the callers check that the weight streams).
  P.tiled = !C::kX16 || (aligned(P.w, 16) && P.row_bytes % 16 == 0 && x16::header_bytes(P.K) % 16 == 0);
  if (P.tiled) {
    const int box_rows = MODE == kGateUp ? C::R / 2 : C::R;
    if (int e = make_tile_map(&wmap, P.w, P.row_bytes, stack_rows, C::BOXW, box_rows, 4)) return e;
    if constexpr (F == LX_W_NVFP4)
      if (int e = make_tile_map(&smap, P.scale, P.K / 16, stack_rows, C::SCALE_SEG, box_rows, 1)) return e;
  }
  const int rows_per_tile = MODE == kGateUp ? C::R / 2 : C::R;
  const int64_t rows_total = MODE == kGateUp ? P.I : P.N;
  const int64_t tiles = (rows_total + rows_per_tile - 1) / rows_per_tile * (MODE == kDense ? 1 : P.groups);
  const int64_t resident = static_cast<int64_t>(ctas_per_sm[dev]) * sm_count[dev];
  int64_t units = tiles;
  P.split_k = 0;
  if constexpr (MODE == kDense && C::R * C::COLS * 4 <= kSplitBytesPerCta) {
    // Stage-granular split: one pass over the weights, activations resident in the unit buffer, and scratch at hand.
    const int T = terms_for(C::kMma, P.x_dtype == LX_BF16), n_cols = P.M * T;
    const int64_t n_stages = (P.K + C::KSTAGE - 1) / C::KSTAGE;
    const int64_t x_bytes = n_stages * (C::KSTAGE / C::GV) * 16 * NT * (NT == 1 ? n_cols : 8);
    if (n_cols <= C::COLS && x_bytes <= C::XBYTES && resident <= kSplitMaxCtas && split_enabled() &&
        split_scratch(&P.partials, &P.flags) == kOk) {
      P.split_k = 1;
      units = tiles * n_stages;
    }
  }
  const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min(units, resident)));
  return launch_kernel(kernel, dim3(grid), dim3(C::kThreads), smem, stream, wmap, smap, P);
}

// Which (math, stored format) pairs lx_gemm_w and lx_moe_experts_grouped compute, decided as the reference decides it
// (lernex/dromos engine/cuda/gemm_w.cuh:274-289): nothing below architecture 80; BF16 math with every format; INT8 math
// with INT8 weights; FP8 math with FP8 weights from architecture 89. FP8 math on NVFP4 weights and FP4 math are products
// of the 12x parts only. 0 = admitted, else the error to return. lx_arch() honours the architecture override.
inline int math_admitted(int math, int wtype) {
  const int arch = lx_arch();
  if (arch < 80) return kNotSupported;
  switch (math) {
    case LX_MATH_BF16: return kOk;
    case LX_MATH_INT8: return wtype == LX_W_INT8 ? kOk : kNotSupported;
    case LX_MATH_FP8: return wtype == LX_W_FP8 && arch >= 89 ? kOk : kNotSupported;
    default: return kNotSupported;
  }
}

// gemm_tc.cu: the tcgen05 product for batched decode rows, and the workspace its prepared activations need.
int tc_product(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype, void* y, int y_dtype,
               int ld_y, int M, int N, int K, float alpha, float beta, void* workspace, cudaStream_t stream, bool quantized = false);
int64_t tc_workspace_bytes(int M, int K);
bool tc_enabled();
// Where the all-gather epilogue of a sharded product stores: every rank's copy of the whole y and arrival counter.
struct PeerTargets {
  void* const* y_all;      // host array: every rank's whole-y buffer (peer-mapped device pointers), this rank's too
  int* const* arrivals;    // host array: every rank's counter pair {arrivals semaphore, finished warps of its own grid}
  int ranks, self;         // how many ranks, and which of them this one is
  int64_t col0;            // first column of this rank's slice in the whole y
};
int tc_product_allgather(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype,
                         const PeerTargets& T, int y_dtype, int ld_y, int M, int N, int K, float alpha, void* workspace,
                         int* arrivals_added, cudaStream_t stream);
int tc_wait_arrivals(int* counter, int total, cudaStream_t stream);
// Rows of one expert that a tile of the tensor-core expert kernels multiplies at once, and the tables that cut the sorted
// pairs into such chunks (written by group_kernel, read by the kernels of moe_tc.cu; they live in the workspace).
constexpr int kExpertChunkRows = 16;
struct ExpertChunkTables {
  int32_t* n_chunks;      // one word: how many chunks
  int32_t* chunk_expert;  // per chunk: its expert,
  int32_t* chunk_row0;    //   the sorted position of its first row,
  int32_t* chunk_rows;    //   its rows (1..16)
  int32_t* pos_chunk;     // per sorted position: its chunk
  int32_t* pos_col;       //   and its row inside the chunk
};
ExpertChunkTables expert_chunk_tables(uint8_t* ws, int64_t base, int P, int E, int L, int I);
bool experts_tc_ok(const lx_weight& gate_up, const lx_weight& down, int L, int I);
int64_t experts_tc_workspace(int64_t base, int P, int E, int L, int I);
int experts_tc(const void* latent, const float* weights, const lx_weight& gate_up, const lx_weight& down, const int32_t* offsets,
               const int32_t* pairs, uint16_t* mid, float* rows, uint8_t* ws, int64_t base, int T, int L, int I, int E, int top_k,
               int* status, cudaStream_t stream, bool quantized = false, int stack_experts = 0);
bool tc_rows_ok(const lx_weight& w, int N, int K);
bool gemv_shape_ok(int wtype, int K, bool x_bf16);
bool tc_rows_shape_ok(int wtype, int N, int K);
int tc_product_rows(const void* x, int x_dtype, int ld_x, const lx_weight& w, const void* bias, int bias_dtype, void* y, int y_dtype,
                    int ld_y, int M, int N, int K, float alpha, float beta, cudaStream_t stream);

struct ActLayout {
  int64_t ld_q, ld_bs;
  int64_t q_off, scale_off, bs_off, total;
};
ActLayout act_layout(int M, int K, int math);

}  // namespace b200
