/* libdromos_b200.so: the decode weight-streaming products of the Dromos kernel ABI, for NVIDIA B200 (sm_100a).
 *
 * Every function below has the name, argument list, argument meaning and error behaviour of the function
 * it replaces in the reference project's backend interface (lernex/dromos engine/cuda/kernels.h and
 * engine/cuda/tunable.h; the line cited beside each declaration). The reference's dispatcher resolves
 * backend entry points by name with dlsym from one shared library chosen by LX_KERNELS=<file>
 * (engine/dispatch/dispatch.cpp:198-205, tools/gen_dispatch.py:200-211), so exporting these names is the
 * whole integration: functions this library does not export answer LX_ERR_NOT_SUPPORTED from the
 * dispatcher's own stub (tools/gen_dispatch.py:168-184).
 *
 * Where the behaviour is narrower than the reference's: lx_gemm_w and lx_moe_experts_grouped compute LX_MATH_BF16 on
 * every format, LX_MATH_INT8 on INT8 weights and LX_MATH_FP8 on FP8 weights; LX_MATH_FP4 and LX_MATH_FP8 on NVFP4 weights
 * (products of the 12x parts in the reference) answer LX_ERR_NOT_SUPPORTED, as does any pair under an architecture
 * override below the pair's first architecture. Tile-variant families exist for lx_gemm_w only, with one variant each.
 *
 * Conventions (kernels.h:1-4, 29-38): pointers are device pointers to row-major buffers, ld_* is a row
 * stride in elements, `stream` is a cudaStream_t passed as void* (null = default stream), weights are
 * [out, in] and y = x @ W^T. Functions return a cudaError_t value: 0 success, 1 invalid argument, 801 an
 * unsupported format / math / shape. No function falls back to the CPU.
 */
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef LX_API
#define LX_API __attribute__((visibility("default")))
#endif

/* kernels.h:27 */
typedef enum { LX_F32 = 0, LX_BF16 = 1 } lx_dtype;
/* kernels.h:243 */
typedef enum { LX_W_BF16 = 0, LX_W_INT8 = 1, LX_W_FP8 = 2, LX_W_NVFP4 = 3, LX_W_BF16X = 4 } lx_wtype;
/* kernels.h:431 */
typedef enum { LX_MATH_BF16 = 0, LX_MATH_INT8 = 1, LX_MATH_FP8 = 2, LX_MATH_FP4 = 3 } lx_math;
/* kernels.h:302-303 */
#define LX_ERR_NOT_SUPPORTED 801
typedef enum { LX_BACKEND_CUDA = 0, LX_BACKEND_HIP = 1, LX_BACKEND_METAL = 2, LX_BACKEND_CPU = 3 } lx_backend;
/* tunable.h:27-32 */
#define LX_ERR_TUNE_REJECTED 802
#define LX_ERR_TUNE_VARIANT 803

/* kernels.h:411-417. A host struct; data / scale / expert_global are device pointers.
 *   LX_W_BF16   data bf16 [N, K]
 *   LX_W_INT8   data int8 [N, K], scale f32 [N]:                 w = q * scale[n]
 *   LX_W_FP8    data e4m3 [N, K], scale f32 [N]:                 w = fp8 * scale[n]
 *   LX_W_NVFP4  data u8 [N, K/2] (low nibble = even k), scale e4m3 [N, K/16], global f32
 *   LX_W_BF16X  data = N records of lx_bf16x_row_bytes(K) bytes (+ overflow records)
 * Stacks [E, N, K] are the experts one after the other; an NVFP4 stack may carry expert_global f32 [E]. */
typedef struct {
  lx_wtype type;
  const void* data;
  const void* scale;
  float global;
  const float* expert_global;
} lx_weight;

/* ---- decode GEMV, M <= 8 rows -------------------------------------------------------------------------
 * y[m, n] = alpha * (sum_k x[m, k] * w[n, k] + bias[n]) + beta * y[m, n]; f32 accumulation; y is read only
 * when beta != 0; deterministic; a row's bits do not depend on M. */
/* kernels.h:436 (engine/cuda/gemv.cu:1183) */
LX_API int lx_gemv_w(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, const void* bias,
                     lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                     float beta, void* stream);
/* kernels.h:244 (gemv.cu:1239): bf16 or int8 weights with a per-row scale */
LX_API int lx_gemv(const void* x, lx_dtype x_dtype, int ld_x, const void* w, lx_wtype w_type, const float* w_scale,
                   const void* bias, lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K,
                   float alpha, float beta, void* stream);
/* kernels.h:589 (engine/cuda/bf16x.cu:1297): LX_W_BF16X weights, y bit-identical to the bf16 product */
LX_API int lx_gemv_bf16x(const void* x, lx_dtype x_dtype, int ld_x, const void* w, const void* bias,
                         lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                         float beta, void* stream);
/* kernels.h:594: the same product on plain bf16 weights */
LX_API int lx_gemv_decode_bf16(const void* x, lx_dtype x_dtype, int ld_x, const void* w, const void* bias,
                               lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K,
                               float alpha, float beta, void* stream);

/* ---- batched decode / prefill product, any M ------------------------------------------------------------
 * kernels.h:448, 451 (engine/cuda/gemm_w.cu:187-192). workspace: at least lx_gemm_workspace_bytes. */
LX_API int lx_gemm_w(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, lx_math math, const void* bias,
                     lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                     float beta, void* workspace, void* stream);
LX_API int64_t lx_gemm_workspace_bytes(int M, int K, lx_math math);
/* kernels.h:475 (engine/cuda/gemm_skinny.cu:286): bf16 weights, bf16 x, any M in chunks of 64 */
LX_API int lx_gemm_skinny(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, const void* bias,
                          lx_dtype bias_dtype, void* y, lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha,
                          float beta, void* stream);

/* ---- quantizers (load time) ----------------------------------------------------------------------------- */
/* kernels.h:492 (engine/cuda/quant_act.cu:279) */
LX_API int lx_quantize_act(const void* x, lx_dtype x_dtype, int ld_x, lx_math math, void* q, int ld_q, float* scale,
                           void* block_scale, int ld_bs, int M, int K, void* stream);
/* kernels.h:518 (engine/cuda/quant.cu:140). NVFP4 synchronizes the stream and writes out->global. */
LX_API int lx_quantize_weight(const void* w, lx_weight* out, int64_t rows, int cols, void* stream);
/* kernels.h:523 (quant.cu:196) */
LX_API int lx_dequantize_weight(const lx_weight* w, void* out, int64_t rows, int cols, void* stream);
/* kernels.h:251 (gemv.cu:1251) */
LX_API int lx_quantize_w8(const void* w, int8_t* q, float* scale, int64_t rows, int cols, void* stream);

/* ---- lossless bf16 (LX_W_BF16X) --------------------------------------------------------------------------
 * kernels.h:574-583 (engine/cuda/bf16x.cu:1236-1295). lx_bf16x_bytes and lx_bf16x_encode synchronize the
 * stream and are load-time calls. */
LX_API int64_t lx_bf16x_row_bytes(int K);
LX_API int64_t lx_bf16x_bytes(const void* w, int64_t rows, int K, void* stream);
LX_API int lx_bf16x_encode(const void* w, int64_t rows, int K, void* out, int64_t out_bytes, void* stream);
LX_API int lx_bf16x_decode(const void* data, int64_t rows, int K, void* w, void* stream);

/* ---- mixture of experts -------------------------------------------------------------------------------- */
/* kernels.h:208 (engine/cuda/moe.cu:249, route.cuh:18-81) */
LX_API int lx_moe_route(const float* logits, const float* selection_bias, int32_t* ids, float* weights,
                        float* entropy, float* confidence, int T, int E, int top_k, void* stream);
/* The f32 GEMV of decode-sized steps that defines the router's logits: y[M, N] = x[M, K] @ w[N, K]^T + bias[N],
 * M <= 8, a row's bits independent of M; lx_router_route's logits equal it bit for bit. kernels.h:814-819
 * (engine/cuda/spec.cu:933-940). */
LX_API int lx_spec_gemv_f32(const float* x, int ld_x, const float* w, const float* bias, float* y, int ld_y, int M,
                            int N, int K, void* stream);
/* kernels.h:508, 511 (engine/cuda/moe_grouped.cu:381-388) */
LX_API int lx_moe_experts_grouped(const void* latent, const int32_t* ids, const float* weights,
                                  const lx_weight* gate_up, const lx_weight* down, lx_math math, float* out,
                                  void* workspace, int T, int L, int I, int E, int top_k, void* stream);
LX_API int64_t lx_moe_grouped_workspace_bytes(int T, int L, int I, int E, int top_k, lx_math math);
/* Few tokens (T <= 8, top_k <= 8), any stored format per stack, weight-only f32 sums, batch-invariant rows.
 * kernels.h:504-507 (engine/cuda/moe_decode.cu:397-436). BF16X stacks: both or neither (else LX_ERR_NOT_SUPPORTED). */
LX_API int lx_moe_experts_decode(const void* latent, const int32_t* ids, const float* weights,
                                 const lx_weight* gate_up, const lx_weight* down, float* out, void* workspace, int T,
                                 int L, int I, int top_k, void* stream);
LX_API int64_t lx_moe_decode_workspace_bytes(int T, int I, int top_k);
/* The same on BF16X encodings and on plain bf16 stacks, bit-identical to each other and to lx_moe_experts.
 * kernels.h:603-611 (engine/cuda/bf16x.cu:1336-1369). */
LX_API int lx_moe_experts_bf16x(const void* latent, const int32_t* ids, const float* weights, const void* gate_up,
                                const void* down, float* out, void* workspace, int T, int L, int I, int top_k,
                                void* stream);
LX_API int lx_moe_experts_decode_bf16(const void* latent, const int32_t* ids, const float* weights,
                                      const void* gate_up, const void* down, float* out, void* workspace, int T,
                                      int L, int I, int top_k, void* stream);
LX_API int64_t lx_moe_bf16x_workspace_bytes(int T, int I, int top_k);
/* bf16 stacks, any T; the intermediates live in a stream-ordered allocation for the length of the call, as in the
 * reference. kernels.h:224 (engine/cuda/moe.cu:288-310). */
LX_API int lx_moe_experts(const void* latent, const int32_t* ids, const float* weights, const void* gate_up,
                          const void* down, float* out, int T, int L, int I, int top_k, void* stream);
/* The router of a decode-sized step (M <= 8, E <= 1024, K <= 2048) in one launch: logits = x @ w^T + bias, then the
 * routing of lx_moe_route on those logits; ticket is one zeroed int32 word the call leaves at zero. kernels.h:211-218
 * (engine/cuda/moe.cu:82-157, 264-286). The routing outputs equal lx_moe_route on the returned logits bit for bit; the
 * logits are this library's own f32 sums (one warp per expert), not those of lx_spec_gemv_f32, which is outside the
 * path and not exported. */
LX_API int lx_router_route(const float* x, int ld_x, const float* w, const float* bias, float* logits,
                           const float* selection_bias, int32_t* ids, float* weights, float* entropy, float* confidence,
                           int32_t* ticket, int M, int E, int K, int top_k, void* stream);

/* ---- architecture and variant table (tunable.h:37-75, engine/cuda/tunable.cu) ---------------------------- */
typedef struct {
  int M, N, K;
  int experts;
  int weight;
  int math;
} lx_tune_problem;
LX_API int lx_arch(void);
LX_API int lx_set_arch_override(int arch);
LX_API int lx_tune_get(const char* kernel, int M, int N, int K);
LX_API int lx_tune_set(const char* kernel, int M, int N, int K, int variant);
LX_API int lx_tune_force(const char* kernel, int M, int N, int K, int variant);
LX_API void lx_tune_clear(void);
LX_API int lx_tune_kernels(const char** names, int capacity);
LX_API int lx_tune_variants(const char* kernel);
LX_API const char* lx_tune_variant_name(const char* kernel, int variant);
LX_API int lx_tune_run(const char* kernel, int variant, const lx_tune_problem* problem, float* out, void* stream);
LX_API int lx_tune_runnable(const char* kernel);
LX_API int lx_tune_key(const char* kernel, const lx_tune_problem* problem, char* out, int capacity);

/* ---- what the loader probes (kernels.h:308-309; engine/dispatch/dispatch.cpp:122-126) -------------------- */
LX_API int lx_rt_backend(void);      /* LX_BACKEND_CUDA */
LX_API int lx_rt_device_count(void);
/* kernels.h:373 (engine/cuda/bandwidth.cu:104): read-only DRAM bandwidth of the current device */
LX_API int lx_bandwidth_probe(int64_t bytes, int reps, double* read_gbps, double* spec_gbps, void* stream);

/* ---- additions of this library (no counterpart in the reference) ---------------------------------------- */
/* Kernels this library has launched in this process since it was loaded (every stream, every thread). */
LX_API int64_t lx_b200_kernel_launches(void);
/* Reads and clears the device-side status word of the current device: 0, or a code saying which bounded wait
 * inside a kernel ran out (the kernel then finished without hanging; its output is not valid).
 * Synchronizes the device. */
LX_API int lx_b200_last_error(void);
/* The shared-memory plan of the decode GEMV kernels that bring weights in with bulk copies (BF16X; INT8 / FP8 / NVFP4 on
 * rows short enough), for a weight format, K, M <= 8 and activation dtype; nothing is launched. out[0..11] = ring slots
 * (0: no such kernel for this case), whole units per stage (0 / 1), blocks per stage, stages per unit, bytes between two
 * rows of a slot, bytes of a slot, bytes between two header rows (NVFP4: where the block scales start in a slot), bytes
 * of a header slot, and the offsets of the header ring, the ring and the barriers in dynamic shared memory, and its total.
 * Returns 0, or 1 for a null pointer, K <= 0 or M outside 1..8. For tests of the layout on machines without a GPU. */
LX_API int lx_b200_gemv_ring_plan(int wtype, int K, int M, int x_is_bf16, int32_t* out);

/* A row-sharded product whose epilogue is the all-gather (no counterpart in the reference, which is single-GPU). Every
 * rank calls it with its rows of W (N rows, the columns col0 .. col0 + N - 1 of the whole y): the outputs are stored
 * straight into every rank's copy of the whole y, y_all[r] (host array of `ranks` peer-mapped device pointers to
 * [M, ld_y] buffers, this rank's own, y_all[rank], among them), and when the product is done each rank's arrival
 * semaphore, arrivals[r][0] (arrivals[r]: two int32 words, peer-mapped, zero before the first call; word 1 is used by
 * rank r's own kernels), has been increased by *arrivals_added. A consumer of
 * the whole y calls lx_b200_wait_arrivals(counter, total) on its own counter with total = the sum of every rank's
 * *arrivals_added: a counting semaphore, it waits until the counter holds `total` and takes them (arrivals of the next
 * round that come early stay), so the pair of calls can sit in a replayed graph. The wait is bounded (1 s); a timeout
 * shows in lx_b200_last_error.
 * BF16 / INT8 / FP8 weights, M within one pass (64 rows of bf16 activations); up to 8 rows of INT8 / FP8 need no
 * workspace, otherwise lx_gemm_workspace_bytes(M, K, LX_MATH_BF16). Other cases answer LX_ERR_NOT_SUPPORTED: use
 * lx_gemv_w / lx_gemm_w and a collective. y = alpha * (x W^T + bias); nothing is read from y. */
LX_API int lx_b200_linear_allgather(const void* x, lx_dtype x_dtype, int ld_x, const lx_weight* w, const void* bias,
                                    lx_dtype bias_dtype, void* const* y_all, int* const* arrivals, int ranks, int rank,
                                    int64_t col0,
                                    lx_dtype y_dtype, int ld_y, int M, int N, int K, float alpha, void* workspace,
                                    int* arrivals_added, void* stream);
LX_API int lx_b200_wait_arrivals(int* counter, int total, void* stream);
/* The all-gather of a row-sharded product's outputs as one kernel, for any product entry point (no counterpart in the
 * reference, which is single-GPU). Rank `rank` has written its slice, columns col0 .. col0 + cols - 1 of the whole
 * [M, ld_y] output, into its own buffer y_all[rank] (e.g. lx_gemv_w with y pointing at that column and ld_y as the row
 * stride); the call stores the slice into every other rank's y_all[r] (host array of `ranks` peer-mapped device pointers),
 * adds one arrival to every rank's semaphore arrivals[r][0] (arrivals[r]: two int32 words, peer-mapped, zero before the
 * first call; word 1 is rank r's own) and waits until this rank's semaphore holds `ranks` arrivals, which it takes: when
 * the kernel is done this rank's y is whole. The wait is bounded (LX_B200_WAIT_MS, default 1000); a wait that gives up
 * shows as 6 in lx_b200_last_error. Every rank must make the call once per round; callers alternate two y buffers so
 * that a rank one round ahead never overwrites what a slower rank still reads. */
LX_API int lx_b200_exchange_slices(void* const* y_all, int* const* arrivals, int ranks, int rank, int64_t col0, int cols,
                                   lx_dtype y_dtype, int ld_y, int M, void* stream);
/* The same all-gather for small slices, with the flag inside the data (no counterpart in the reference). Rank r owns
 * columns bounds[r] .. bounds[r + 1] - 1 of the [M, ld_y] output y (this rank's own buffer; ranks + 1 host integers).
 * The call sends this rank's slice as 16-byte packets {8 bytes of y, sequence, 8 bytes, sequence} into region `rank` of
 * every peer's receive buffer boxes[r] (host array of peer-mapped device pointers; each buffer is two halves of
 * ranks * region packets, zeroed once when allocated), polls the packets the peers send it and unpacks them into y: no
 * fence and no semaphore on the critical path, twice the bytes on the wire. seq and done are two zeroed words of this
 * rank's own device memory that belong to these buffers: the sequence number is kept on the device, so the call can sit
 * in a replayed graph, and its parity names the half a call uses (a rank one call ahead never overwrites packets a
 * slower rank still polls). Slice rows must be whole 8-byte pieces (else LX_ERR_NOT_SUPPORTED). The polls are bounded (LX_B200_WAIT_MS);
 * one that gives up shows as 7 in lx_b200_last_error and the next call still uses the next sequence number. */
LX_API int lx_b200_exchange_packets(void* y, void* const* boxes, int64_t region, uint32_t* seq, int* done, int ranks, int rank,
                                    const int64_t* bounds, lx_dtype y_dtype, int ld_y, int M, void* stream);

/* Routed experts split over ranks, in three calls that read nothing back on the host (no counterpart in the reference,
 * which is single-GPU). Routing and tokens are replicated: every rank calls with the same latent [T, L], ids and weights
 * [T, top_k] of ALL tokens, and holds gate_up / down stacks of its own experts own0 .. own1 - 1 only (expert own0 first).
 *   lx_b200_moe_experts_owned   rows[p, :] = weights[p] * expert(ids[p], latent[p / top_k]) for the pairs p whose expert
 *                               this rank owns (f32 [T * top_k, L], other rows untouched). Arguments, maths and errors as
 *                               lx_moe_experts_grouped, workspace of lx_moe_grouped_workspace_bytes(T, L, I, E, top_k, math);
 *                               stacks the tcgen05 expert kernels read as stored (BF16 / INT8 / FP8, one format).
 *   lx_b200_moe_exchange_rows   sends this rank's rows to every rank and receives theirs, as flag-in-data packets (see
 *                               lx_b200_exchange_packets; boxes[r]: two halves of half_packets >= T * top_k * L / 2 packets
 *                               of 16 bytes, zeroed once; seq, done: two zeroed words of this rank's memory). workspace is the one the call above
 *                               just used with the same sizes (its grouping tables say which rows are whose); bounds:
 *                               ranks + 1 expert indices, rank r owns experts bounds[r] .. bounds[r + 1] - 1. A poll that
 *                               gives up (LX_B200_WAIT_MS) shows as 8 in lx_b200_last_error.
 *   lx_b200_moe_sum_rows        out[t, :] = rows[t * top_k, :] + rows[t * top_k + 1, :] + ... in that order: the bits one
 *                               GPU with every expert gives, however the experts are split. */
LX_API int lx_b200_moe_experts_owned(const void* latent, const int32_t* ids, const float* weights, const lx_weight* gate_up,
                                     const lx_weight* down, lx_math math, float* rows, void* workspace, int T, int L, int I,
                                     int E, int own0, int own1, int top_k, void* stream);
LX_API int lx_b200_moe_exchange_rows(float* rows, const void* workspace, void* const* boxes, int64_t half_packets, uint32_t* seq,
                                     int* done, int ranks, int rank, const int* bounds, int T, int L, int I, int E, int top_k,
                                     void* stream);
LX_API int lx_b200_moe_sum_rows(const float* rows, float* out, int T, int L, int top_k, void* stream);

/* Routed experts for callers that must not allocate. No counterpart in the reference: its lx_moe_experts_grouped always
 * takes a caller workspace. Same arguments, result and error codes as lx_moe_experts_grouped above minus the workspace:
 * the scratch is a fixed 8 MiB array inside the library image, of which lx_b200_moe_static_scratch_bytes() are usable
 * (every GPU that loads the library holds the array until the process exits). A call whose scratch need,
 * lx_moe_grouped_workspace_bytes(T, L, I, E, top_k, math), exceeds that returns LX_B200_ERR_SCRATCH and launches
 * nothing. The call itself allocates nothing: no cudaMalloc, no cudaFree, no stream-ordered pool. The first call on
 * each device looks the array's device address up (cudaGetSymbolAddress, with that device current) and keeps it; make
 * that first call outside any stream capture. All calls on a device share the one array, which keeps whatever the last
 * call left in it (nothing in it needs to start at zero): calls that overlap on the GPU, on any streams, race on it and
 * are the caller's to serialize. A bounded wait that gives up inside this call shows in lx_b200_last_error() like any
 * other. */
#define LX_B200_ERR_SCRATCH 804
LX_API int lx_b200_moe_experts_grouped_static(const void* latent, const int32_t* ids, const float* weights,
                                              const lx_weight* gate_up, const lx_weight* down, lx_math math, float* out,
                                              int T, int L, int I, int E, int top_k, void* stream);
LX_API int64_t lx_b200_moe_static_scratch_bytes(void);
/* The device address of that array on the current device (null if the lookup fails). Its first 256 bytes are a header:
 * word 0 is the status word this entry point's kernels write when one of their bounded waits gives up;
 * lx_b200_last_error() reads and clears it together with the library's own status word. */
LX_API void* lx_b200_moe_static_scratch_ptr(void);

#ifdef __cplusplus
}
#endif
