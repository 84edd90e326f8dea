// The lossless bf16 encoding LX_W_BF16X: size query, encoder and decoder (the ABI of lernex/dromos
// engine/cuda/kernels.h:574-583; the layout is documented in engine/cuda/bf16x.cuh:13-28 and restated in stream.cuh).
//
// Encoding a row: per 128 values the largest exponent is the block's base; a value keeps sign|mantissa in one byte and
// base - exponent as a 4-bit code; a value more than 15 binades below its base is a patch (position << 8 | exponent),
// listed in ascending position in the row's header slots, or in an overflow record after all rows when the row has
// more patches than slots. Rows are independent except for where their overflow records land, which is fixed by
// a prefix sum over the rows' record sizes in row order, so the bytes never depend on scheduling.
#include <algorithm>

#include "launch.cuh"

namespace b200 {
namespace {

constexpr int kBlock = 256;
constexpr int kWarpsPerBlock = kBlock / 32;

__host__ __device__ inline int64_t record_bytes(int64_t patches) { return (4 * (patches + 2) + 7) / 8 * 8; }

// One warp per row: the row's number of patches.
__global__ void __launch_bounds__(kBlock) count_kernel(const uint16_t* __restrict__ w, int64_t rows, int K,
                                                       int32_t* __restrict__ counts) {
  // no early trigger: what this kernel writes may be the weight of the next product, whose kernels read weights
  // before their own wait
  pdl_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint16_t* src = w + row * K;
  int n = 0;
  for (int k0 = 0; k0 < K; k0 += 128) {
    int e[4], base = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + 32 * i + lane;
      e[i] = k < K ? (src[k] >> 7) & 0xff : -1;
      base = max(base, e[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) base = max(base, __shfl_xor_sync(0xffffffffu, base, o));
#pragma unroll
    for (int i = 0; i < 4; ++i) n += e[i] >= 0 && base - e[i] > 15;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
  if (lane == 0) counts[row] = n;
}

// One CTA: offsets[r] = bytes of overflow records of rows before r (exclusive prefix in row order), total at [rows].
__global__ void __launch_bounds__(1024) scan_kernel(const int32_t* __restrict__ counts, int64_t rows, int slots,
                                                    int64_t* __restrict__ offsets) {
  // no early trigger: what this kernel writes may be the weight of the next product, whose kernels read weights
  // before their own wait
  pdl_wait();
  __shared__ int64_t part[1024];
  const int t = threadIdx.x;
  const int64_t per = (rows + 1023) / 1024;
  const int64_t r0 = min(rows, t * per), r1 = min(rows, r0 + per);
  int64_t sum = 0;
  for (int64_t r = r0; r < r1; ++r) sum += counts[r] > slots ? record_bytes(counts[r]) : 0;
  part[t] = sum;
  __syncthreads();
  if (t == 0) {
    int64_t run = 0;
    for (int i = 0; i < 1024; ++i) {
      const int64_t v = part[i];
      part[i] = run;
      run += v;
    }
    offsets[rows] = run;
  }
  __syncthreads();
  int64_t run = part[t];
  for (int64_t r = r0; r < r1; ++r) {
    offsets[r] = run;
    run += counts[r] > slots ? record_bytes(counts[r]) : 0;
  }
}

// One warp per row: writes the row's record and, for a row with more patches than slots, its overflow record.
__global__ void __launch_bounds__(kBlock) encode_kernel(const uint16_t* __restrict__ w, int64_t rows, int K,
                                                        const int32_t* __restrict__ counts,
                                                        const int64_t* __restrict__ offsets, uint8_t* __restrict__ out) {
  // no early trigger: what this kernel writes may be the weight of the next product, whose kernels read weights
  // before their own wait
  pdl_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int H = x16::header_bytes(K), P = x16::patch_slots(K), B = x16::blocks(K);
  const int64_t rb = x16::row_bytes(K);
  const uint16_t* src = w + row * K;
  uint8_t* rec = out + row * rb;
  uint32_t* slots = reinterpret_cast<uint32_t*>(rec);
  // header: empty slots, zero padding after the base bytes
  for (int i = lane; i < P; i += 32) slots[i] = x16::kNoPatch;
  for (int i = 4 * P + B + lane; i < H; i += 32) rec[i] = 0;
  const int n_patches = counts[row];
  uint32_t* list = slots;
  if (n_patches > P) {
    const int64_t at = rows * rb + offsets[row] - row * rb;  // from the row's own start, in bytes
    uint32_t* r = reinterpret_cast<uint32_t*>(rec + at);
    const int64_t words = record_bytes(n_patches) / 4;
    for (int64_t i = n_patches + 1 + lane; i < words; i += 32) r[i] = 0;  // padding after the terminator
    __syncwarp();
    if (lane == 0) {
      slots[0] = 0x80000000u | static_cast<uint32_t>(at / 8);
      r[0] = static_cast<uint32_t>(n_patches);
      r[n_patches + 1] = x16::kNoPatch;
    }
    list = r + 1;
  }
  __syncwarp();
  int placed = 0;  // patches written so far (the same in every lane)
  for (int b = 0; b < B; ++b) {
    const int k0 = 128 * b;
    uint8_t* blk = rec + H + static_cast<int64_t>(b) * 192;
    int v[4], e[4], base = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + 32 * i + lane;
      v[i] = k < K ? src[k] : -1;
      e[i] = v[i] >= 0 ? (v[i] >> 7) & 0xff : 0;
      base = max(base, e[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) base = max(base, __shfl_xor_sync(0xffffffffu, base, o));
    if (lane == 0) rec[4 * P + b] = static_cast<uint8_t>(base);
    uint32_t code[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool live = v[i] >= 0;
      blk[32 * i + lane] = live ? static_cast<uint8_t>(((v[i] >> 8) & 0x80) | (v[i] & 0x7f)) : 0;
      const int d = base - e[i];
      const bool patched = live && d > 15;
      const uint32_t mask = __ballot_sync(0xffffffffu, patched);
      if (patched) list[placed + __popc(mask & ((1u << lane) - 1))] = (static_cast<uint32_t>(k0 + 32 * i + lane) << 8) | e[i];
      placed += __popc(mask);
      code[i] = live && !patched ? d : 0;
    }
    // Code bytes: word g covers values 8g .. 8g + 7, its byte j holding value 8g + j low and 8g + 4 + j high. Value
    // 32 i + lane sits in word 4 i + lane / 8; lanes with (lane & 4) == 0 own a byte and fetch its high nibble from
    // the lane four above.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t hi = __shfl_down_sync(0xffffffffu, code[i], 4);
      if ((lane & 4) == 0) blk[128 + 4 * (4 * i + (lane >> 3)) + (lane & 3)] = static_cast<uint8_t>(code[i] | (hi << 4));
    }
  }
}

// One warp per row: every value from its byte, code and base, then the row's patches over them.
__global__ void __launch_bounds__(kBlock) decode_kernel(const uint8_t* __restrict__ data, int64_t rows, int K,
                                                        uint16_t* __restrict__ w) {
  // no early trigger: what this kernel writes may be the weight of the next product, whose kernels read weights
  // before their own wait
  pdl_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int H = x16::header_bytes(K), P = x16::patch_slots(K);
  const uint8_t* rec = data + row * x16::row_bytes(K);
  uint16_t* dst = w + row * K;
  for (int k = lane; k < K; k += 32) {
    const int b = k >> 7, off = k & 127;
    const uint8_t* blk = rec + H + static_cast<int64_t>(b) * 192;
    const uint32_t sm = blk[off];
    const uint32_t cb = blk[128 + (off >> 3) * 4 + (off & 3)];
    const uint32_t e = (rec[4 * P + b] - ((off & 4) ? cb >> 4 : cb & 15u)) & 0xffu;
    dst[k] = static_cast<uint16_t>(((sm & 0x80u) << 8) | (e << 7) | (sm & 0x7fu));
  }
  __syncwarp();
  const uint32_t* list = reinterpret_cast<const uint32_t*>(rec);
  int n = P;
  const uint32_t s0 = list[0];
  if (s0 != x16::kNoPatch && (s0 & 0x80000000u)) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(rec + static_cast<int64_t>(s0 & 0x7fffffffu) * 8);
    n = static_cast<int>(r[0]);
    list = r + 1;
  }
  for (int i = lane; i < n; i += 32) {
    const uint32_t p = list[i];
    if (p == x16::kNoPatch) continue;
    const uint32_t k = p >> 8;
    if (k < static_cast<uint32_t>(K)) dst[k] = static_cast<uint16_t>((dst[k] & 0x807fu) | ((p & 0xffu) << 7));
  }
}

// Runs the counting passes into stream-ordered scratch. On success *counts and *offsets are live device buffers the
// caller frees with cudaFreeAsync; *area is the total size of the overflow records. Synchronizes the stream.
int plan(const void* w, int64_t rows, int K, cudaStream_t s, int32_t** counts, int64_t** offsets, int64_t* area) {
  *counts = nullptr;
  *offsets = nullptr;
  if (cudaMallocAsync(counts, sizeof(int32_t) * rows, s) != cudaSuccess) return static_cast<int>(cudaGetLastError());
  if (cudaMallocAsync(offsets, sizeof(int64_t) * (rows + 1), s) != cudaSuccess) {
    const int e = static_cast<int>(cudaGetLastError());
    cudaFreeAsync(*counts, s);
    return e;
  }
  int e = launch_kernel(count_kernel, dim3(static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock)), dim3(kBlock),
                        0, s, static_cast<const uint16_t*>(w), rows, K, *counts);
  if (!e) e = launch_kernel(scan_kernel, dim3(1), dim3(1024), 0, s, static_cast<const int32_t*>(*counts), rows,
                            x16::patch_slots(K), *offsets);
  if (!e) e = static_cast<int>(cudaMemcpyAsync(area, *offsets + rows, sizeof(int64_t), cudaMemcpyDeviceToHost, s));
  if (!e) e = static_cast<int>(cudaStreamSynchronize(s));
  if (e) {
    cudaFreeAsync(*counts, s);
    cudaFreeAsync(*offsets, s);
  }
  return e;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int64_t lx_bf16x_row_bytes(int K) { return K > 0 && K < (1 << 23) ? x16::row_bytes(K) : -1; }

extern "C" int64_t lx_bf16x_bytes(const void* w, int64_t rows, int K, void* stream) {
  if (rows <= 0 || K <= 0 || K >= (1 << 23) || !w) return -static_cast<int64_t>(kInvalid);
  auto s = static_cast<cudaStream_t>(stream);
  int32_t* counts;
  int64_t* offsets;
  int64_t area = 0;
  if (const int e = plan(w, rows, K, s, &counts, &offsets, &area)) return -static_cast<int64_t>(e);
  cudaFreeAsync(counts, s);
  cudaFreeAsync(offsets, s);
  return rows * x16::row_bytes(K) + area;
}

extern "C" int lx_bf16x_encode(const void* w, int64_t rows, int K, void* out, int64_t out_bytes, void* stream) {
  if (rows <= 0) return kOk;
  const int64_t rb = K > 0 && K < (1 << 23) ? x16::row_bytes(K) : 0;
  if (!rb || !w || !out || !aligned(out, 8) || out_bytes < rows * rb) return kInvalid;
  auto s = static_cast<cudaStream_t>(stream);
  int32_t* counts;
  int64_t* offsets;
  int64_t area = 0;
  if (const int e = plan(w, rows, K, s, &counts, &offsets, &area)) return e;
  int e = rows * rb + area > out_bytes ? kInvalid : kOk;
  if (!e)
    e = launch_kernel(encode_kernel, dim3(static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock)), dim3(kBlock), 0,
                      s, static_cast<const uint16_t*>(w), rows, K, static_cast<const int32_t*>(counts),
                      static_cast<const int64_t*>(offsets), static_cast<uint8_t*>(out));
  cudaFreeAsync(counts, s);
  cudaFreeAsync(offsets, s);
  return e;
}

extern "C" int lx_bf16x_decode(const void* data, int64_t rows, int K, void* w, void* stream) {
  if (rows <= 0) return kOk;
  if (K <= 0 || K >= (1 << 23) || !data || !w) return kInvalid;
  return launch_kernel(decode_kernel, dim3(static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock)), dim3(kBlock), 0,
                       static_cast<cudaStream_t>(stream), static_cast<const uint8_t*>(data), rows, K,
                       static_cast<uint16_t*>(w));
}
