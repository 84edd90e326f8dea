// The kernels that have alternatives and the names of their variants (the registry behind lx_tune_kernels,
// lx_tune_variants and lx_tune_variant_name).
//
// The four decode GEMV kernels of the quantized and plain formats share one list. As in the reference, a name starts
// with "s<split>", the number of K slices a row's products are added in: variants with the same split add in the same
// order and give the same bits.
//   s16d4c2  the decode GEMV of gemv.cuh, two CTAs per SM, 64 bytes per row in flight per lane
//   s16d8c1  the same kernel, one CTA per SM, 128 bytes in flight
//   s8ring   the TMA-ring mma.sync kernel of stream.cuh     another order: lx_tune_set refuses it, lx_tune_force takes it
//   s1tc     the tcgen05 product (INT8 / FP8, wide weights) another order again
//   s16d1c1  one CTA per SM, units brought into shared memory by bulk copies (gemv_ring8.cuh: INT8 / FP8 rows short enough
//            for two units to fit; gemv_x16.cuh: the lossless format); the decode GEMV's sums. Named for a weight it does
//            not take, it is the default.
// "gemv_bf16x" lists only forms of the decode GEMV, without a split: its variants are the format's own, change no sum and
// are admitted at every key (the kernel must keep the bits of the bf16 kernel's default): d4c2 and d8c1 as above, and
//   d1c1     the format's own kernel (gemv_x16.cuh): one CTA per SM, records brought into shared memory by bulk copies
// What runs when the table holds nothing for a shape: d4c2 when two CTAs' activation columns fit an SM, else d8c1
// (BF16X: d1c1).
//
// "gemm_w.<kind>.sm100" are the families of lx_gemm_w by operand kind (the reference's names, engine/cuda/gemm_w.cu):
// each has the one tile shape of the tcgen05 product, rows of W split evenly over the SMs, so there is nothing to pick.
#pragma once

#include <cstring>

namespace b200 {

struct VariantList {
  const char* kernel;
  int count;
  const char* const* names;
};

enum GemvVariant { kGemvD4C2 = 0, kGemvD8C1 = 1, kGemvRing = 2, kGemvTc = 3, kGemvX16Pipe = 4, kGemvVariants = 5 };
inline const char* const kGemvVariantNames[kGemvVariants] = {"s16d4c2", "s16d8c1", "s8ring", "s1tc", "s16d1c1"};
constexpr int kX16Variants = 3;
inline const char* const kX16VariantNames[kX16Variants] = {"d4c2", "d8c1", "d1c1"};
// The lossless kernel's third entry is its own kernel, not the ring: an index of its list as a GemvVariant.
inline int x16_variant(int index) { return index == 2 ? kGemvX16Pipe : index; }
inline const char* const kGemmWVariantNames[1] = {"rows128"};
// Variants of one class add a row's products in the same order (same bits).
inline int gemv_order_class(int variant) { return variant == kGemvRing ? 1 : variant == kGemvTc ? 2 : 0; }

constexpr int kGemvKernels = 5;  // the first entries of the table, indexed by lx_wtype
constexpr int kVariantKernels = 11;
inline const VariantList kVariantTable[kVariantKernels] = {
    {"gemv_w_bf16", kGemvVariants, kGemvVariantNames},  {"gemv_w_int8", kGemvVariants, kGemvVariantNames},
    {"gemv_w_fp8", kGemvVariants, kGemvVariantNames},   {"gemv_w_nvfp4", kGemvVariants, kGemvVariantNames},
    {"gemv_bf16x", kX16Variants, kX16VariantNames},
    {"gemm_w.bf16.sm100", 1, kGemmWVariantNames},  {"gemm_w.w8i8.sm100", 1, kGemmWVariantNames},
    {"gemm_w.w8f8.sm100", 1, kGemmWVariantNames},  {"gemm_w.w4a16.sm100", 1, kGemmWVariantNames},
    {"gemm_w.i8.sm100", 1, kGemmWVariantNames},    {"gemm_w.f8.sm100", 1, kGemmWVariantNames},
};

inline const char* gemv_kernel_name(int wtype) {
  return wtype >= 0 && wtype < kGemvKernels ? kVariantTable[wtype].kernel : nullptr;
}
inline int gemv_kernel_wtype(const char* name) {
  for (int i = 0; i < kGemvKernels; ++i)
    if (name && std::strcmp(kVariantTable[i].kernel, name) == 0) return i;
  return -1;
}
// A variant's index by any of its names ("s16d4c2" or "d4c2"), -1 when there is none.
inline int gemv_variant_by_name(const char* name) {
  for (int i = 0; i < kGemvVariants; ++i) {
    const char* full = kGemvVariantNames[i];
    const char* bare = full + std::strspn(full, "s0123456789");
    if (name && (std::strcmp(full, name) == 0 || std::strcmp(bare, name) == 0)) return i;
  }
  return -1;
}

}  // namespace b200
