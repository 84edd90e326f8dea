// The kernels that have alternatives and the names of their variants (the registry behind lx_tune_kernels,
// lx_tune_variants and lx_tune_variant_name). The five decode GEMV kernels (one per weight format) share one list:
//   d4c2   the decode GEMV of gemv.cuh, two CTAs per SM, 64 bytes per row in flight per lane
//   d8c1   the same kernel, one CTA per SM, 128 bytes in flight; both add a row's products in the same order (same bits)
//   ring   the TMA-ring mma.sync kernel of stream.cuh       another order: lx_tune_set refuses it, lx_tune_force takes it
//   tc     the tcgen05 product (INT8 / FP8, wide weights)   another order again
// What runs when the table holds nothing for a shape: d4c2 when two CTAs' activation columns fit an SM, else d8c1
// (BF16X: always d8c1, it needs the registers).
#pragma once

#include <cstring>

namespace b200 {

struct VariantList {
  const char* kernel;
  int count;
  const char* const* names;
};

enum GemvVariant { kGemvD4C2 = 0, kGemvD8C1 = 1, kGemvRing = 2, kGemvTc = 3, kGemvVariants = 4 };
inline const char* const kGemvVariantNames[kGemvVariants] = {"d4c2", "d8c1", "ring", "tc"};
// Variants of one class add a row's products in the same order (same bits).
inline int gemv_order_class(int variant) { return variant == kGemvRing ? 1 : variant == kGemvTc ? 2 : 0; }

constexpr int kVariantKernels = 5;
inline const VariantList kVariantTable[kVariantKernels] = {
    {"gemv_w_bf16", kGemvVariants, kGemvVariantNames},  {"gemv_w_int8", kGemvVariants, kGemvVariantNames},
    {"gemv_w_fp8", kGemvVariants, kGemvVariantNames},   {"gemv_w_nvfp4", kGemvVariants, kGemvVariantNames},
    {"gemv_bf16x", kGemvVariants, kGemvVariantNames},
};

inline const char* gemv_kernel_name(int wtype) {
  return wtype >= 0 && wtype < kVariantKernels ? kVariantTable[wtype].kernel : nullptr;
}
inline int gemv_kernel_wtype(const char* name) {
  for (int i = 0; i < kVariantKernels; ++i)
    if (name && std::strcmp(kVariantTable[i].kernel, name) == 0) return i;
  return -1;
}

}  // namespace b200
