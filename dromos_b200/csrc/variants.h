// The kernels that have alternatives and the names of their variants (the registry behind lx_tune_kernels,
// lx_tune_variants and lx_tune_variant_name). A decode GEMV variant is "s<ring stages>r<rows per CTA>u<64-byte steps
// per warp per stage>"; index 0 is what runs when the table holds nothing for a shape.
#pragma once

namespace b200 {

struct VariantList {
  const char* kernel;
  int count;
  const char* const* names;
};

constexpr int kGemvVariants = 8;
inline const char* const kGemvVariantNames[kGemvVariants] = {"s4r32u2", "s4r16u1", "s3r32u4", "s3r64u4",
                                                                "s6r32u2", "s8r16u1", "s4r64u2", "s6r16u2"};

constexpr int kVariantKernels = 5;
inline const VariantList kVariantTable[kVariantKernels] = {
    {"gemv_w_bf16", kGemvVariants, kGemvVariantNames},  {"gemv_w_int8", kGemvVariants, kGemvVariantNames},
    {"gemv_w_fp8", kGemvVariants, kGemvVariantNames},   {"gemv_w_nvfp4", kGemvVariants, kGemvVariantNames},
    {"gemv_bf16x", kGemvVariants, kGemvVariantNames},
};

inline const char* gemv_kernel_name(int wtype) {
  return wtype >= 0 && wtype < kVariantKernels ? kVariantTable[wtype].kernel : nullptr;
}

}  // namespace b200
