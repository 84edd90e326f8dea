// The kernels that have alternatives and the names of their variants (the registry behind lx_tune_kernels,
// lx_tune_variants and lx_tune_variant_name). A decode GEMV variant is "s<ring stages>r<rows per tile>u<64-byte steps
// per warp per stage>[w<consumer warps, 8 when absent>]"; index 0 is what runs when the table holds nothing for a shape.
#pragma once

namespace b200 {

struct VariantList {
  const char* kernel;
  int count;
  const char* const* names;
};

constexpr int kGemvVariants = 14;
inline const char* const kGemvVariantNames[kGemvVariants] = {"s4r32u2", "s8r32u2", "s4r32u4", "s4r64u2w16", "s6r16u1", "s6r32u1w16",
                                                                "s4r16u4", "s4r32u2w16", "s5r32u2w16", "s3r64u4w16",
                                                                "s6r32u4x8", "s6r32u2w16x8", "s12r32u2x8", "s6r64u2w16x8"};

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
