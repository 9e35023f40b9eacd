// Grouped GEMMs of the w4a8_mx and w4a16 recipes.
#include "common.cuh"

namespace b200moe {
int mx_gemm1(const b200moe_gemm_args*, cudaStream_t) { return B200MOE_EUNSUPPORTED; }
int mx_gemm2(const b200moe_gemm_args*, cudaStream_t) { return B200MOE_EUNSUPPORTED; }
int w4a16_gemm1(const b200moe_gemm_args*, cudaStream_t) { return B200MOE_EUNSUPPORTED; }
int w4a16_gemm2(const b200moe_gemm_args*, cudaStream_t) { return B200MOE_EUNSUPPORTED; }
}  // namespace b200moe
