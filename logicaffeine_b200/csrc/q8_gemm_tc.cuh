// Interface of the tcgen05 Q8 GEMM kernel (q8_gemm_tc.cu).
#pragma once
#include "ops.cuh"
#include "ptx.cuh"

namespace logos {
logos_status_t launch_q8_gemm_tc(const GemmArgs& g, cudaStream_t st);
logos_status_t launch_splitk_reduce(const float* partials, int splits, void* c, int c_dtype, ActOut c_act,
                                    int64_t ldc, const void* aux, int64_t m, int64_t n, int epilogue,
                                    cudaStream_t st);
void gemm_set_trace(long long* buf);
// Encoded tensor maps, cached by (address, shape, box): d2 == 0 asks for a 2-D map [d1][d0] with the
// given swizzle; otherwise a 3-D map [d2][d1][d0], box depth 1, no swizzle.
logos_status_t cached_map(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint32_t elem, uint64_t d0,
                          uint64_t d1, uint64_t pitch1, uint32_t box0, uint32_t box1,
                          CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, uint64_t d2 = 0, uint64_t pitch2 = 0);
}  // namespace logos
