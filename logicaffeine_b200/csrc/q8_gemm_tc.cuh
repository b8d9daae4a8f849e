// Interface of the tcgen05 Q8 GEMM kernel (q8_gemm_tc.cu).
#pragma once
#include "ops.cuh"

namespace logos {
logos_status_t launch_q8_gemm_tc(const GemmArgs& g, cudaStream_t st);
logos_status_t launch_splitk_reduce(const float* partials, int splits, void* c, int c_dtype, ActOut c_act,
                                    int64_t ldc, const void* aux, int64_t m, int64_t n, int epilogue,
                                    cudaStream_t st);
void gemm_set_trace(long long* buf);
}  // namespace logos
