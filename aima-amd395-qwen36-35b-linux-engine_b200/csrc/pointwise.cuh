// Launchers of the row-wise helpers (see pointwise.cu).
#pragma once

#include "common.cuh"

namespace aima {

cudaError_t launch_rmsnorm_rows(const void* x, const void* residual,
                                const void* weight, void* residual_out,
                                void* norm_out, int rows, float eps,
                                cudaStream_t stream);

cudaError_t launch_gemv_bf16(const void* weight, const void* x, void* out,
                             int m, int k, cudaStream_t stream);

}  // namespace aima
