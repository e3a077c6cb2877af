// Tensor-core GEMM path (tcgen05 + TMEM accumulators, TMA-fed) for bf16 operands.
#pragma once
#include <cuda_runtime.h>

#include "kernels.h"

namespace pcpb {

// True when launch_gemm_tc can run this problem (bf16 operands, shapes and strides the tiled kernel
// supports).  The caller falls back to the generic kernel otherwise.
bool gemm_tc_supported(const GemmArgs& g);
// Number of kernel launches launch_gemm_tc enqueues for this problem.
int gemm_tc_launches(const GemmArgs& g);
cudaError_t launch_gemm_tc(cudaStream_t st, const GemmArgs& g);
// Scratch bytes a weight-gradient GEMM of this shape would like for its split-K slabs (0 = none).
size_t gemm_tc_scratch_wanted(int M, int N, int K);

}  // namespace pcpb
