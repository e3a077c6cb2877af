// Causal attention on tcgen05 / tensor memory (bf16, head_dim 128).  Same arguments as the mma.sync kernels.
#pragma once
#include <cuda_runtime.h>

#include "attn_flash.h"

namespace pcpb {

bool attn_tc_supported(const FlashArgs& a);
// err_word: device int that receives a non-zero role code when a bounded wait expires.
cudaError_t launch_attn_tc_fwd(cudaStream_t st, const FlashArgs& a, int* err_word);   // 1 kernel
cudaError_t launch_attn_tc_bwd(cudaStream_t st, const FlashArgs& a, int* err_word);   // 3 kernels

}  // namespace pcpb
