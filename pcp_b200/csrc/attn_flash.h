// Tiled causal attention (bf16, head_dim 128, 64, 32 or 16), forward and backward.
#pragma once
#include <cuda_runtime.h>

namespace pcpb {

struct FlashArgs {
  const void* qkn;      // [B*T, d + dkv]   normalised roped q then k
  const void* qkv;      // [B*T, d + 2 dkv] raw projections (v part is read)
  void* o;              // [B*T, d]
  float* mrow;          // [B*H*T] row max of the scaled masked scores
  float* lrow;          // [B*H*T] row sum of exp(s - max)
  int B, T, H, Hkv, hd;
  float scale;          // 1/sqrt(hd) rounded to bf16
  int no_guard;         // forward only: 1 = plain softmax, p = e / l (generation graphs are not sanitised);
                        // 0 = the training graphs' p = e / (l + 1e-4)
  // backward
  const void* dout;     // [B*T, d]
  void* dqkn;           // [B*T, d + dkv]   gradient wrt qkn (q and k parts written)
  void* dqkv;           // [B*T, d + 2 dkv] (v part written)
  float* drow;          // [B*H*T] scratch: rowsum(do*o) scaled
  float4* stat4;        // [B*H*T] scratch: (max, 1/(l+1e-4), 1/(l+2e-4), D) per query row, written by the prep kernel
};

bool flash_supported(const FlashArgs& a);
cudaError_t launch_flash_fwd(cudaStream_t st, const FlashArgs& a);
cudaError_t launch_flash_bwd(cudaStream_t st, const FlashArgs& a);      // 3 kernels

}  // namespace pcpb
