#include "gemm_tc.h"

namespace pcpb {
bool gemm_tc_supported(const GemmArgs&) { return false; }
int gemm_tc_launches(const GemmArgs&) { return 1; }
cudaError_t launch_gemm_tc(cudaStream_t, const GemmArgs&) { return cudaErrorNotSupported; }
}  // namespace pcpb
