// Backward pass (placeholder until the kernels land).
#include "host_util.h"
#include "ptx.cuh"

namespace fda {
size_t bwd_workspace_bytes(const FdaProblem& p) { (void)p; return 256; }
int launch_bwd(const FdaBwdArgs& a, cudaStream_t stream) { (void)a; (void)stream; return FDA_ERR_UNSUPPORTED; }
int read_status_bwd(int32_t* out4) {
  int zero[4] = {0, 0, 0, 0};
  FDA_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_fda_status, sizeof(int) * 4));
  FDA_CUDA_TRY(cudaMemcpyToSymbol(g_fda_status, zero, sizeof(int) * 4));
  return FDA_OK;
}
}  // namespace fda
