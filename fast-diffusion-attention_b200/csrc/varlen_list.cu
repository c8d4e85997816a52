// Device-side preparation of the varlen work list (see varlen_list.cuh).
#include "varlen_list.cuh"

#include "host_util.h"

namespace fda {

__global__ void __launch_bounds__(256) varlen_prepare_kernel(const int32_t* __restrict__ cu_seqlens, int batch,
                                                             int unit_rows, int* out) {
  int* order = out + 1;
  int* cum = out + 1 + batch;
  // rank of a sample = number of samples that come before it: longer ones, and equally long ones with a smaller
  // index (a stable order, so the list is a pure function of cu_seqlens)
  for (int i = threadIdx.x; i < batch; i += blockDim.x) {
    const int ni = cu_seqlens[i + 1] - cu_seqlens[i];
    int rank = 0;
    for (int j = 0; j < batch; ++j) {
      const int nj = cu_seqlens[j + 1] - cu_seqlens[j];
      rank += (nj > ni || (nj == ni && j < i)) ? 1 : 0;
    }
    order[rank] = i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int sum = 0;
    for (int v = 0; v < batch; ++v) {
      cum[v] = sum;
      const int b = order[v];
      const int n = (cu_seqlens[b + 1] - cu_seqlens[b]) / 2;
      sum += (n + unit_rows - 1) / unit_rows;
    }
    cum[batch] = sum;
    out[0] = sum;
  }
}

int launch_varlen_prepare(const int32_t* cu_seqlens, int batch, int unit_rows, int* out, void* stream) {
  varlen_prepare_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(cu_seqlens, batch, unit_rows, out);
  FDA_CUDA_TRY(cudaGetLastError());
  return FDA_OK;
}

}  // namespace fda
