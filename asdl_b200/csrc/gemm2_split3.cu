// The "split3" flavour of the persistent tcgen05 GEMM (see umma_gemm2.cuh), in a translation
// unit of its own so that the flavours compile in parallel.
#include <algorithm>

#include "gemm2_host.h"

namespace b200 {

void g2_run_split3(const GemmProblem2& single, const GemmProblem2* probs, const GemmWork2* work, int n_work,
                  int n_sms, cudaStream_t stream, const int* prefix, int n_probs) {
  if (n_work <= 0) return;
  static bool attr_set_on[64] = {false};
  int dev = 0;
  B200_CUDA_CHECK(cudaGetDevice(&dev));
  bool& attr_set = attr_set_on[dev & 63];
  if (!attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(umma_gemm2_kernel<128, 8, 1, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         G2Split3::SMEM_BYTES));
    attr_set = true;
  }
  const int grid = std::min(n_work, 1 * n_sms);
  umma_gemm2_kernel<128, 8, 1, 3><<<grid, G2Split3::THREADS, G2Split3::SMEM_BYTES, stream>>>(single, probs, work, n_work, prefix, n_probs);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

}  // namespace b200
