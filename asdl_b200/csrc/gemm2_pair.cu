// The CTA-pair flavour of the persistent tcgen05 GEMM (see umma_gemm2_pair.cuh), in a translation
// unit of its own so that the flavours compile in parallel.
#include <algorithm>

#include "gemm2_host.h"
#include "umma_gemm2_pair.cuh"

namespace b200 {

int g2_pair_tiles(const GemmProblem2& P) {
  const int T = (P.tiles_m + 1) / 2;
  return (P.flags & G2F_SYM) ? T * (T + 1) / 2 : T * P.tiles_n;
}

void g2_run_pair(const GemmProblem2& single, int n_work, int n_sms, cudaStream_t stream) {
  if (n_work <= 0) return;
  static bool attr_set_on[64] = {false};
  int dev = 0;
  B200_CUDA_CHECK(cudaGetDevice(&dev));
  bool& attr_set = attr_set_on[dev & 63];
  if (!attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(umma_gemm2_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         G2P_SMEM_BYTES));
    attr_set = true;
  }
  const int pairs = std::max(1, std::min(n_work, n_sms / 2));
  umma_gemm2_pair_kernel<<<2 * pairs, G2P_THREADS, G2P_SMEM_BYTES, stream>>>(single, n_work);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

}  // namespace b200
