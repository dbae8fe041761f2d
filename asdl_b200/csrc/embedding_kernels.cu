// Statistics of an embedding layer without a sort or a bincount: tokens scatter their contribution
// with reductions (red.global.add), one warp per token row.
//   embedding_diag_stats   diag[idx[t], :] += scale * g[t, :]^2      (diagonal Fisher of the table)
//   embedding_counts       counts[example, idx] += 1                 (rows of the one-hot input sum;
//                          the input-side Kronecker factor is counts^T counts, formed by the SYRK)
// Stands in for the per-example bincount and the Python loop over tokens of
// asdl/operations/embedding.py:12-46.
#include "host_utils.h"

namespace b200 {

namespace {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(256)
embedding_diag_kernel(const int64_t* __restrict__ idx, const T* __restrict__ g, float* __restrict__ out, int64_t tokens,
                      int dim, int64_t ld_g, int64_t vocab, int64_t padding_idx, float scale) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); t < tokens;
       t += static_cast<int64_t>(gridDim.x) * warps_per_block) {
    const int64_t row = idx[t];
    if (row < 0 || row >= vocab || row == padding_idx) continue;   // an index outside the table contributes nothing
    const T* src = g + t * ld_g;
    float* dst = out + row * dim;
    for (int c = lane; c < dim; c += 32) {
      const float v = to_f32<T>(src[c]);
      atomicAdd(dst + c, scale * v * v);
    }
  }
}

__global__ void __launch_bounds__(256)
embedding_counts_kernel(const int64_t* __restrict__ idx, float* __restrict__ counts, int64_t examples, int64_t per_example,
                        int64_t vocab) {
  const int64_t total = examples * per_example;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = idx[e];
    if (row < 0 || row >= vocab) continue;
    atomicAdd(counts + (e / per_example) * vocab + row, 1.f);
  }
}

}  // namespace

// out[vocab, dim] (fp32, contiguous) += scale * g^2 scattered by idx; idx: int64 [tokens], g: [tokens, dim] fp32 / bf16.
void embedding_diag_stats(at::Tensor idx, at::Tensor g, at::Tensor out, int64_t padding_idx, double scale) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.dim() == 1 && idx.is_contiguous(), "idx must be a contiguous int64 CUDA vector");
  TORCH_CHECK(g.is_cuda() && g.dim() == 2 && g.stride(1) == 1 && g.size(0) == idx.size(0) &&
                  (g.scalar_type() == at::kFloat || g.scalar_type() == at::kBFloat16),
              "g must be a [tokens, dim] fp32 / bf16 CUDA matrix with unit column stride");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.dim() == 2 && out.is_contiguous() && out.size(1) == g.size(1),
              "out must be a contiguous fp32 [vocab, dim] CUDA matrix");
  const int64_t tokens = idx.size(0);
  if (tokens == 0 || g.size(1) == 0) return;
  const int dev = g.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  const int blocks = static_cast<int>(std::min<int64_t>((tokens + 7) / 8, 4 * 148));
  if (g.scalar_type() == at::kFloat)
    embedding_diag_kernel<float><<<blocks, 256, 0, stream>>>(idx.data_ptr<int64_t>(), g.data_ptr<float>(), out.data_ptr<float>(),
                                                            tokens, static_cast<int>(g.size(1)), g.stride(0), out.size(0), padding_idx,
                                                            static_cast<float>(scale));
  else
    embedding_diag_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        idx.data_ptr<int64_t>(), reinterpret_cast<const __nv_bfloat16*>(g.data_ptr()), out.data_ptr<float>(), tokens,
        static_cast<int>(g.size(1)), g.stride(0), out.size(0), padding_idx, static_cast<float>(scale));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// counts[examples, vocab] (fp32, contiguous) += number of occurrences of every index per example; idx: int64 [examples, per_example].
void embedding_counts(at::Tensor idx, at::Tensor counts) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.dim() == 2 && idx.is_contiguous(), "idx must be a contiguous int64 [examples, tokens] CUDA matrix");
  TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kFloat && counts.dim() == 2 && counts.is_contiguous() &&
                  counts.size(0) == idx.size(0),
              "counts must be a contiguous fp32 [examples, vocab] CUDA matrix");
  const int64_t total = idx.numel();
  if (total == 0) return;
  const int dev = idx.get_device();
  c10::cuda::CUDAGuard guard(dev);
  const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 4 * 148));
  embedding_counts_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream(dev).stream()>>>(
      idx.data_ptr<int64_t>(), counts.data_ptr<float>(), idx.size(0), idx.size(1), counts.size(1));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

}  // namespace b200
