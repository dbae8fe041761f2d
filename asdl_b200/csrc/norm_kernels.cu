// Unit-wise (2 x 2 per feature) curvature of normalisation layers, NHWC activations.
//
// For a BatchNorm2d with weight w, bias b, output y and output gradient g the per-sample
// parameter gradients are  gw[n, c] = sum_hw ((y - b) / w) * g  and  gb[n, c] = sum_hw g, and the
// curvature block of feature c is  sum_n [[gw^2, gw gb], [gw gb, gb^2]]
// (the reference: asdl/operations/batchnorm.py, cov_unit_wise).
//
//   bn_stats_partial   one CTA per (channel chunk, sample, hw split): y and g are read exactly once
//                      with 16-byte loads, the normalised input is reconstructed in registers,
//                      per-lane partial sums are combined through shared memory and written to a
//                      [split, n, c, 2] scratch tensor.
//   bn_stats_finalize  one thread per feature: sums the splits, forms the three products over
//                      the samples and applies  stats <- beta * stats + alpha * new.
#include <cuda_bf16.h>

#include "host_utils.h"

namespace b200 {

template <typename T, int VEC>
struct VecLoad;
template <>
struct VecLoad<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  }
};
template <>
struct VecLoad<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float (&out)[4]) {
    const float4 raw = *reinterpret_cast<const float4*>(p);
    out[0] = raw.x;
    out[1] = raw.y;
    out[2] = raw.z;
    out[3] = raw.w;
  }
};

constexpr int BN_GROUPS = 8;    // channel groups (of VEC channels) per CTA
constexpr int BN_LANES = 32;    // hw lanes per CTA
constexpr int BN_THREADS = BN_GROUPS * BN_LANES;

template <typename T, int VEC>
__global__ void __launch_bounds__(BN_THREADS)
bn_stats_partial(const T* __restrict__ y, const T* __restrict__ g, const float* __restrict__ w,
                 const float* __restrict__ b, float* __restrict__ part, int n_samples, int channels,
                 int hw, int hw_per_split) {
  __shared__ float red[BN_LANES][BN_GROUPS * VEC * 2 + 1];
  const int group = threadIdx.x % BN_GROUPS;
  const int lane = threadIdx.x / BN_GROUPS;
  const int c0 = (blockIdx.x * BN_GROUPS + group) * VEC;
  const int n = blockIdx.y;
  const int hw_begin = blockIdx.z * hw_per_split;
  const int hw_end = min(hw, hw_begin + hw_per_split);
  float acc_w[VEC], acc_b[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc_w[i] = acc_b[i] = 0.f;
  if (c0 < channels) {
    float inv_w[VEC], bias[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      inv_w[i] = 1.f / w[c0 + i];
      bias[i] = b[c0 + i];
    }
    const size_t base = static_cast<size_t>(n) * hw * channels + c0;
    for (int p = hw_begin + lane; p < hw_end; p += BN_LANES) {
      float yv[VEC], gv[VEC];
      VecLoad<T, VEC>::load(y + base + static_cast<size_t>(p) * channels, yv);
      VecLoad<T, VEC>::load(g + base + static_cast<size_t>(p) * channels, gv);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        acc_w[i] = fmaf((yv[i] - bias[i]) * inv_w[i], gv[i], acc_w[i]);
        acc_b[i] += gv[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    red[lane][(group * VEC + i) * 2] = acc_w[i];
    red[lane][(group * VEC + i) * 2 + 1] = acc_b[i];
  }
  __syncthreads();
  if (threadIdx.x < BN_GROUPS * VEC * 2) {
    float s = 0.f;
#pragma unroll 8
    for (int l = 0; l < BN_LANES; ++l) s += red[l][threadIdx.x];
    const int c = blockIdx.x * BN_GROUPS * VEC + threadIdx.x / 2;
    if (c < channels)
      part[((static_cast<size_t>(blockIdx.z) * n_samples + n) * channels + c) * 2 + (threadIdx.x & 1)] = s;
  }
}

__global__ void bn_stats_finalize(const float* __restrict__ part, float* __restrict__ stats,
                                  int n_samples, int channels, int splits, float alpha, float beta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float ww = 0.f, wb = 0.f, bb = 0.f;
  for (int n = 0; n < n_samples; ++n) {
    float gw = 0.f, gb = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float2 v = *reinterpret_cast<const float2*>(
          part + ((static_cast<size_t>(s) * n_samples + n) * channels + c) * 2);
      gw += v.x;
      gb += v.y;
    }
    ww = fmaf(gw, gw, ww);
    wb = fmaf(gw, gb, wb);
    bb = fmaf(gb, gb, bb);
  }
  float4* out = reinterpret_cast<float4*>(stats) + c;
  float4 prev = make_float4(0.f, 0.f, 0.f, 0.f);
  if (beta != 0.f) prev = *out;
  *out = make_float4(fmaf(beta, prev.x, alpha * ww), fmaf(beta, prev.y, alpha * wb),
                     fmaf(beta, prev.z, alpha * wb), fmaf(beta, prev.w, alpha * bb));
}

// y, g: [n, c, h, w] tensors stored channels_last (NHWC), bf16 or fp32, same dtype.
// stats: [c, 2, 2] fp32 contiguous.
void bn_unitwise_stats(at::Tensor y, at::Tensor g, at::Tensor weight, at::Tensor bias, at::Tensor stats,
                       double alpha, double beta) {
  TORCH_CHECK(y.is_cuda() && g.is_cuda() && y.dim() == 4 && y.sizes() == g.sizes() &&
                  y.scalar_type() == g.scalar_type(), "y and g must be CUDA tensors of one shape and dtype");
  TORCH_CHECK(y.is_contiguous(at::MemoryFormat::ChannelsLast) && g.is_contiguous(at::MemoryFormat::ChannelsLast),
              "y and g must be stored channels_last");
  const int n = static_cast<int>(y.size(0)), c = static_cast<int>(y.size(1));
  const int hw = static_cast<int>(y.size(2) * y.size(3));
  const bool bf16 = y.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf16 || y.scalar_type() == at::kFloat, "y must be bf16 or fp32");
  const int vec = bf16 ? 8 : 4;
  TORCH_CHECK(c % vec == 0, "the channel count must be a multiple of ", vec);
  TORCH_CHECK(weight.is_cuda() && bias.is_cuda() && weight.scalar_type() == at::kFloat &&
                  bias.scalar_type() == at::kFloat && weight.is_contiguous() && bias.is_contiguous() &&
                  weight.numel() == c && bias.numel() == c, "weight / bias must be contiguous fp32 [c]");
  TORCH_CHECK(stats.is_cuda() && stats.scalar_type() == at::kFloat && stats.is_contiguous() &&
                  stats.numel() == 4LL * c, "stats must be a contiguous fp32 [c, 2, 2] tensor");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(y.data_ptr()) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(g.data_ptr()) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(stats.data_ptr()) & 15) == 0, "16-byte alignment required");
  const int dev = y.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  const int chunks = (c + BN_GROUPS * vec - 1) / (BN_GROUPS * vec);
  // enough CTAs to fill the GPU a few times over, at least 4 rows of BN_LANES positions per split
  int splits = (148 * 4 + chunks * n - 1) / (chunks * n);
  splits = std::max(1, std::min(splits, (hw + 4 * BN_LANES - 1) / (4 * BN_LANES)));
  const int hw_per_split = (hw + splits - 1) / splits;
  splits = (hw + hw_per_split - 1) / hw_per_split;
  auto part = at::empty({splits, n, c, 2}, stats.options());
  dim3 grid(chunks, n, splits);
  if (bf16)
    bn_stats_partial<__nv_bfloat16, 8><<<grid, BN_THREADS, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(y.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(g.data_ptr()),
        weight.data_ptr<float>(), bias.data_ptr<float>(), part.data_ptr<float>(), n, c, hw, hw_per_split);
  else
    bn_stats_partial<float, 4><<<grid, BN_THREADS, 0, stream>>>(
        y.data_ptr<float>(), g.data_ptr<float>(), weight.data_ptr<float>(), bias.data_ptr<float>(),
        part.data_ptr<float>(), n, c, hw, hw_per_split);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
  bn_stats_finalize<<<(c + 127) / 128, 128, 0, stream>>>(part.data_ptr<float>(), stats.data_ptr<float>(), n, c,
                                                         splits, static_cast<float>(alpha),
                                                         static_cast<float>(beta));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

}  // namespace b200
