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
//   bn_stats_finalize  one warp per feature: sums the splits, forms the three products over
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

// Same partial sums for a layer whose output has passed through a fused activation / residual
// add: the normalised input comes from the layer input and the batch statistics, and the output
// gradient is masked by the activation (g = dy where y > 0).
template <bool RELU>
__global__ void __launch_bounds__(BN_THREADS)
bn_stats_partial_xhat(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                      const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean,
                      const float* __restrict__ invstd, float* __restrict__ part, int n_samples,
                      int channels, int hw, int hw_per_split) {
  constexpr int VEC = 8;
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
    float mu[VEC], is[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      mu[i] = mean[c0 + i];
      is[i] = invstd[c0 + i];
    }
    const size_t base = static_cast<size_t>(n) * hw * channels + c0;
    for (int p = hw_begin + lane; p < hw_end; p += BN_LANES) {
      float xv[VEC], gv[VEC];
      VecLoad<__nv_bfloat16, 8>::load(x + base + static_cast<size_t>(p) * channels, xv);
      VecLoad<__nv_bfloat16, 8>::load(dy + base + static_cast<size_t>(p) * channels, gv);
      if (RELU) {
        float yv[VEC];
        VecLoad<__nv_bfloat16, 8>::load(y + base + static_cast<size_t>(p) * channels, yv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) gv[i] = yv[i] > 0.f ? gv[i] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        acc_w[i] = fmaf((xv[i] - mu[i]) * is[i], gv[i], acc_w[i]);
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

// One warp per feature: the lanes stride over the samples.
__global__ void __launch_bounds__(256)
bn_stats_finalize(const float* __restrict__ part, float* __restrict__ stats, int n_samples, int channels,
                  int splits, float alpha, float beta) {
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (c >= channels) return;  // whole warp
  float ww = 0.f, wb = 0.f, bb = 0.f;
  for (int n = lane; n < n_samples; n += 32) {
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
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ww += __shfl_xor_sync(0xffffffffu, ww, o);
    wb += __shfl_xor_sync(0xffffffffu, wb, o);
    bb += __shfl_xor_sync(0xffffffffu, bb, o);
  }
  if (lane != 0) return;
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
  bn_stats_finalize<<<(c + 7) / 8, 256, 0, stream>>>(part.data_ptr<float>(), stats.data_ptr<float>(), n, c,
                                                         splits, static_cast<float>(alpha),
                                                         static_cast<float>(beta));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// Variant for layers with a fused activation: x is the layer input, mean / invstd its batch
// statistics, dy the gradient of the layer output and y (optional) the output that a ReLU masks.
void bn_unitwise_stats_xhat(at::Tensor x, at::Tensor dy, c10::optional<at::Tensor> y, at::Tensor mean,
                            at::Tensor invstd, at::Tensor stats, double alpha, double beta) {
  auto ok = [&](const at::Tensor& t) {
    return t.is_cuda() && t.dim() == 4 && t.scalar_type() == at::kBFloat16 && t.sizes() == x.sizes() &&
           t.is_contiguous(at::MemoryFormat::ChannelsLast) && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  TORCH_CHECK(ok(x) && ok(dy) && (!y.has_value() || ok(*y)), "x, dy and y must be channels_last bf16 CUDA tensors");
  const int n = static_cast<int>(x.size(0)), c = static_cast<int>(x.size(1));
  const int hw = static_cast<int>(x.size(2) * x.size(3));
  TORCH_CHECK(c % 8 == 0, "the channel count must be a multiple of 8");
  TORCH_CHECK(mean.is_cuda() && invstd.is_cuda() && mean.scalar_type() == at::kFloat &&
                  invstd.scalar_type() == at::kFloat && mean.is_contiguous() && invstd.is_contiguous() &&
                  mean.numel() == c && invstd.numel() == c, "mean / invstd must be contiguous fp32 [c]");
  TORCH_CHECK(stats.is_cuda() && stats.scalar_type() == at::kFloat && stats.is_contiguous() &&
                  stats.numel() == 4LL * c && (reinterpret_cast<uintptr_t>(stats.data_ptr()) & 15) == 0,
              "stats must be a contiguous fp32 [c, 2, 2] tensor");
  const int dev = x.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  const int chunks = (c + BN_GROUPS * 8 - 1) / (BN_GROUPS * 8);
  int splits = (148 * 4 + chunks * n - 1) / (chunks * n);
  splits = std::max(1, std::min(splits, (hw + 4 * BN_LANES - 1) / (4 * BN_LANES)));
  const int hw_per_split = (hw + splits - 1) / splits;
  splits = (hw + hw_per_split - 1) / hw_per_split;
  auto part = at::empty({splits, n, c, 2}, stats.options());
  dim3 grid(chunks, n, splits);
  const auto* xp = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  const auto* gp = reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr());
  if (y.has_value())
    bn_stats_partial_xhat<true><<<grid, BN_THREADS, 0, stream>>>(
        xp, gp, reinterpret_cast<const __nv_bfloat16*>(y->data_ptr()), mean.data_ptr<float>(),
        invstd.data_ptr<float>(), part.data_ptr<float>(), n, c, hw, hw_per_split);
  else
    bn_stats_partial_xhat<false><<<grid, BN_THREADS, 0, stream>>>(
        xp, gp, nullptr, mean.data_ptr<float>(), invstd.data_ptr<float>(), part.data_ptr<float>(), n, c, hw,
        hw_per_split);
  bn_stats_finalize<<<(c + 7) / 8, 256, 0, stream>>>(part.data_ptr<float>(), stats.data_ptr<float>(), n, c,
                                                     splits, static_cast<float>(alpha), static_cast<float>(beta));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch(2);
}

}  // namespace b200
