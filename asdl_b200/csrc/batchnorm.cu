// Training-mode BatchNorm2d for NHWC (channels_last) bf16 activations with fp32 parameters and
// statistics.  The activation tensor is treated as a row-major [rows = n*h*w, c] matrix; every
// thread owns 8 consecutive channels (one 16-byte load) and walks down the rows, so all global
// accesses are full 128-byte lines and each pass moves exactly the bytes it has to:
//
//   forward    bn_sums (read x)            -> per-split partial sums and sums of squares
//              bn_fwd_finalize             -> mean, 1/std, running statistics, scale/shift
//              bn_apply   (read x, write y)   y = x * scale + shift
//   backward   bn_bwd_sums (read x, dy)    -> per-split partial sums of dy and dy * xhat
//              bn_bwd_finalize             -> dweight, dbias and the three dx coefficients
//              bn_dx      (read x, dy, write dx)
//
// Partial sums are combined in double precision by the finalize kernels (one warp per channel),
// which keeps var = E[x^2] - E[x]^2 accurate.
#include <cuda_bf16.h>

#include "host_utils.h"

namespace b200 {

namespace {

constexpr int GROUPS = 8;    // channel groups of 8 channels per CTA -> 64 channels
constexpr int LANES = 32;    // row lanes per CTA
constexpr int THREADS = GROUPS * LANES;
constexpr int UNROLL = 8;    // independent 16-byte loads in flight per thread (forward sums)

__device__ __forceinline__ void unpack8(const uint4& raw, float (&out)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return raw;
}

__device__ __forceinline__ uint4 ld_stream(const __nv_bfloat16* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// Combines the per-lane accumulators acc[2][8] of a CTA and writes one (first, second) pair per
// channel to part[(split * channels + c) * 2].
__device__ __forceinline__ void cta_reduce_store(float (&first)[8], float (&second)[8], float* part,
                                                 int channels, int split) {
  __shared__ float red[LANES][GROUPS * 16 + 1];
  const int group = threadIdx.x % GROUPS;
  const int lane = threadIdx.x / GROUPS;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    red[lane][(group * 8 + i) * 2] = first[i];
    red[lane][(group * 8 + i) * 2 + 1] = second[i];
  }
  __syncthreads();
  if (threadIdx.x < GROUPS * 16) {
    float s = 0.f;
#pragma unroll 8
    for (int l = 0; l < LANES; ++l) s += red[l][threadIdx.x];
    const int c = blockIdx.x * GROUPS * 8 + threadIdx.x / 2;
    if (c < channels) part[(static_cast<size_t>(split) * channels + c) * 2 + (threadIdx.x & 1)] = s;
  }
}

__global__ void __launch_bounds__(THREADS)
bn_sums(const __nv_bfloat16* __restrict__ x, float* __restrict__ part, long long rows, int channels,
        long long rows_per_split) {
  const int group = threadIdx.x % GROUPS;
  const int lane = threadIdx.x / GROUPS;
  const int c0 = (blockIdx.x * GROUPS + group) * 8;
  const long long r_begin = blockIdx.y * rows_per_split;
  const long long r_end = min(rows, r_begin + rows_per_split);
  float sum[8], sq[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sum[i] = sq[i] = 0.f;
  if (c0 < channels) {
    const __nv_bfloat16* base = x + c0;
    long long r = r_begin + lane;
    for (; r + (UNROLL - 1) * LANES < r_end; r += UNROLL * LANES) {
      uint4 raw[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) raw[u] = ld_stream(base + (r + u * LANES) * channels);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        float v[8];
        unpack8(raw[u], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          sum[i] += v[i];
          sq[i] = fmaf(v[i], v[i], sq[i]);
        }
      }
    }
    for (; r < r_end; r += LANES) {
      float v[8];
      unpack8(ld_stream(base + r * channels), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sum[i] += v[i];
        sq[i] = fmaf(v[i], v[i], sq[i]);
      }
    }
  }
  cta_reduce_store(sum, sq, part, channels, blockIdx.y);
}

// coef layout (fp32, [5, c]): scale, shift (forward); k_dy, k_x, k_const (backward)
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per channel: the lanes stride over the splits, combine in double precision.
__global__ void __launch_bounds__(256)
bn_fwd_finalize(const float* __restrict__ part, const float* __restrict__ weight,
                const float* __restrict__ bias, float* __restrict__ running_mean,
                float* __restrict__ running_var, float* __restrict__ mean_out,
                float* __restrict__ invstd_out, float* __restrict__ coef, long long* __restrict__ tracked,
                int channels, int splits, long long rows, float momentum, float eps) {
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (c >= channels) return;  // whole warp
  double s = 0.0, q = 0.0;
  for (int k = lane; k < splits; k += 32) {
    const float2 v = *reinterpret_cast<const float2*>(part + (static_cast<size_t>(k) * channels + c) * 2);
    s += v.x;
    q += v.y;
  }
  s = warp_sum(s);
  q = warp_sum(q);
  if (lane != 0) return;
  if (c == 0 && tracked != nullptr) *tracked += 1;
  const double mean = s / static_cast<double>(rows);
  double var = q / static_cast<double>(rows) - mean * mean;
  var = var > 0.0 ? var : 0.0;
  const float invstd = static_cast<float>(1.0 / sqrt(var + static_cast<double>(eps)));
  mean_out[c] = static_cast<float>(mean);
  invstd_out[c] = invstd;
  // explicit roundings: the backward pass recomputes scale and shift bit for bit (ReLU mask from x)
  const float scale = __fmul_rn(weight[c], invstd);
  coef[c] = scale;
  coef[channels + c] = __fmaf_rn(-static_cast<float>(mean), scale, bias[c]);
  if (running_mean != nullptr) {
    const double unbiased = rows > 1 ? var * static_cast<double>(rows) / static_cast<double>(rows - 1) : var;
    running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * static_cast<float>(mean);
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * static_cast<float>(unbiased);
  }
}

__device__ __forceinline__ void load8(const float* p, float (&out)[8]) {
  const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
  out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w;
  out[4] = hi.x; out[5] = hi.y; out[6] = hi.z; out[7] = hi.w;
}

// y = act(x * scale[c] + shift[c] (+ residual))
template <bool RES, bool RELU>
__global__ void __launch_bounds__(256)
bn_apply(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
         const float* __restrict__ scale, const float* __restrict__ shift, __nv_bfloat16* __restrict__ y,
         long long vecs, int vec_per_row) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
#pragma unroll 4
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < vecs; i += stride) {
    const int c0 = static_cast<int>(i % vec_per_row) * 8;
    float a[8], v[8], out[8];
    unpack8(ld_stream(x + i * 8), v);
    load8(scale + c0, a);
    load8(shift + c0, out);
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = fmaf(v[k], a[k], out[k]);
    if (RES) {
      float r[8];
      unpack8(ld_stream(res + i * 8), r);
#pragma unroll
      for (int k = 0; k < 8; ++k) out[k] += r[k];
    }
    if (RELU) {
#pragma unroll
      for (int k = 0; k < 8; ++k) out[k] = fmaxf(out[k], 0.f);
    }
    *reinterpret_cast<uint4*>(y + i * 8) = pack8(out);
  }
}

// How the backward kernels find the ReLU mask: no activation, from the saved output y, or recomputed from x
// (y > 0 exactly when x * scale[c] + shift[c] > 0; only without a residual).  Recomputing saves one read of an
// activation-sized tensor in each of the two backward passes.
enum : int { MASK_NONE = 0, MASK_FROM_Y = 1, MASK_FROM_X = 2 };

// g = masked dy;   dx = g * k_dy[c] + x * k_x[c] + k_const[c];   dres = g (optional)
template <int MASK, bool DRES>
__global__ void __launch_bounds__(256)
bn_dx(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
      const __nv_bfloat16* __restrict__ y, const float* __restrict__ scale, const float* __restrict__ shift,
      const float* __restrict__ k_dy, const float* __restrict__ k_x,
      const float* __restrict__ k_const, __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dres,
      long long vecs, int vec_per_row) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
#pragma unroll 2
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < vecs; i += stride) {
    const int c0 = static_cast<int>(i % vec_per_row) * 8;
    float g[8], xv[8], a[8], b[8], out[8];
    unpack8(ld_stream(dy + i * 8), g);
    unpack8(ld_stream(x + i * 8), xv);
    if (MASK == MASK_FROM_Y) {
      float yv[8];
      unpack8(ld_stream(y + i * 8), yv);
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = yv[k] > 0.f ? g[k] : 0.f;
    }
    if (MASK == MASK_FROM_X) {
      float sc[8], sh[8];
      load8(scale + c0, sc);
      load8(shift + c0, sh);
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = fmaf(xv[k], sc[k], sh[k]) > 0.f ? g[k] : 0.f;
    }
    load8(k_dy + c0, a);
    load8(k_x + c0, b);
    load8(k_const + c0, out);
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = fmaf(g[k], a[k], fmaf(xv[k], b[k], out[k]));
    *reinterpret_cast<uint4*>(dx + i * 8) = pack8(out);
    if (DRES) *reinterpret_cast<uint4*>(dres + i * 8) = pack8(g);
  }
}

template <int MASK>
__global__ void __launch_bounds__(THREADS)
bn_bwd_sums(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
            const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean,
            const float* __restrict__ invstd, const float* __restrict__ weight, const float* __restrict__ bias,
            float* __restrict__ part, long long rows, int channels, long long rows_per_split) {
  const int group = threadIdx.x % GROUPS;
  const int lane = threadIdx.x / GROUPS;
  const int c0 = (blockIdx.x * GROUPS + group) * 8;
  const long long r_begin = blockIdx.y * rows_per_split;
  const long long r_end = min(rows, r_begin + rows_per_split);
  float s_dy[8], s_dyx[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) s_dy[i] = s_dyx[i] = 0.f;
  if (c0 < channels) {
    float mu[8], is[8], sc[8], sh[8];
    load8(mean + c0, mu);
    load8(invstd + c0, is);
    if (MASK == MASK_FROM_X) {   // the forward pass's scale and shift, same roundings
      load8(weight + c0, sc);
      load8(bias + c0, sh);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sc[i] = __fmul_rn(sc[i], is[i]);
        sh[i] = __fmaf_rn(-mu[i], sc[i], sh[i]);
      }
    }
    const __nv_bfloat16* bx = x + c0;
    const __nv_bfloat16* bg = dy + c0;
    const __nv_bfloat16* by = y + c0;
    constexpr int U = MASK == MASK_FROM_Y ? 2 : 4;  // two or three tensors in flight per row
    auto masked = [&](const float (&xv)[8], float (&gv)[8]) {
      if (MASK == MASK_FROM_X) {
#pragma unroll
        for (int i = 0; i < 8; ++i) gv[i] = fmaf(xv[i], sc[i], sh[i]) > 0.f ? gv[i] : 0.f;
      }
    };
    long long r = r_begin + lane;
    for (; r + (U - 1) * LANES < r_end; r += U * LANES) {
      uint4 rx[U], rg[U], ry[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        rx[u] = ld_stream(bx + (r + u * LANES) * channels);
        rg[u] = ld_stream(bg + (r + u * LANES) * channels);
        if (MASK == MASK_FROM_Y) ry[u] = ld_stream(by + (r + u * LANES) * channels);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float xv[8], gv[8];
        unpack8(rx[u], xv);
        unpack8(rg[u], gv);
        if (MASK == MASK_FROM_Y) {
          float yv[8];
          unpack8(ry[u], yv);
#pragma unroll
          for (int i = 0; i < 8; ++i) gv[i] = yv[i] > 0.f ? gv[i] : 0.f;
        }
        masked(xv, gv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          s_dy[i] += gv[i];
          s_dyx[i] = fmaf((xv[i] - mu[i]) * is[i], gv[i], s_dyx[i]);
        }
      }
    }
    for (; r < r_end; r += LANES) {
      float xv[8], gv[8];
      unpack8(ld_stream(bx + r * channels), xv);
      unpack8(ld_stream(bg + r * channels), gv);
      if (MASK == MASK_FROM_Y) {
        float yv[8];
        unpack8(ld_stream(by + r * channels), yv);
#pragma unroll
        for (int i = 0; i < 8; ++i) gv[i] = yv[i] > 0.f ? gv[i] : 0.f;
      }
      masked(xv, gv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s_dy[i] += gv[i];
        s_dyx[i] = fmaf((xv[i] - mu[i]) * is[i], gv[i], s_dyx[i]);
      }
    }
  }
  cta_reduce_store(s_dy, s_dyx, part, channels, blockIdx.y);
}

// dx = w*invstd * (dy - mean(dy) - xhat * mean(dy*xhat))
//    = dy * k_dy + x * k_x + k_const  with
//   k_dy = w*invstd, k_x = -k_dy * invstd * m2, k_const = -k_dy * (m1 - mean * invstd * m2)
__global__ void __launch_bounds__(256)
bn_bwd_finalize(const float* __restrict__ part, const float* __restrict__ weight, const float* __restrict__ bias,
                const float* __restrict__ mean, const float* __restrict__ invstd,
                float* __restrict__ dweight, float* __restrict__ dbias,
                float* __restrict__ coef, int channels, int splits, long long rows) {
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (c >= channels) return;  // whole warp
  double s1 = 0.0, s2 = 0.0;
  for (int k = lane; k < splits; k += 32) {
    const float2 v = *reinterpret_cast<const float2*>(part + (static_cast<size_t>(k) * channels + c) * 2);
    s1 += v.x;
    s2 += v.y;
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  if (lane != 0) return;
  dbias[c] = static_cast<float>(s1);
  dweight[c] = static_cast<float>(s2);
  const double m1 = s1 / static_cast<double>(rows), m2 = s2 / static_cast<double>(rows);
  const double k_dy = static_cast<double>(weight[c]) * invstd[c];
  coef[2 * channels + c] = static_cast<float>(k_dy);
  coef[3 * channels + c] = static_cast<float>(-k_dy * invstd[c] * m2);
  coef[4 * channels + c] = static_cast<float>(-k_dy * (m1 - static_cast<double>(mean[c]) * invstd[c] * m2));
  if (bias != nullptr) {   // the forward pass's scale and shift (rows 0 and 1) for a ReLU mask recomputed from x
    const float scale = __fmul_rn(weight[c], invstd[c]);
    coef[c] = scale;
    coef[channels + c] = __fmaf_rn(-mean[c], scale, bias[c]);
  }
}

struct Shape {
  long long rows;
  int channels;
  int chunks;
  int splits;
  long long rows_per_split;
};

Shape plan(const at::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.scalar_type() == at::kBFloat16 &&
                  x.is_contiguous(at::MemoryFormat::ChannelsLast),
              "expected a 4-d channels_last bf16 CUDA tensor");
  Shape s;
  s.channels = static_cast<int>(x.size(1));
  s.rows = x.size(0) * x.size(2) * x.size(3);
  TORCH_CHECK(s.channels % 8 == 0 && s.rows > 0, "the channel count must be a multiple of 8");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "16-byte alignment required");
  s.chunks = (s.channels + GROUPS * 8 - 1) / (GROUPS * 8);
  long long want = (148 * 8 + s.chunks - 1) / s.chunks;                   // ~8 CTAs per SM in total
  long long most = (s.rows + 2 * UNROLL * LANES - 1) / (2 * UNROLL * LANES);  // >= 2 unrolled trips each
  long long splits = std::max<long long>(1, std::min(want, most));
  s.rows_per_split = (s.rows + splits - 1) / splits;
  s.splits = static_cast<int>((s.rows + s.rows_per_split - 1) / s.rows_per_split);
  return s;
}

void check_vec(const at::Tensor& t, int c, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() == c, name,
              " must be a contiguous fp32 CUDA vector with one entry per channel");
}

int affine_grid(long long vecs) {
  return static_cast<int>(std::min<long long>((vecs + 255) / 256, 148LL * 16));
}

void check_like(const at::Tensor& t, const at::Tensor& x, const char* name) {
  TORCH_CHECK(t.sizes() == x.sizes() && t.scalar_type() == at::kBFloat16 && t.is_cuda() &&
                  t.is_contiguous(at::MemoryFormat::ChannelsLast) &&
                  (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0,
              name, " must match x (channels_last bf16, 16-byte aligned)");
}

}  // namespace

// y = act(batch_norm(x) (+ residual)).  Returns (y, mean, invstd).  running_mean / running_var and
// the batch counter are updated in place when given.
std::vector<at::Tensor> bn_forward_train(at::Tensor x, at::Tensor weight, at::Tensor bias,
                                         c10::optional<at::Tensor> running_mean,
                                         c10::optional<at::Tensor> running_var,
                                         c10::optional<at::Tensor> num_batches_tracked, double momentum,
                                         double eps, c10::optional<at::Tensor> residual, bool relu) {
  const Shape s = plan(x);
  check_vec(weight, s.channels, "weight");
  check_vec(bias, s.channels, "bias");
  float *rm = nullptr, *rv = nullptr;
  if (running_mean.has_value() && running_var.has_value()) {
    check_vec(*running_mean, s.channels, "running_mean");
    check_vec(*running_var, s.channels, "running_var");
    rm = running_mean->data_ptr<float>();
    rv = running_var->data_ptr<float>();
  }
  long long* tracked = nullptr;
  if (num_batches_tracked.has_value()) {
    TORCH_CHECK(num_batches_tracked->is_cuda() && num_batches_tracked->scalar_type() == at::kLong &&
                    num_batches_tracked->numel() == 1, "num_batches_tracked must be a CUDA int64 scalar");
    tracked = reinterpret_cast<long long*>(num_batches_tracked->data_ptr<int64_t>());
  }
  const __nv_bfloat16* rp = nullptr;
  if (residual.has_value()) {
    check_like(*residual, x, "residual");
    rp = reinterpret_cast<const __nv_bfloat16*>(residual->data_ptr());
  }
  const int dev = x.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  auto f32 = weight.options();
  auto part = at::empty({s.splits, s.channels, 2}, f32);
  auto mean = at::empty({s.channels}, f32), invstd = at::empty({s.channels}, f32);
  auto coef = at::empty({2, s.channels}, f32);
  auto y = at::empty_like(x);
  const auto* xp = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  auto* yp = reinterpret_cast<__nv_bfloat16*>(y.data_ptr());
  bn_sums<<<dim3(s.chunks, s.splits), THREADS, 0, stream>>>(xp, part.data_ptr<float>(), s.rows, s.channels,
                                                            s.rows_per_split);
  bn_fwd_finalize<<<(s.channels + 7) / 8, 256, 0, stream>>>(
      part.data_ptr<float>(), weight.data_ptr<float>(), bias.data_ptr<float>(), rm, rv, mean.data_ptr<float>(),
      invstd.data_ptr<float>(), coef.data_ptr<float>(), tracked, s.channels, s.splits, s.rows,
      static_cast<float>(momentum), static_cast<float>(eps));
  const long long vecs = s.rows * (s.channels / 8);
  const int grid = affine_grid(vecs), vpr = s.channels / 8;
  const float* scale = coef.data_ptr<float>();
  const float* shift = scale + s.channels;
  if (rp != nullptr && relu)
    bn_apply<true, true><<<grid, 256, 0, stream>>>(xp, rp, scale, shift, yp, vecs, vpr);
  else if (rp != nullptr)
    bn_apply<true, false><<<grid, 256, 0, stream>>>(xp, rp, scale, shift, yp, vecs, vpr);
  else if (relu)
    bn_apply<false, true><<<grid, 256, 0, stream>>>(xp, nullptr, scale, shift, yp, vecs, vpr);
  else
    bn_apply<false, false><<<grid, 256, 0, stream>>>(xp, nullptr, scale, shift, yp, vecs, vpr);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch(3);
  return {y, mean, invstd};
}

// Backward of y = act(batch_norm(x) (+ residual)).  The ReLU mask comes from `y`, or - when `bias_for_mask` is given
// instead (ReLU without a residual) - is recomputed from x, which saves a read of y in both passes.
// Returns (dx, dweight, dbias) and, with `want_dres`, the gradient of the residual (dy masked by
// the activation; without an activation it is dy itself and is not returned).
std::vector<at::Tensor> bn_backward_train(at::Tensor x, at::Tensor dy, at::Tensor weight, at::Tensor mean,
                                          at::Tensor invstd, c10::optional<at::Tensor> y, bool want_dres,
                                          c10::optional<at::Tensor> bias_for_mask) {
  const Shape s = plan(x);
  check_like(dy, x, "dy");
  check_vec(weight, s.channels, "weight");
  check_vec(mean, s.channels, "mean");
  check_vec(invstd, s.channels, "invstd");
  const bool from_x = bias_for_mask.has_value();
  TORCH_CHECK(!(from_x && (y.has_value() || want_dres)), "the mask is recomputed from x only without y and without a residual");
  const bool relu = y.has_value() || from_x;
  const __nv_bfloat16* yp = nullptr;
  if (y.has_value()) {
    check_like(*y, x, "y");
    yp = reinterpret_cast<const __nv_bfloat16*>(y->data_ptr());
  }
  const float* bp = nullptr;
  if (from_x) {
    check_vec(*bias_for_mask, s.channels, "bias");
    bp = bias_for_mask->data_ptr<float>();
  }
  const bool dres_out = want_dres && relu;
  const int dev = x.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  auto f32 = weight.options();
  auto part = at::empty({s.splits, s.channels, 2}, f32);
  auto dweight = at::empty({s.channels}, f32), dbias = at::empty({s.channels}, f32);
  auto coef = at::empty({5, s.channels}, f32);
  auto dx = at::empty_like(x);
  at::Tensor dres;
  if (dres_out) dres = at::empty_like(x);
  const auto* xp = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  const auto* gp = reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr());
  auto* dxp = reinterpret_cast<__nv_bfloat16*>(dx.data_ptr());
  auto* drp = dres_out ? reinterpret_cast<__nv_bfloat16*>(dres.data_ptr()) : nullptr;
  const dim3 sgrid(s.chunks, s.splits);
  const float *wp = weight.data_ptr<float>(), *mp = mean.data_ptr<float>(), *ip = invstd.data_ptr<float>();
  if (from_x)
    bn_bwd_sums<MASK_FROM_X><<<sgrid, THREADS, 0, stream>>>(xp, gp, xp, mp, ip, wp, bp, part.data_ptr<float>(), s.rows,
                                                            s.channels, s.rows_per_split);
  else if (relu)
    bn_bwd_sums<MASK_FROM_Y><<<sgrid, THREADS, 0, stream>>>(xp, gp, yp, mp, ip, wp, nullptr, part.data_ptr<float>(), s.rows,
                                                            s.channels, s.rows_per_split);
  else
    bn_bwd_sums<MASK_NONE><<<sgrid, THREADS, 0, stream>>>(xp, gp, xp, mp, ip, wp, nullptr, part.data_ptr<float>(), s.rows,
                                                          s.channels, s.rows_per_split);
  bn_bwd_finalize<<<(s.channels + 7) / 8, 256, 0, stream>>>(
      part.data_ptr<float>(), wp, bp, mp, ip, dweight.data_ptr<float>(), dbias.data_ptr<float>(), coef.data_ptr<float>(),
      s.channels, s.splits, s.rows);
  const long long vecs = s.rows * (s.channels / 8);
  const int grid = affine_grid(vecs), vpr = s.channels / 8;
  const float* k = coef.data_ptr<float>();
  const float *sc = k, *sh = k + s.channels;
  const float *k_dy = k + 2 * s.channels, *k_x = k + 3 * s.channels, *k_c = k + 4 * s.channels;
  if (from_x)
    bn_dx<MASK_FROM_X, false><<<grid, 256, 0, stream>>>(gp, xp, nullptr, sc, sh, k_dy, k_x, k_c, dxp, nullptr, vecs, vpr);
  else if (relu && dres_out)
    bn_dx<MASK_FROM_Y, true><<<grid, 256, 0, stream>>>(gp, xp, yp, sc, sh, k_dy, k_x, k_c, dxp, drp, vecs, vpr);
  else if (relu)
    bn_dx<MASK_FROM_Y, false><<<grid, 256, 0, stream>>>(gp, xp, yp, sc, sh, k_dy, k_x, k_c, dxp, nullptr, vecs, vpr);
  else
    bn_dx<MASK_NONE, false><<<grid, 256, 0, stream>>>(gp, xp, nullptr, sc, sh, k_dy, k_x, k_c, dxp, nullptr, vecs, vpr);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch(3);
  if (dres_out) return {dx, dweight, dbias, dres};
  return {dx, dweight, dbias};
}

}  // namespace b200
