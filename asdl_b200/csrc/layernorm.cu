// LayerNorm forward / backward over the last dimension for bf16 activations with fp32 parameters.
//
// A warp owns a row at a time; lane l holds the 8-element vectors l, l + 32, ... of the row in
// registers (VPL vectors per lane, so the feature size is 256 * VPL), which makes every global
// access a 16-byte load / store and the row statistics two warp reductions (mean first, then the
// centred sum of squares: no cancellation).  The backward pass produces the input gradient per
// row and accumulates the weight / bias gradients of the lane's own columns in registers over all
// rows of the warp; warps are combined through shared memory, CTAs through a [ctas, 2, d] partial
// buffer that a second kernel sums (one thread per column, coalesced over columns).
// Rows wider than 1024 elements are split over two or four warps (256 * VPL elements each, VPL <= 4), which
// meet at a named barrier for every row statistic: the backward kernel would otherwise need 40 registers
// per vector slot and spill from 1536 elements on.
//
// PyTorch's own kernels for the weight / bias gradient of LayerNorm take ~60 us per layer at
// d = 1024, 8192 rows on this GPU; these take the time of one pass over dy and x.
#include <cuda_bf16.h>

#include "host_utils.h"

namespace b200 {

namespace {

constexpr int LN_WARPS = 8;
constexpr int LN_THREADS = LN_WARPS * 32;

__device__ __forceinline__ void ln_unpack8(const uint4& raw, float (&out)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint4 ln_pack8(const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return raw;
}

__device__ __forceinline__ float ln_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void ln_load8(const float* p, float (&out)[8]) {
  const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
  out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w;
  out[4] = hi.x; out[5] = hi.y; out[6] = hi.z; out[7] = hi.w;
}

// Sum over the SPLIT warps that share a row: every warp leaves its partial in shared memory, the group
// meets at a named barrier and every warp adds the SPLIT partials.  `slot` alternates so that one barrier
// per reduction is enough (a warp can only be one reduction ahead of the slowest warp of its group).
template <int SPLIT>
__device__ __forceinline__ float ln_group_sum(float v, float (*scratch)[LN_WARPS], int& slot, int warp) {
  v = ln_warp_sum(v);
  if constexpr (SPLIT == 1) return v;
  const int group = warp / SPLIT;
  if ((threadIdx.x & 31) == 0) scratch[slot][warp] = v;
  asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(SPLIT * 32) : "memory");
  float t = 0.f;
#pragma unroll
  for (int s = 0; s < SPLIT; ++s) t += scratch[slot][group * SPLIT + s];
  slot = (slot + 1) % 3;
  return t;
}

// A row of D = 256 * VPL * SPLIT elements is handled by SPLIT warps, each keeping 256 * VPL of it in
// registers (VPL 16-byte vectors per lane); SPLIT > 1 keeps the register need of wide rows at that of VPL <= 4.
template <int VPL, int SPLIT>
__global__ void __launch_bounds__(LN_THREADS)
ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
              const float* __restrict__ beta, __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out,
              float* __restrict__ rstd_out, long long rows, float eps) {
  constexpr int D = 256 * VPL * SPLIT;
  constexpr int GROUPS = LN_WARPS / SPLIT;
  __shared__ float scratch[3][LN_WARPS];
  int slot = 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = warp / SPLIT, col0 = (warp % SPLIT) * 256 * VPL;
  float g[VPL][8], b[VPL][8];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    ln_load8(gamma + col0 + (v * 32 + lane) * 8, g[v]);
    ln_load8(beta + col0 + (v * 32 + lane) * 8, b[v]);
  }
  for (long long r = static_cast<long long>(blockIdx.x) * GROUPS + group; r < rows;
       r += static_cast<long long>(gridDim.x) * GROUPS) {
    const __nv_bfloat16* xr = x + r * D + col0;
    float xv[VPL][8];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      ln_unpack8(__ldg(reinterpret_cast<const uint4*>(xr + (v * 32 + lane) * 8)), xv[v]);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += xv[v][i];
    }
    const float mean = ln_group_sum<SPLIT>(s, scratch, slot, warp) * (1.f / D);
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float c = xv[v][i] - mean;
        q = fmaf(c, c, q);
      }
    const float rstd = rsqrtf(ln_group_sum<SPLIT>(q, scratch, slot, warp) * (1.f / D) + eps);
    __nv_bfloat16* yr = y + r * D + col0;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      float out[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = fmaf((xv[v][i] - mean) * rstd, g[v][i], b[v][i]);
      *reinterpret_cast<uint4*>(yr + (v * 32 + lane) * 8) = ln_pack8(out);
    }
    if (lane == 0 && col0 == 0) {
      mean_out[r] = mean;
      rstd_out[r] = rstd;
    }
  }
}

template <int VPL, int SPLIT>
__global__ void __launch_bounds__(LN_THREADS)
ln_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
              const float* __restrict__ gamma, const float* __restrict__ mean, const float* __restrict__ rstd,
              __nv_bfloat16* __restrict__ dx, float* __restrict__ part, long long rows) {
  constexpr int D = 256 * VPL * SPLIT;
  constexpr int GROUPS = LN_WARPS / SPLIT;
  __shared__ float red[LN_WARPS][2][32 * 8 + 1];  // one vector slot (v) at a time
  __shared__ float scratch[3][LN_WARPS];
  int slot = 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = warp / SPLIT, col0 = (warp % SPLIT) * 256 * VPL;
  float g[VPL][8], dg[VPL][8], db[VPL][8];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    ln_load8(gamma + col0 + (v * 32 + lane) * 8, g[v]);
#pragma unroll
    for (int i = 0; i < 8; ++i) dg[v][i] = db[v][i] = 0.f;
  }
  for (long long r = static_cast<long long>(blockIdx.x) * GROUPS + group; r < rows;
       r += static_cast<long long>(gridDim.x) * GROUPS) {
    const float mu = mean[r], rs = rstd[r];
    float xh[VPL][8], gy[VPL][8];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      float xv[8], dv[8];
      ln_unpack8(__ldg(reinterpret_cast<const uint4*>(x + r * D + col0 + (v * 32 + lane) * 8)), xv);
      ln_unpack8(__ldg(reinterpret_cast<const uint4*>(dy + r * D + col0 + (v * 32 + lane) * 8)), dv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        xh[v][i] = (xv[i] - mu) * rs;
        dg[v][i] = fmaf(dv[i], xh[v][i], dg[v][i]);
        db[v][i] += dv[i];
        gy[v][i] = dv[i] * g[v][i];
        c1 = fmaf(gy[v][i], xh[v][i], c1);
        c2 += gy[v][i];
      }
    }
    c1 = ln_group_sum<SPLIT>(c1, scratch, slot, warp) * (1.f / D);
    c2 = ln_group_sum<SPLIT>(c2, scratch, slot, warp) * (1.f / D);
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      float out[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = rs * (gy[v][i] - c2 - xh[v][i] * c1);
      *reinterpret_cast<uint4*>(dx + r * D + col0 + (v * 32 + lane) * 8) = ln_pack8(out);
    }
  }
  // combine the warps of the CTA that hold the same columns, one vector slot at a time
  float* out = part + static_cast<size_t>(blockIdx.x) * 2 * D;
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      red[warp][0][lane * 8 + i] = dg[v][i];
      red[warp][1][lane * 8 + i] = db[v][i];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 2 * 256 * SPLIT; e += LN_THREADS) {
      const int col = e & 255, which = (e >> 8) & 1, slice = e >> 9;
      float s = 0.f;
#pragma unroll
      for (int gi = 0; gi < GROUPS; ++gi) s += red[gi * SPLIT + slice][which][col];
      out[which * D + slice * 256 * VPL + v * 256 + col] = s;
    }
    __syncthreads();
  }
}

// dgamma[j] = sum over CTAs of part[c][0][j], dbeta[j] likewise (coalesced over j).
__global__ void ln_bwd_finalize(const float* __restrict__ part, float* __restrict__ dgamma,
                                float* __restrict__ dbeta, int ctas, int d) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= d) return;
  float sg = 0.f, sb = 0.f;
  for (int c = 0; c < ctas; ++c) {
    sg += part[(static_cast<size_t>(c) * 2) * d + j];
    sb += part[(static_cast<size_t>(c) * 2 + 1) * d + j];
  }
  dgamma[j] = sg;
  dbeta[j] = sb;
}

int ln_grid(long long rows, int groups) {
  return static_cast<int>(std::max<long long>(1, std::min<long long>((rows + groups - 1) / groups, 148LL * 2)));
}

void ln_check(const at::Tensor& x, const at::Tensor& gamma, int& vpl, long long& rows) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() >= 1,
              "x must be a contiguous bf16 CUDA tensor");
  const long long d = x.size(-1);
  TORCH_CHECK(d % 256 == 0 && d >= 256 && d <= 4096, "the normalised size must be a multiple of 256 up to 4096");
  vpl = static_cast<int>(d / 256);
  TORCH_CHECK(vpl == 1 || vpl == 2 || vpl == 3 || vpl == 4 || vpl == 6 || vpl == 8 || vpl == 12 || vpl == 16,
              "unsupported normalised size");
  rows = x.numel() / d;
  TORCH_CHECK(gamma.is_cuda() && gamma.scalar_type() == at::kFloat && gamma.is_contiguous() && gamma.numel() == d,
              "weight must be a contiguous fp32 vector of the normalised size");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "16-byte alignment required");
}

template <int V, int S>
void launch_fwd(int grid, cudaStream_t stream, const __nv_bfloat16* x, const float* gamma, const float* beta,
                __nv_bfloat16* y, float* mean, float* rstd, long long rows, float eps) {
  ln_fwd_kernel<V, S><<<grid, LN_THREADS, 0, stream>>>(x, gamma, beta, y, mean, rstd, rows, eps);
}

template <int V, int S>
void launch_bwd(int grid, cudaStream_t stream, const __nv_bfloat16* x, const __nv_bfloat16* dy, const float* gamma,
                const float* mean, const float* rstd, __nv_bfloat16* dx, float* part, long long rows) {
  ln_bwd_kernel<V, S><<<grid, LN_THREADS, 0, stream>>>(x, dy, gamma, mean, rstd, dx, part, rows);
}

// rows of 256 * v elements: up to v = 4 one warp per row, wider rows split over 2 or 4 warps
#define LN_DISPATCH(VPL_VALUE, FN, ...)         \
  switch (VPL_VALUE) {                          \
    case 1: FN<1, 1>(__VA_ARGS__); break;       \
    case 2: FN<2, 1>(__VA_ARGS__); break;       \
    case 3: FN<3, 1>(__VA_ARGS__); break;       \
    case 4: FN<4, 1>(__VA_ARGS__); break;       \
    case 6: FN<3, 2>(__VA_ARGS__); break;       \
    case 8: FN<4, 2>(__VA_ARGS__); break;       \
    case 12: FN<3, 4>(__VA_ARGS__); break;      \
    default: FN<4, 4>(__VA_ARGS__); break;      \
  }

// warps of a CTA that work on different rows at a time
int ln_groups(int vpl) { return vpl <= 4 ? LN_WARPS : (vpl <= 8 ? LN_WARPS / 2 : LN_WARPS / 4); }

}  // namespace

bool ln_supported_size(int64_t d) {
  if (d % 256 != 0) return false;
  const int64_t v = d / 256;
  return v == 1 || v == 2 || v == 3 || v == 4 || v == 6 || v == 8 || v == 12 || v == 16;
}

// Returns (y, mean, rstd); mean / rstd have one entry per row.
std::vector<at::Tensor> ln_forward(at::Tensor x, at::Tensor weight, at::Tensor bias, double eps) {
  int vpl;
  long long rows;
  ln_check(x, weight, vpl, rows);
  TORCH_CHECK(bias.is_cuda() && bias.scalar_type() == at::kFloat && bias.is_contiguous() &&
                  bias.numel() == weight.numel(), "bias must match weight");
  const int dev = x.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  auto y = at::empty_like(x);
  auto mean = at::empty({rows}, weight.options()), rstd = at::empty({rows}, weight.options());
  if (rows == 0) return {y, mean, rstd};
  const int grid = ln_grid(rows, ln_groups(vpl));
  const auto* xp = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  auto* yp = reinterpret_cast<__nv_bfloat16*>(y.data_ptr());
  LN_DISPATCH(vpl, launch_fwd, grid, stream, xp, weight.data_ptr<float>(), bias.data_ptr<float>(), yp,
              mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, static_cast<float>(eps));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return {y, mean, rstd};
}

// Returns (dx, dweight, dbias).
std::vector<at::Tensor> ln_backward(at::Tensor x, at::Tensor dy, at::Tensor weight, at::Tensor mean,
                                    at::Tensor rstd) {
  int vpl;
  long long rows;
  ln_check(x, weight, vpl, rows);
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && dy.sizes() == x.sizes() &&
                  (reinterpret_cast<uintptr_t>(dy.data_ptr()) & 15) == 0, "dy must match x");
  TORCH_CHECK(mean.is_cuda() && rstd.is_cuda() && mean.scalar_type() == at::kFloat && rstd.scalar_type() == at::kFloat &&
                  mean.numel() == rows && rstd.numel() == rows && mean.is_contiguous() && rstd.is_contiguous(),
              "mean / rstd must hold one fp32 value per row");
  const int dev = x.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  const long long d = x.size(-1);
  auto dx = at::empty_like(x);
  auto dweight = at::zeros({d}, weight.options()), dbias = at::zeros({d}, weight.options());
  if (rows == 0) return {dx, dweight, dbias};
  const int grid = ln_grid(rows, ln_groups(vpl));
  auto part = at::empty({grid, 2, d}, weight.options());
  const auto* xp = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  const auto* gp = reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr());
  auto* dxp = reinterpret_cast<__nv_bfloat16*>(dx.data_ptr());
  LN_DISPATCH(vpl, launch_bwd, grid, stream, xp, gp, weight.data_ptr<float>(), mean.data_ptr<float>(),
              rstd.data_ptr<float>(), dxp, part.data_ptr<float>(), rows);
  ln_bwd_finalize<<<static_cast<int>((d + 127) / 128), 128, 0, stream>>>(
      part.data_ptr<float>(), dweight.data_ptr<float>(), dbias.data_ptr<float>(), grid, static_cast<int>(d));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch(2);
  return {dx, dweight, dbias};
}

}  // namespace b200
