// Bandwidth-bound staging kernels that feed the tcgen05 GEMMs:
//   * cast_pad_bf16  : [rows, n] fp32/bf16 -> bf16 with a TMA-legal row pitch, optional residual
//                      ("lo") so that hi+lo carries ~16 mantissa bits.
//   * im2col_bf16    : conv input (any strides: NCHW or channels_last) -> patch matrix
//                      [N*Ho*Wo, ld] bf16, columns ordered (kh, kw, c) or (c, kh, kw).
#include "host_utils.h"
#include <cuda_bf16.h>

namespace b200 {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__global__ void cast_pad_bf16_kernel(const T* __restrict__ src, long long lds, float scale,
                                     __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                                     long long ldo, long long rows, int n) {
  const long long total = rows * ldo;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / ldo;
    const int c = static_cast<int>(i - r * ldo);
    float v = (c < n) ? to_f32<T>(src[r * lds + c]) * scale : 0.f;
    __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[i] = h;
    if (lo != nullptr) lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
  }
}

void cast_pad_bf16(at::Tensor src, at::Tensor hi, c10::optional<at::Tensor> lo, double scale) {
  TORCH_CHECK(src.is_cuda() && src.dim() == 2 && src.stride(1) == 1, "src must be 2-D, unit col stride");
  TORCH_CHECK(hi.is_cuda() && hi.scalar_type() == at::kBFloat16 && hi.dim() == 2 &&
                  hi.is_contiguous() && hi.size(0) == src.size(0) && hi.size(1) >= src.size(1),
              "hi must be contiguous bf16 [rows, >= n]");
  __nv_bfloat16* lo_p = nullptr;
  if (lo.has_value()) {
    TORCH_CHECK(lo->sizes() == hi.sizes() && lo->is_contiguous() &&
                    lo->scalar_type() == at::kBFloat16, "lo must match hi");
    lo_p = reinterpret_cast<__nv_bfloat16*>(lo->data_ptr());
  }
  c10::cuda::CUDAGuard guard(src.get_device());
  const long long rows = src.size(0);
  const int n = static_cast<int>(src.size(1));
  const long long ldo = hi.size(1);
  const long long total = rows * ldo;
  if (total == 0) return;
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<long long>((total + threads - 1) / threads, 148 * 16));
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  auto* hi_p = reinterpret_cast<__nv_bfloat16*>(hi.data_ptr());
  if (src.scalar_type() == at::kFloat) {
    cast_pad_bf16_kernel<float><<<blocks, threads, 0, stream>>>(
        src.data_ptr<float>(), src.stride(0), static_cast<float>(scale), hi_p, lo_p, ldo, rows, n);
  } else if (src.scalar_type() == at::kBFloat16) {
    cast_pad_bf16_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(src.data_ptr()), src.stride(0),
        static_cast<float>(scale), hi_p, lo_p, ldo, rows, n);
  } else if (src.scalar_type() == at::kHalf) {
    cast_pad_bf16_kernel<__half><<<blocks, threads, 0, stream>>>(
        reinterpret_cast<const __half*>(src.data_ptr()), src.stride(0), static_cast<float>(scale),
        hi_p, lo_p, ldo, rows, n);
  } else {
    TORCH_CHECK(false, "unsupported source dtype");
  }
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// Three-way split of an fp32 matrix: v = hi + mid + lo with every part a bf16 number, which carries
// the full 24-bit significand of v.  Six tensor-core products of such parts (hi*hi, hi*mid, mid*hi,
// hi*lo, mid*mid, lo*hi) reproduce an fp32 product to ~2^-24.
__global__ void cast_split3_kernel(const float* __restrict__ src, long long lds, __nv_bfloat16* __restrict__ hi,
                                   __nv_bfloat16* __restrict__ mid, __nv_bfloat16* __restrict__ lo,
                                   long long ldo, long long rows, int n) {
  const long long total = rows * ldo;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / ldo;
    const int c = static_cast<int>(i - r * ldo);
    const float v = (c < n) ? src[r * lds + c] : 0.f;
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h);
    const __nv_bfloat16 m = __float2bfloat16_rn(r1);
    hi[i] = h;
    mid[i] = m;
    lo[i] = __float2bfloat16_rn(r1 - __bfloat162float(m));
  }
}

void cast_split3(at::Tensor src, at::Tensor hi, at::Tensor mid, at::Tensor lo) {
  TORCH_CHECK(src.is_cuda() && src.dim() == 2 && src.stride(1) == 1 && src.scalar_type() == at::kFloat,
              "src must be a 2-D fp32 CUDA tensor with unit column stride");
  for (const at::Tensor* t : {&hi, &mid, &lo})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16 && t->dim() == 2 && t->is_contiguous() &&
                    t->size(0) == src.size(0) && t->size(1) >= src.size(1) && t->sizes() == hi.sizes(),
                "outputs must be contiguous bf16 [rows, >= n] tensors of one shape");
  c10::cuda::CUDAGuard guard(src.get_device());
  const long long rows = src.size(0);
  const long long ldo = hi.size(1);
  if (rows == 0) return;
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const long long total = rows * ldo;
  const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148LL * 16));
  cast_split3_kernel<<<blocks, 256, 0, stream>>>(
      src.data_ptr<float>(), src.stride(0), reinterpret_cast<__nv_bfloat16*>(hi.data_ptr()),
      reinterpret_cast<__nv_bfloat16*>(mid.data_ptr()), reinterpret_cast<__nv_bfloat16*>(lo.data_ptr()), ldo, rows,
      static_cast<int>(src.size(1)));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// Grouped fp32 -> bf16 hi/lo staging: one launch converts many matrices.  Each table row holds
// (src fp32 ptr, hi ptr, lo ptr or 0, rows, n, src pitch, dst pitch) as int64.  blockIdx.y is the matrix;
// the grid is as wide as the largest matrix needs, so the CTAs of a small matrix past its end leave at once.
// Matrices whose rows are 16-byte aligned on both sides go eight elements per thread and trip (two 16-byte loads,
// one 16-byte store per part); the others one element at a time.
__global__ void __launch_bounds__(256) cast_pad_grouped_kernel(const long long* __restrict__ table) {
  const long long* e = table + static_cast<long long>(blockIdx.y) * 7;
  const float* src = reinterpret_cast<const float*>(e[0]);
  __nv_bfloat16* hi = reinterpret_cast<__nv_bfloat16*>(e[1]);
  __nv_bfloat16* lo = reinterpret_cast<__nv_bfloat16*>(e[2]);
  const long long rows = e[3], n = e[4], lds = e[5], ldo = e[6];
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const bool vec = ((n & 7) == 0) && ((ldo & 7) == 0) && ((lds & 3) == 0) &&
                   (((e[0] | e[1] | e[2]) & 15) == 0);
  if (vec) {
    const long long vpr = ldo >> 3, total = rows * vpr;
    for (long long v = first; v < total; v += step) {
      const long long r = v / vpr, c = (v - r * vpr) << 3;
      float x[8];
      if (c < n) {
        const float4 a = *reinterpret_cast<const float4*>(src + r * lds + c);
        const float4 b = *reinterpret_cast<const float4*>(src + r * lds + c + 4);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) x[k] = 0.f;
      }
      uint32_t ph[4], pl[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __nv_bfloat16 h0 = __float2bfloat16_rn(x[2 * k]), h1 = __float2bfloat16_rn(x[2 * k + 1]);
        const __nv_bfloat16 l0 = __float2bfloat16_rn(x[2 * k] - __bfloat162float(h0));
        const __nv_bfloat16 l1 = __float2bfloat16_rn(x[2 * k + 1] - __bfloat162float(h1));
        ph[k] = static_cast<uint32_t>(__bfloat16_as_ushort(h0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h1)) << 16);
        pl[k] = static_cast<uint32_t>(__bfloat16_as_ushort(l0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(l1)) << 16);
      }
      *reinterpret_cast<uint4*>(hi + (v << 3)) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
      if (lo != nullptr) *reinterpret_cast<uint4*>(lo + (v << 3)) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
    }
    return;
  }
  const long long total = rows * ldo;
  for (long long i = first; i < total; i += step) {
    const long long r = i / ldo;
    const long long c = i - r * ldo;
    const float v = (c < n) ? src[r * lds + c] : 0.f;
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[i] = h;
    if (lo != nullptr) lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
  }
}

// `max_elems`: rows x destination pitch of the largest matrix of the table (0: unknown, a narrow grid is used).
void cast_pad_bf16_grouped(at::Tensor table, int64_t count, int64_t max_elems) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.is_contiguous() &&
                  table.numel() == count * 7, "table must be a CUDA int64 [count, 7] tensor");
  if (count == 0) return;
  c10::cuda::CUDAGuard guard(table.get_device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  // eight elements per thread and at least two trips per thread for the largest matrix, at most 512 CTAs per matrix
  int gx = 32;
  if (max_elems > 0) gx = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((max_elems / 8 + 511) / 512, 512)));
  cast_pad_grouped_kernel<<<dim3(gx, static_cast<unsigned>(count)), 256, 0, stream>>>(
      reinterpret_cast<const long long*>(table.data_ptr<int64_t>()));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// Transposing cast bf16 -> fp32: dst[i][j] = float(src[j * src_ld + i]) for i < rows, j < cols.
// Weight gradients of linear layers leave autograd as transposed (column-major) bf16 tensors; this
// brings one into the row-major fp32 layout of the parameter in one coalesced pass (32 x 32 tiles
// through shared memory).  All arguments are kernel parameters, so the launch can be captured in a
// CUDA graph.
__global__ void transpose_cast_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst,
                                      long long rows, long long cols, long long lds, long long ldd) {
  __shared__ float tile[32][33];
  const long long tiles_r = (rows + 31) / 32, tiles_c = (cols + 31) / 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (long long t = blockIdx.x; t < tiles_r * tiles_c; t += gridDim.x) {
    const long long tr = t / tiles_c, tc = t - tr * tiles_c;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long j = tc * 32 + ty + 8 * k, i = tr * 32 + tx;
      tile[ty + 8 * k][tx] = (i < rows && j < cols) ? __bfloat162float(src[j * lds + i]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long i = tr * 32 + ty + 8 * k, j = tc * 32 + tx;
      if (i < rows && j < cols) dst[i * ldd + j] = tile[tx][ty + 8 * k];
    }
    __syncthreads();
  }
}

// src: bf16 [rows, cols] tensor with strides (1, ld) (a transposed matrix); dst: fp32 [rows, cols] row-major.
void transpose_cast(at::Tensor src, at::Tensor dst) {
  TORCH_CHECK(src.is_cuda() && dst.is_cuda() && src.dim() == 2 && dst.dim() == 2 && src.sizes() == dst.sizes(),
              "src and dst must be CUDA matrices of the same shape");
  TORCH_CHECK(src.scalar_type() == at::kBFloat16 && dst.scalar_type() == at::kFloat, "bf16 -> fp32 only");
  TORCH_CHECK(src.stride(0) == 1 && src.stride(1) >= src.size(0) && dst.stride(1) == 1 && dst.stride(0) >= dst.size(1),
              "src must be column-major and dst row-major");
  const long long rows = src.size(0), cols = src.size(1);
  if (rows == 0 || cols == 0) return;
  c10::cuda::CUDAGuard guard(src.get_device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const long long tiles = ((rows + 31) / 32) * ((cols + 31) / 32);
  const int grid = static_cast<int>(std::min<long long>(tiles, 148LL * 8));
  transpose_cast_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(src.data_ptr()),
                                                  dst.data_ptr<float>(), rows, cols, src.stride(1), dst.stride(0));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

struct Im2colParams {
  long long sN, sC, sH, sW;  // input strides in elements
  int N, C, H, W;
  int KH, KW, SH, SW, PH, PW, DH, DW;
  int Ho, Wo;
  long long ldo;   // output row pitch (elements), >= C*KH*KW
  int c_major;     // 1: columns ordered (c, kh, kw); 0: (kh, kw, c)
};

// Scalar path: one thread per output element (coalesced along the output row).
template <typename T>
__global__ void im2col_generic_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                      __nv_bfloat16* __restrict__ out_lo, Im2colParams p) {
  const long long rows = static_cast<long long>(p.N) * p.Ho * p.Wo;
  const long long total = rows * p.ldo;
  const int ncols = p.C * p.KH * p.KW;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / p.ldo;
    const int col = static_cast<int>(i - r * p.ldo);
    float v = 0.f;
    if (col < ncols) {
      int c, kh, kw;
      if (p.c_major) {
        c = col / (p.KH * p.KW);
        const int t = col - c * p.KH * p.KW;
        kh = t / p.KW;
        kw = t - kh * p.KW;
      } else {
        const int t = col / p.C;
        c = col - t * p.C;
        kh = t / p.KW;
        kw = t - kh * p.KW;
      }
      const int wo = static_cast<int>(r % p.Wo);
      const long long t2 = r / p.Wo;
      const int ho = static_cast<int>(t2 % p.Ho);
      const int n = static_cast<int>(t2 / p.Ho);
      const int hi = ho * p.SH - p.PH + kh * p.DH;
      const int wi = wo * p.SW - p.PW + kw * p.DW;
      if (hi >= 0 && hi < p.H && wi >= 0 && wi < p.W)
        v = to_f32<T>(x[n * p.sN + c * p.sC + hi * p.sH + wi * p.sW]);
    }
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    out[i] = h;
    if (out_lo != nullptr) out_lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
  }
}

// Vector path: channels_last bf16 input, C % 8 == 0, (kh, kw, c) column order.  One thread moves
// 8 channels (16 bytes) of one tap of one output pixel.
__global__ void im2col_nhwc_vec8_kernel(const __nv_bfloat16* __restrict__ x,
                                        __nv_bfloat16* __restrict__ out, Im2colParams p) {
  const int c8n = p.C >> 3;
  const int taps = p.KH * p.KW;
  const long long rows = static_cast<long long>(p.N) * p.Ho * p.Wo;
  const long long total = rows * taps * c8n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c8 = static_cast<int>(i % c8n);
    const long long t = i / c8n;
    const int tap = static_cast<int>(t % taps);
    const long long r = t / taps;
    const int kh = tap / p.KW, kw = tap - kh * p.KW;
    const int wo = static_cast<int>(r % p.Wo);
    const long long t2 = r / p.Wo;
    const int ho = static_cast<int>(t2 % p.Ho);
    const int n = static_cast<int>(t2 / p.Ho);
    const int hi = ho * p.SH - p.PH + kh * p.DH;
    const int wi = wo * p.SW - p.PW + kw * p.DW;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (hi >= 0 && hi < p.H && wi >= 0 && wi < p.W)
      v = *reinterpret_cast<const uint4*>(x + n * p.sN + hi * p.sH + wi * p.sW + c8 * 8);
    *reinterpret_cast<uint4*>(out + r * p.ldo + static_cast<long long>(tap) * p.C + c8 * 8) = v;
  }
}

// x: 4-D conv input [N, C, H, W] (logical), any memory format.  out: [N*Ho*Wo, ld] bf16, contiguous.
void im2col_bf16(at::Tensor x, at::Tensor out, c10::optional<at::Tensor> out_lo,
                 std::vector<int64_t> kernel, std::vector<int64_t> stride,
                 std::vector<int64_t> padding, std::vector<int64_t> dilation, bool c_major) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4, "x must be a 4-D CUDA tensor");
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == at::kBFloat16 &&
                  out.dim() == 2, "out must be contiguous 2-D bf16");
  Im2colParams p;
  p.N = x.size(0); p.C = x.size(1); p.H = x.size(2); p.W = x.size(3);
  p.sN = x.stride(0); p.sC = x.stride(1); p.sH = x.stride(2); p.sW = x.stride(3);
  p.KH = kernel[0]; p.KW = kernel[1]; p.SH = stride[0]; p.SW = stride[1];
  p.PH = padding[0]; p.PW = padding[1]; p.DH = dilation[0]; p.DW = dilation[1];
  p.Ho = (p.H + 2 * p.PH - p.DH * (p.KH - 1) - 1) / p.SH + 1;
  p.Wo = (p.W + 2 * p.PW - p.DW * (p.KW - 1) - 1) / p.SW + 1;
  p.ldo = out.size(1);
  p.c_major = c_major ? 1 : 0;
  const long long rows = static_cast<long long>(p.N) * p.Ho * p.Wo;
  TORCH_CHECK(out.size(0) == rows && p.ldo >= static_cast<long long>(p.C) * p.KH * p.KW,
              "out has the wrong shape");
  if (rows == 0) return;
  c10::cuda::CUDAGuard guard(x.get_device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  auto* out_p = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  __nv_bfloat16* lo_p = nullptr;
  if (out_lo.has_value()) {
    TORCH_CHECK(out_lo->sizes() == out.sizes() && out_lo->is_contiguous() &&
                    out_lo->scalar_type() == at::kBFloat16, "out_lo must match out");
    lo_p = reinterpret_cast<__nv_bfloat16*>(out_lo->data_ptr());
  }
  const int threads = 256;
  // with a single filter tap the (c, kh, kw) and (kh, kw, c) column orders are the same
  const bool vec = lo_p == nullptr && (!c_major || p.KH * p.KW == 1) && x.scalar_type() == at::kBFloat16 && p.sC == 1 && (p.C % 8) == 0 &&
                   p.ldo == static_cast<long long>(p.C) * p.KH * p.KW && (p.sW % 8) == 0 &&
                   (p.sH % 8) == 0 && (p.sN % 8) == 0 &&
                   (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0;
  if (vec) {
    const long long total = rows * p.KH * p.KW * (p.C >> 3);
    const int blocks = static_cast<int>(std::min<long long>((total + threads - 1) / threads, 148 * 32));
    im2col_nhwc_vec8_kernel<<<blocks, threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), out_p, p);
  } else {
    const long long total = rows * p.ldo;
    const int blocks = static_cast<int>(std::min<long long>((total + threads - 1) / threads, 148 * 32));
    if (x.scalar_type() == at::kFloat)
      im2col_generic_kernel<float><<<blocks, threads, 0, stream>>>(x.data_ptr<float>(), out_p, lo_p, p);
    else if (x.scalar_type() == at::kBFloat16)
      im2col_generic_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
          reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), out_p, lo_p, p);
    else if (x.scalar_type() == at::kHalf)
      im2col_generic_kernel<__half><<<blocks, threads, 0, stream>>>(
          reinterpret_cast<const __half*>(x.data_ptr()), out_p, lo_p, p);
    else
      TORCH_CHECK(false, "unsupported input dtype");
  }
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

}  // namespace b200
