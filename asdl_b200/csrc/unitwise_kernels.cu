// Small curvature kernels that replace chains of elementwise PyTorch launches:
//
//   ln_unitwise_stats      unit-wise 2x2 curvature blocks of a LayerNorm from its output y and output
//                          gradient g ([rows, d]): per feature f
//                              [[sum (xh g)^2, sum xh g^2], [sum xh g^2, sum g^2]],  xh = (y - bias_f) / weight_f
//                          in one pass over y and g plus a tiny finalize (moving average folded in);
//                          stands in for asdl/operations/layernorm.py:70-78.
//   unitwise_inverse_mt    closed-form inverse of the damped 2x2 blocks of many layers in one launch
//                          (asdl/symmatrix.py:687-698);
//   unitwise_apply_mt      (weight.grad, bias.grad) <- inv . (weight.grad, bias.grad) for many layers in
//                          one launch (asdl/symmatrix.py:700-719);
//   bias_precondition_mt   bias.grad <- B^-1 bias.grad for many layers in one launch (one warp per row of
//                          B^-1; the K-FAC bias part of asdl/symmatrix.py:536-548);
//   diag_linear_stats      diagonal Fisher of a linear layer, sum_n g_n^2 (x) a_n^2, as one pass over
//                          rows with the squares formed in registers (asdl/operations/linear.py:57-66).
//
// "Multi-tensor" kernels take a table with one row of addresses per layer as a KERNEL PARAMETER (up to
// 256 layers per launch), so the launch count does not grow with the number of layers, nothing is
// copied to the device for a call, and a CUDA graph captures the table by value.
#include "host_utils.h"
#include "sm100_ptx.cuh"

namespace b200 {

namespace {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// grid: (column chunks of 256, row chunks); thread = one column, walks its chunk of rows
template <typename T>
__global__ void __launch_bounds__(256) ln_stats_partial(const T* __restrict__ y, const T* __restrict__ g,
                                                        const float* __restrict__ weight,
                                                        const float* __restrict__ bias, float* __restrict__ part,
                                                        long long rows, int d, long long rows_per_chunk) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= d) return;
  const long long r0 = blockIdx.y * rows_per_chunk;
  const long long r1 = (r0 + rows_per_chunk < rows) ? r0 + rows_per_chunk : rows;
  const float b = bias[c], iw = 1.f / weight[c];
  float ww = 0.f, wb = 0.f, bb = 0.f;
  for (long long r = r0; r < r1; ++r) {
    const float gv = to_f(g[r * d + c]);
    const float gw = (to_f(y[r * d + c]) - b) * iw * gv;
    ww = fmaf(gw, gw, ww);
    wb = fmaf(gw, gv, wb);
    bb = fmaf(gv, gv, bb);
  }
  float* p = part + (static_cast<size_t>(blockIdx.y) * d + c) * 3;
  p[0] = ww;
  p[1] = wb;
  p[2] = bb;
}

__global__ void ln_stats_finalize(const float* __restrict__ part, float* __restrict__ stats, int d, int chunks,
                                  float alpha, float beta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  double ww = 0.0, wb = 0.0, bb = 0.0;   // chunks are summed in a fixed order: deterministic
  for (int k = 0; k < chunks; ++k) {
    const float* p = part + (static_cast<size_t>(k) * d + c) * 3;
    ww += p[0];
    wb += p[1];
    bb += p[2];
  }
  float* s = stats + 4 * static_cast<size_t>(c);
  const float o0 = beta != 0.f ? beta * s[0] : 0.f, o1 = beta != 0.f ? beta * s[1] : 0.f;
  const float o2 = beta != 0.f ? beta * s[2] : 0.f, o3 = beta != 0.f ? beta * s[3] : 0.f;
  s[0] = o0 + alpha * static_cast<float>(ww);
  s[1] = o1 + alpha * static_cast<float>(wb);
  s[2] = o2 + alpha * static_cast<float>(wb);
  s[3] = o3 + alpha * static_cast<float>(bb);
}

constexpr int MT_MAX = 256;
struct MtTable {
  long long rows[MT_MAX][4];
};

// table rows: (stats ptr, inv ptr, features)
__global__ void unitwise_inverse_kernel(const __grid_constant__ MtTable table, float damping) {
  const long long* e = table.rows[blockIdx.y];
  const float* s = reinterpret_cast<const float*>(e[0]);
  float* inv = reinterpret_cast<float*>(e[1]);
  const long long f = e[2];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < f;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 m = *reinterpret_cast<const float4*>(s + 4 * i);
    const float a = m.x + damping, b = m.y, c = m.z, d = m.w + damping;
    const float r = 1.f / (a * d - b * c);
    *reinterpret_cast<float4*>(inv + 4 * i) = make_float4(d * r, -b * r, -c * r, a * r);
  }
}

// table rows: (inv ptr, weight.grad ptr, bias.grad ptr, features)
__global__ void unitwise_apply_kernel(const __grid_constant__ MtTable table, float grad_scale) {
  const long long* e = table.rows[blockIdx.y];
  const float* inv = reinterpret_cast<const float*>(e[0]);
  float* gw = reinterpret_cast<float*>(e[1]);
  float* gb = reinterpret_cast<float*>(e[2]);
  const long long f = e[3];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < f;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 m = *reinterpret_cast<const float4*>(inv + 4 * i);
    const float w = gw[i] * grad_scale, b = gb[i] * grad_scale;
    gw[i] = fmaf(m.x, w, m.y * b);
    gb[i] = fmaf(m.z, w, m.w * b);
  }
}

// table rows: (B^-1 ptr (n x n, contiguous), bias.grad ptr, scratch ptr, n); one warp per row of B^-1.
// The products go to the scratch vector first (every row needs the whole old vector); the second
// kernel copies them back.
__global__ void __launch_bounds__(256) bias_mv_kernel(const __grid_constant__ MtTable table, float grad_scale) {
  const long long* e = table.rows[blockIdx.y];
  const float* binv = reinterpret_cast<const float*>(e[0]);
  const float* b = reinterpret_cast<const float*>(e[1]);
  float* out = reinterpret_cast<float*>(e[2]);
  const int n = static_cast<int>(e[3]);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = blockIdx.x * 8 + warp; r < n; r += gridDim.x * 8) {
    const float* row = binv + static_cast<size_t>(r) * n;
    float acc = 0.f;
    for (int c = lane; c < n; c += 32) acc = fmaf(row[c], b[c], acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[r] = acc * grad_scale;
  }
}
__global__ void bias_copy_kernel(const __grid_constant__ MtTable table) {
  const long long* e = table.rows[blockIdx.y];
  float* b = reinterpret_cast<float*>(e[1]);
  const float* out = reinterpret_cast<const float*>(e[2]);
  const int n = static_cast<int>(e[3]);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) b[i] = out[i];
}

// out[o][i] (+)= sum_r g[r][o]^2 a[r][i]^2 ; grid: (in tiles of 64, out tiles of 64); 256 threads, 4 x 4 each
template <typename T>
__global__ void __launch_bounds__(256) diag_linear_kernel(const T* __restrict__ a, const T* __restrict__ g,
                                                          float* __restrict__ out, float* __restrict__ out_bias,
                                                          long long rows, int d_in, int d_out, float alpha, float beta) {
  __shared__ float sa[32][64];
  __shared__ float sg[32][64];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int i0 = blockIdx.x * 64, o0 = blockIdx.y * 64;
  float acc[4][4] = {};
  float accb[4] = {};
  for (long long r0 = 0; r0 < rows; r0 += 32) {
    for (int e = threadIdx.x; e < 32 * 64; e += 256) {
      const int rr = e >> 6, cc = e & 63;
      const long long r = r0 + rr;
      float va = 0.f, vg = 0.f;
      if (r < rows) {
        if (i0 + cc < d_in) va = to_f(a[r * d_in + i0 + cc]);
        if (o0 + cc < d_out) vg = to_f(g[r * d_out + o0 + cc]);
      }
      sa[rr][cc] = va * va;
      sg[rr][cc] = vg * vg;
    }
    __syncthreads();
#pragma unroll 8
    for (int rr = 0; rr < 32; ++rr) {
      float av[4], gv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        av[u] = sa[rr][tx + 16 * u];
        gv[u] = sg[rr][ty + 16 * u];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (tx == 0) accb[u] += gv[u];
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] = fmaf(gv[u], av[v], acc[u][v]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int o = o0 + ty + 16 * u;
    if (o >= d_out) continue;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int i = i0 + tx + 16 * v;
      if (i < d_in) {
        float* p = out + static_cast<size_t>(o) * d_in + i;
        *p = (beta != 0.f ? beta * *p : 0.f) + alpha * acc[u][v];
      }
    }
    if (out_bias != nullptr && tx == 0 && blockIdx.x == 0)
      out_bias[o] = (beta != 0.f ? beta * out_bias[o] : 0.f) + alpha * accb[u];
  }
}

int sms(int dev) { return at::cuda::getDeviceProperties(dev)->multiProcessorCount; }

// Packs rows [begin, begin + MT_MAX) of `rows` (each with `cols` entries) into a kernel-parameter table.
int pack_table(const std::vector<std::vector<int64_t>>& rows, size_t begin, int cols, MtTable& t) {
  const int n = static_cast<int>(std::min<size_t>(MT_MAX, rows.size() - begin));
  for (int i = 0; i < n; ++i) {
    TORCH_CHECK(static_cast<int>(rows[begin + i].size()) == cols, "every table row needs ", cols, " entries");
    for (int c = 0; c < 4; ++c) t.rows[i][c] = c < cols ? rows[begin + i][c] : 0;
  }
  return n;
}

int current_device() {
  int dev = 0;
  B200_CUDA_CHECK(cudaGetDevice(&dev));
  return dev;
}

}  // namespace

void ln_unitwise_stats(at::Tensor y, at::Tensor g, at::Tensor weight, at::Tensor bias, at::Tensor stats, double alpha,
                       double beta) {
  TORCH_CHECK(y.is_cuda() && g.is_cuda() && y.dim() == 2 && y.sizes() == g.sizes() && y.is_contiguous() &&
                  g.is_contiguous() && y.scalar_type() == g.scalar_type(), "y and g must be contiguous [rows, d] CUDA tensors");
  const bool bf16 = y.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf16 || y.scalar_type() == at::kFloat, "y must be bf16 or fp32");
  const long long rows = y.size(0);
  const int d = static_cast<int>(y.size(1));
  TORCH_CHECK(weight.is_cuda() && bias.is_cuda() && weight.scalar_type() == at::kFloat && bias.scalar_type() == at::kFloat &&
                  weight.is_contiguous() && bias.is_contiguous() && weight.numel() == d && bias.numel() == d,
              "weight / bias must be contiguous fp32 [d]");
  TORCH_CHECK(stats.is_cuda() && stats.scalar_type() == at::kFloat && stats.is_contiguous() && stats.numel() == 4LL * d,
              "stats must be a contiguous fp32 [d, 2, 2] tensor");
  if (rows == 0 || d == 0) return;
  const int dev = y.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  const int col_chunks = (d + 255) / 256;
  int chunks = std::max(1, (4 * sms(dev)) / col_chunks);
  chunks = static_cast<int>(std::min<long long>(chunks, (rows + 15) / 16));
  const long long per = (rows + chunks - 1) / chunks;
  chunks = static_cast<int>((rows + per - 1) / per);
  auto part = at::empty({chunks, d, 3}, stats.options());
  dim3 grid(col_chunks, chunks);
  if (bf16)
    ln_stats_partial<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(y.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(g.data_ptr()),
        weight.data_ptr<float>(), bias.data_ptr<float>(), part.data_ptr<float>(), rows, d, per);
  else
    ln_stats_partial<float><<<grid, 256, 0, stream>>>(y.data_ptr<float>(), g.data_ptr<float>(), weight.data_ptr<float>(),
                                                      bias.data_ptr<float>(), part.data_ptr<float>(), rows, d, per);
  ln_stats_finalize<<<(d + 255) / 256, 256, 0, stream>>>(part.data_ptr<float>(), stats.data_ptr<float>(), d, chunks,
                                                         static_cast<float>(alpha), static_cast<float>(beta));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch(2);
}

// rows: (address of the [f, 2, 2] blocks, address of the [f, 2, 2] inverses, f); fp32, contiguous, on the current device
void unitwise_inverse_mt(std::vector<std::vector<int64_t>> rows, double damping) {
  const int dev = current_device();
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  for (size_t begin = 0; begin < rows.size(); begin += MT_MAX) {
    MtTable t;
    const int n = pack_table(rows, begin, 3, t);
    unitwise_inverse_kernel<<<dim3(8, n), 256, 0, stream>>>(t, static_cast<float>(damping));
    B200_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
}

// rows: (address of the [f, 2, 2] inverses, of weight.grad [f], of bias.grad [f], f)
void unitwise_apply_mt(std::vector<std::vector<int64_t>> rows, double grad_scale) {
  const int dev = current_device();
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  for (size_t begin = 0; begin < rows.size(); begin += MT_MAX) {
    MtTable t;
    const int n = pack_table(rows, begin, 4, t);
    unitwise_apply_kernel<<<dim3(8, n), 256, 0, stream>>>(t, static_cast<float>(grad_scale));
    B200_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
}

// rows: (address of B^-1 [n, n] contiguous, of bias.grad [n], of a scratch vector [n], n)
void bias_precondition_mt(std::vector<std::vector<int64_t>> rows, double grad_scale) {
  const int dev = current_device();
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  for (size_t begin = 0; begin < rows.size(); begin += MT_MAX) {
    MtTable t;
    const int n = pack_table(rows, begin, 4, t);
    int64_t n_max = 1;
    for (int i = 0; i < n; ++i) n_max = std::max<int64_t>(n_max, t.rows[i][3]);
    const unsigned gx = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((n_max + 7) / 8, 64)));
    bias_mv_kernel<<<dim3(gx, n), 256, 0, stream>>>(t, static_cast<float>(grad_scale));
    bias_copy_kernel<<<dim3(4, n), 256, 0, stream>>>(t);
    B200_CUDA_CHECK(cudaGetLastError());
    count_launch(2);
  }
}

void diag_linear_stats(at::Tensor a, at::Tensor g, at::Tensor out, c10::optional<at::Tensor> out_bias, double alpha,
                       double beta) {
  TORCH_CHECK(a.is_cuda() && g.is_cuda() && a.dim() == 2 && g.dim() == 2 && a.size(0) == g.size(0) && a.is_contiguous() &&
                  g.is_contiguous() && a.scalar_type() == g.scalar_type(), "a [rows, in] and g [rows, out] must be contiguous");
  const bool bf16 = a.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf16 || a.scalar_type() == at::kFloat, "a must be bf16 or fp32");
  const long long rows = a.size(0);
  const int d_in = static_cast<int>(a.size(1)), d_out = static_cast<int>(g.size(1));
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous() && out.dim() == 2 &&
                  out.size(0) == d_out && out.size(1) == d_in, "out must be a contiguous fp32 [out, in] tensor");
  float* ob = nullptr;
  if (out_bias.has_value()) {
    TORCH_CHECK(out_bias->is_cuda() && out_bias->scalar_type() == at::kFloat && out_bias->is_contiguous() &&
                    out_bias->numel() == d_out, "out_bias must be a contiguous fp32 [out] tensor");
    ob = out_bias->data_ptr<float>();
  }
  const int dev = a.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  dim3 grid((d_in + 63) / 64, (d_out + 63) / 64);
  if (bf16)
    diag_linear_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(a.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(g.data_ptr()),
        out.data_ptr<float>(), ob, rows, d_in, d_out, static_cast<float>(alpha), static_cast<float>(beta));
  else
    diag_linear_kernel<float><<<grid, 256, 0, stream>>>(a.data_ptr<float>(), g.data_ptr<float>(), out.data_ptr<float>(), ob,
                                                        rows, d_in, d_out, static_cast<float>(alpha), static_cast<float>(beta));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

}  // namespace b200

// ---- batched matrix-vector product: y[b] = A[b] x[b] for b matrices of one size -----------------------
// The power iteration of Shampoo's inverse roots (asdl/precondition/shampoo.py:532-558) is a chain of such
// products on a batch of statistics; one warp takes one row, so a step reads every matrix exactly once.
namespace b200 {
namespace {
__global__ void __launch_bounds__(256) batched_mv_kernel(const float* __restrict__ a, const float* __restrict__ x,
                                                         float* __restrict__ y, int n) {
  const float* A = a + static_cast<size_t>(blockIdx.y) * n * n;
  const float* xv = x + static_cast<size_t>(blockIdx.y) * n;
  float* yv = y + static_cast<size_t>(blockIdx.y) * n;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = blockIdx.x * 8 + warp; r < n; r += gridDim.x * 8) {
    const float* row = A + static_cast<size_t>(r) * n;
    float acc = 0.f;
    if ((n & 3) == 0) {
      for (int c = 4 * lane; c < n; c += 128) {
        const float4 av = *reinterpret_cast<const float4*>(row + c);
        const float4 xx = *reinterpret_cast<const float4*>(xv + c);
        acc = fmaf(av.x, xx.x, fmaf(av.y, xx.y, fmaf(av.z, xx.z, fmaf(av.w, xx.w, acc))));
      }
    } else {
      for (int c = lane; c < n; c += 32) acc = fmaf(row[c], xv[c], acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) yv[r] = acc;
  }
}
}  // namespace

// a: [b, n, n] fp32 contiguous, x: [b, n]; returns [b, n]
at::Tensor batched_mv(at::Tensor a, at::Tensor x) {
  TORCH_CHECK(a.is_cuda() && x.is_cuda() && a.scalar_type() == at::kFloat && x.scalar_type() == at::kFloat && a.dim() == 3 &&
                  a.size(1) == a.size(2) && x.dim() == 2 && x.size(0) == a.size(0) && x.size(1) == a.size(1) &&
                  a.is_contiguous() && x.is_contiguous(), "a [b, n, n] and x [b, n] must be contiguous fp32 CUDA tensors");
  const int dev = a.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto y = at::empty_like(x);
  const int n = static_cast<int>(a.size(1));
  if (a.size(0) == 0 || n == 0) return y;
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0,
              "16-byte alignment required");
  const unsigned gx = static_cast<unsigned>(std::max(1, std::min((n + 7) / 8, 128)));
  batched_mv_kernel<<<dim3(gx, static_cast<unsigned>(a.size(0))), 256, 0, at::cuda::getCurrentCUDAStream(dev).stream()>>>(
      a.data_ptr<float>(), x.data_ptr<float>(), y.data_ptr<float>(), n);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return y;
}
}  // namespace b200
