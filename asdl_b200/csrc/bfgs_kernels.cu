// K-BFGS building blocks on a dense fp32 inverse-Hessian approximation H [n, n] (n up to a few thousand):
//   bfgs_powell_damping  Powell's damping of the pair (s, y) followed by the Levenberg-Marquardt shift
//                        of y (asdl/precondition/kbfgs.py:177-190): Hy = H y by one warp per row, then one
//                        block forms the dot products and rewrites s and y.
//   bfgs_inv_update      the rank-2 BFGS update of H (asdl/precondition/kbfgs.py:193-217): one kernel
//                        symmetrises H in place tile by tile and accumulates Hy from the symmetrised
//                        tiles while they are in shared memory, one block forms the scalars and decides on
//                        the device whether the pair carries usable curvature, one kernel applies
//                        H += c1 s s^T - c2 (Hy s^T + s Hy^T).  Nothing is read back by the host.
#include "host_utils.h"

namespace b200 {

namespace {

constexpr int BT = 32;   // tile edge of the symmetrise + mat-vec kernel

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// block-wide sum of `k` running values per thread (k <= 5); result valid in every thread
template <int K>
__device__ __forceinline__ void block_sum(float (&v)[K], float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int i = 0; i < K; ++i) v[i] = warp_sum(v[i]);
  __syncthreads();
  if (lane == 0)
    for (int i = 0; i < K; ++i) red[i * 32 + warp] = v[i];
  __syncthreads();
#pragma unroll
  for (int i = 0; i < K; ++i) {
    float t = 0.f;
    for (int w = 0; w < nw; ++w) t += red[i * 32 + w];
    v[i] = t;
  }
}

// Hy[r] = sum_c H[r, c] y[c], one warp per row
__global__ void __launch_bounds__(256)
mv_rows_kernel(const float* __restrict__ H, const float* __restrict__ y, float* __restrict__ Hy, int n, int64_t ld) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n) return;
  const float* row = H + static_cast<int64_t>(r) * ld;
  float acc = 0.f;
  for (int c = lane; c < n; c += 32) acc = fmaf(row[c], y[c], acc);
  acc = warp_sum(acc);
  if (lane == 0) Hy[r] = acc;
}

// theta = (1 - mu1) y'Hy / (y'Hy - s'y) when s'y < mu1 y'Hy (and the gap is positive), else 1;
// s <- theta s + (1 - theta) Hy;  y <- y + mu2 s
__global__ void __launch_bounds__(1024)
powell_kernel(float* __restrict__ s, float* __restrict__ y, const float* __restrict__ Hy, int n, float mu1, float mu2) {
  __shared__ float red[2 * 32];
  float v[2] = {0.f, 0.f};
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    v[0] = fmaf(y[i], Hy[i], v[0]);
    v[1] = fmaf(s[i], y[i], v[1]);
  }
  block_sum<2>(v, red);
  const float ytHy = v[0], sty = v[1], gap = ytHy - sty;
  const float theta = (sty < mu1 * ytHy && gap > 0.f) ? (1.f - mu1) * ytHy / fmaxf(gap, 1e-30f) : 1.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float si = theta * s[i] + (1.f - theta) * Hy[i];
    s[i] = si;
    y[i] += mu2 * si;
  }
}

// Tile pair (bi >= bj): H <- (H + H^T) / 2 on both tiles and Hy += sym(H) y from the tiles in shared memory.
__global__ void __launch_bounds__(BT * 8)
sym_mv_kernel(float* __restrict__ H, const float* __restrict__ y, float* __restrict__ Hy, int n, int64_t ld) {
  __shared__ float S[BT][BT + 1];
  // linear block index -> (bi, bj) with bj <= bi
  int bi = static_cast<int>((sqrtf(8.f * static_cast<float>(blockIdx.x) + 1.f) - 1.f) * 0.5f);
  while ((bi + 1) * (bi + 2) / 2 <= static_cast<int>(blockIdx.x)) ++bi;
  while (bi * (bi + 1) / 2 > static_cast<int>(blockIdx.x)) --bi;
  const int bj = static_cast<int>(blockIdx.x) - bi * (bi + 1) / 2;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  const int r0 = bi * BT, c0 = bj * BT;
  // S[i][j] = 0.5 (H[r0 + i, c0 + j] + H[c0 + j, r0 + i])
#pragma unroll
  for (int k = 0; k < BT / 8; ++k) {
    const int i = ty + 8 * k;
    const int r = r0 + i, c = c0 + tx;
    S[i][tx] = (r < n && c < n) ? H[static_cast<int64_t>(r) * ld + c] : 0.f;
  }
  __syncthreads();
  float low[BT / 8];
#pragma unroll
  for (int k = 0; k < BT / 8; ++k) {
    // element (j = ty + 8k, i = tx) of the transposed tile, read coalesced along the row of the upper tile
    const int j = ty + 8 * k;
    const int r = c0 + j, c = r0 + tx;
    const float up = (r < n && c < n) ? H[static_cast<int64_t>(r) * ld + c] : 0.f;
    low[k] = 0.5f * (S[tx][j] + up);
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < BT / 8; ++k) S[tx][ty + 8 * k] = low[k];
  __syncthreads();
  // write both tiles back
#pragma unroll
  for (int k = 0; k < BT / 8; ++k) {
    const int i = ty + 8 * k;
    const int r = r0 + i, c = c0 + tx;
    if (r < n && c < n) H[static_cast<int64_t>(r) * ld + c] = S[i][tx];
    const int r2 = c0 + i, c2 = r0 + tx;
    if (bi != bj && r2 < n && c2 < n) H[static_cast<int64_t>(r2) * ld + c2] = S[tx][i];
  }
  // Hy[r0 + i] += sum_j S[i][j] y[c0 + j];  and for off-diagonal pairs Hy[c0 + j] += sum_i S[i][j] y[r0 + i]
  if (ty < 4) {
    const int i = ty * 8 + (tx >> 2);   // 4 lanes per row
    float acc = 0.f;
    for (int j = (tx & 3); j < BT; j += 4) acc = fmaf(S[i][j], (c0 + j < n) ? y[c0 + j] : 0.f, acc);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if ((tx & 3) == 0 && r0 + i < n) atomicAdd(Hy + r0 + i, acc);
  } else if (bi != bj) {
    const int j = (ty - 4) * 8 + (tx >> 2);
    float acc = 0.f;
    for (int i = (tx & 3); i < BT; i += 4) acc = fmaf(S[i][j], (r0 + i < n) ? y[r0 + i] : 0.f, acc);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if ((tx & 3) == 0 && c0 + j < n) atomicAdd(Hy + c0 + j, acc);
  }
}

// coef[0] = (s'y + y'Hy) / (s'y)^2, coef[1] = 1 / s'y; both 0 when the pair carries no usable curvature
__global__ void __launch_bounds__(1024)
bfgs_scalars_kernel(const float* __restrict__ s, const float* __restrict__ y, const float* __restrict__ Hy, int n,
                    float* __restrict__ coef) {
  __shared__ float red[5 * 32];
  float v[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float si = s[i], yi = y[i], hi = Hy[i];
    v[0] = fmaf(si, yi, v[0]);
    v[1] = fmaf(yi, hi, v[1]);
    v[2] = fmaf(si, si, v[2]);
    v[3] = fmaf(yi, yi, v[3]);
    v[4] = fmaf(hi, hi, v[4]);
  }
  block_sum<5>(v, red);
  if (threadIdx.x == 0) {
    const float sty = v[0], ytHy = v[1];
    const bool finite = isfinite(sty) && isfinite(ytHy) && isfinite(v[2]) && isfinite(v[3]) && isfinite(v[4]);
    const bool ok = finite && sty > 1e-12f * (1.f + sqrtf(v[2]) * sqrtf(v[3]));
    const float c1 = ok ? (sty + ytHy) / (sty * sty) : 0.f, c2 = ok ? 1.f / sty : 0.f;
    const bool fin2 = isfinite(c1) && isfinite(c2) && isfinite(c1 * v[2]) && isfinite(c2 * sqrtf(v[4]) * sqrtf(v[2]));
    coef[0] = fin2 ? c1 : 0.f;
    coef[1] = fin2 ? c2 : 0.f;
  }
}

__global__ void __launch_bounds__(256)
bfgs_rank2_kernel(float* __restrict__ H, const float* __restrict__ s, const float* __restrict__ Hy,
                  const float* __restrict__ coef, int n, int64_t ld) {
  const float c1 = coef[0], c2 = coef[1];
  if (c1 == 0.f && c2 == 0.f) return;
  const int c = blockIdx.x * 32 + (threadIdx.x & 31);
  const int rb = blockIdx.y * 32 + (threadIdx.x >> 5);
  if (c >= n) return;
  const float sc = s[c], hc = Hy[c];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = rb + 8 * k;
    if (r < n) {
      const float sr = s[r], hr = Hy[r];
      // every term is rounded on its own (no fused multiply-adds), so entries (r, c) and (c, r) get the
      // same increment and a symmetric H stays exactly symmetric
      const float cross = __fadd_rn(__fmul_rn(hr, sc), __fmul_rn(sr, hc));
      const float inc = __fadd_rn(__fmul_rn(c1, __fmul_rn(sr, sc)), -__fmul_rn(c2, cross));
      H[static_cast<int64_t>(r) * ld + c] = __fadd_rn(H[static_cast<int64_t>(r) * ld + c], inc);
    }
  }
}

void check_hsy(const at::Tensor& H, const at::Tensor& s, const at::Tensor& y) {
  TORCH_CHECK(H.is_cuda() && H.scalar_type() == at::kFloat && H.dim() == 2 && H.size(0) == H.size(1) && H.stride(1) == 1,
              "H must be a square fp32 CUDA matrix with unit column stride");
  for (const at::Tensor* v : {&s, &y})
    TORCH_CHECK(v->is_cuda() && v->scalar_type() == at::kFloat && v->dim() == 1 && v->size(0) == H.size(0) && v->is_contiguous(),
                "s and y must be contiguous fp32 CUDA vectors of H's dimension");
}

}  // namespace

// s <- theta s + (1 - theta) H y,  y <- y + mu2 s  (in place)
void bfgs_powell_damping(at::Tensor H, at::Tensor s, at::Tensor y, double mu1, double mu2) {
  check_hsy(H, s, y);
  const int n = static_cast<int>(H.size(0));
  if (n == 0) return;
  const int dev = H.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  auto Hy = at::empty({n}, s.options());
  mv_rows_kernel<<<(n + 7) / 8, 256, 0, stream>>>(H.data_ptr<float>(), y.data_ptr<float>(), Hy.data_ptr<float>(), n, H.stride(0));
  powell_kernel<<<1, 1024, 0, stream>>>(s.data_ptr<float>(), y.data_ptr<float>(), Hy.data_ptr<float>(), n,
                                        static_cast<float>(mu1), static_cast<float>(mu2));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch(2);
}

// H <- sym(H) + (s'y + y'Hy) s s^T / (s'y)^2 - (Hy s^T + s Hy^T) / s'y  (in place; H only symmetrised when
// the pair carries no usable curvature)
void bfgs_inv_update(at::Tensor H, at::Tensor s, at::Tensor y) {
  check_hsy(H, s, y);
  const int n = static_cast<int>(H.size(0));
  if (n == 0) return;
  const int dev = H.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  auto work = at::zeros({n + 2}, s.options());   // Hy | coef
  float* Hy = work.data_ptr<float>();
  float* coef = Hy + n;
  const int nb = (n + BT - 1) / BT;
  sym_mv_kernel<<<nb * (nb + 1) / 2, BT * 8, 0, stream>>>(H.data_ptr<float>(), y.data_ptr<float>(), Hy, n, H.stride(0));
  bfgs_scalars_kernel<<<1, 1024, 0, stream>>>(s.data_ptr<float>(), y.data_ptr<float>(), Hy, n, coef);
  bfgs_rank2_kernel<<<dim3(nb, nb), 256, 0, stream>>>(H.data_ptr<float>(), s.data_ptr<float>(), Hy, coef, n, H.stride(0));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch(3);
}

}  // namespace b200
