// Batched symmetric eigendecomposition of small fp32 matrices (n <= 160) by the parallel cyclic
// two-sided Jacobi method, one CTA per matrix, everything in shared memory:
//     A = V diag(w) V^T,   w ascending (the convention of torch.linalg.eigh).
// A round rotates n/2 disjoint index pairs at once (round-robin tournament ordering, n - 1 rounds
// per sweep); sweeps repeat until the off-diagonal mass reaches the rounding floor (4 n eps of the
// diagonal's norm) or stops shrinking (at most 30 sweeps).  Jacobi rotations are backward stable and the eigenvalues come out with a small
// RELATIVE error, which suits the ill-conditioned curvature factors this is used for: the
// Kronecker-factored eigenbasis of small layers, the |H| of saddle-free Newton steps on small
// models, and the tridiagonal matrices of stochastic Lanczos quadrature.
//
// Stands in for the torch.linalg.eigh / eigvalsh calls of asdl/operations/linear.py:103-118,
// asdl/precondition/newton.py:43 and asdl/mvp.py:140 for matrices of these sizes.
#include "host_utils.h"
#include "sm100_ptx.cuh"

namespace b200 {

namespace {

constexpr int JN = 160;         // largest matrix: A and V (two (JN x (JN + 1)) fp32 arrays) fill 205 of the 227 KB of shared memory
constexpr int JP = JN + 1;      // shared-memory row pitch
constexpr int J_THREADS = 512;
constexpr int J_SMEM = (2 * JN * JP + 4 * JN) * static_cast<int>(sizeof(float)) + 2 * JN * static_cast<int>(sizeof(int));

// Position k (0 .. m-1) of round r of a round-robin tournament over m (even) players: player
// m - 1 stays, the others rotate.  Pairs are (top[k], bot[k]) with top = pos k, bot = pos m-1-k.
__device__ __forceinline__ int rr_player(int pos, int r, int m) {
  if (pos == m - 1) return m - 1;
  return (pos + r) % (m - 1);
}

__global__ void __launch_bounds__(J_THREADS, 1)
jacobi_eigh_kernel(const float* __restrict__ mats, float* __restrict__ evals, float* __restrict__ evecs, int n,
                   int want_vectors, int* status) {
  extern __shared__ float jsm[];
  float* A = jsm;                    // [JN][JP]
  float* V = A + JN * JP;            // [JN][JP]
  float* cs = V + JN * JP;           // cos[JN/2] | sin[JN/2] | reduction scratch [2 * JN]
  int* pp = reinterpret_cast<int*>(cs + 4 * JN);   // p[JN/2] | q[JN/2]
  const int tid = threadIdx.x;
  const float* src = mats + static_cast<size_t>(blockIdx.x) * n * n;
  const int m = (n + 1) & ~1;        // even number of players (a padding index rotates with nobody)
  for (int e = tid; e < m * m; e += J_THREADS) {
    const int r = e / m, c = e - r * m;
    // symmetrise on load: 0.5 (a_rc + a_cr)
    A[r * JP + c] = (r < n && c < n) ? 0.5f * (src[static_cast<size_t>(r) * n + c] + src[static_cast<size_t>(c) * n + r]) : 0.f;
    V[r * JP + c] = (r == c) ? 1.f : 0.f;
  }
  __syncthreads();
  const int half = m / 2;
  float* red = cs + 2 * JN;
  bool converged = false;
  float prev_off = 3.0e38f;
  const float tol = 16.f * static_cast<float>(n) * static_cast<float>(n) * 3.55e-15f;   // (4 n eps)^2
  for (int sweep = 0; sweep <= 30; ++sweep) {
    // convergence: off-diagonal against diagonal sum of squares
    float off = 0.f, dia = 0.f;
    for (int e = tid; e < n * n; e += J_THREADS) {
      const int r = e / n, c = e - r * n;
      const float v = A[r * JP + c];
      if (r == c)
        dia = fmaf(v, v, dia);
      else
        off = fmaf(v, v, off);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      off += __shfl_xor_sync(0xffffffffu, off, o);
      dia += __shfl_xor_sync(0xffffffffu, dia, o);
    }
    if ((tid & 31) == 0) {
      red[tid >> 5] = off;
      red[32 + (tid >> 5)] = dia;
    }
    __syncthreads();
    float off_t = 0.f, dia_t = 0.f;
    for (int w = 0; w < J_THREADS / 32; ++w) {
      off_t += red[w];
      dia_t += red[32 + w];
    }
    __syncthreads();
    // done at the rounding floor, or when a sweep no longer halves what is left (quadratic convergence
    // has ended, the rest is rounding noise)
    if (!(off_t > tol * dia_t) || n == 1 || (sweep >= 3 && off_t > 0.5f * prev_off && off_t < 1e-6f * dia_t)) {
      converged = true;
      break;
    }
    prev_off = off_t;
    if (sweep == 30) break;
    for (int r = 0; r < m - 1; ++r) {
      // rotation of every pair of this round
      if (tid < half) {
        int p = rr_player(tid, r, m), q = rr_player(m - 1 - tid, r, m);
        if (p > q) {
          const int t = p;
          p = q;
          q = t;
        }
        float c = 1.f, s = 0.f;
        if (q < n) {
          const float apq = A[p * JP + q];
          if (fabsf(apq) > 1e-37f) {
            const float tau = (A[q * JP + q] - A[p * JP + p]) / (2.f * apq);
            const float t = (tau >= 0.f ? 1.f : -1.f) / (fabsf(tau) + sqrtf(1.f + tau * tau));
            c = 1.f / sqrtf(1.f + t * t);   // correctly rounded: c^2 + s^2 = 1 to rounding, no drift of the norm
            s = t * c;
          }
        }
        cs[tid] = c;
        cs[JN + tid] = s;
        pp[tid] = p;
        pp[JN + tid] = q;
      }
      __syncthreads();
      // rows: A <- J^T A  (rows p and q of every pair, all columns)
      for (int e = tid; e < half * m; e += J_THREADS) {
        const int k = e / m, col = e - k * m;
        const int p = pp[k], q = pp[JN + k];
        const float c = cs[k], s = cs[JN + k];
        const float ap = A[p * JP + col], aq = A[q * JP + col];
        A[p * JP + col] = c * ap - s * aq;
        A[q * JP + col] = s * ap + c * aq;
      }
      __syncthreads();
      // columns: A <- A J, V <- V J  (columns p and q of every pair, all rows)
      for (int e = tid; e < half * m; e += J_THREADS) {
        const int k = e % half, row = e / half;
        const int p = pp[k], q = pp[JN + k];
        const float c = cs[k], s = cs[JN + k];
        const float ap = A[row * JP + p], aq = A[row * JP + q];
        A[row * JP + p] = c * ap - s * aq;
        A[row * JP + q] = s * ap + c * aq;
        const float vp = V[row * JP + p], vq = V[row * JP + q];
        V[row * JP + p] = c * vp - s * vq;
        V[row * JP + q] = s * vp + c * vq;
      }
      __syncthreads();
    }
  }
  if (!converged && tid == 0) set_error(status, ERR_BAD_ARG);   // no convergence in 30 sweeps (non-finite input)
  // ascending order: rank of every eigenvalue (ties broken by index)
  float* w = red;   // [JN] eigenvalues
  int* rank = pp;   // [JN]
  for (int i = tid; i < n; i += J_THREADS) w[i] = A[i * JP + i];
  __syncthreads();
  for (int i = tid; i < n; i += J_THREADS) {
    const float wi = w[i];
    int rk = 0;
    for (int j = 0; j < n; ++j) {
      const float wj = w[j];
      rk += (wj < wi || (wj == wi && j < i)) ? 1 : 0;
    }
    rank[i] = rk;
  }
  __syncthreads();
  float* ev = evals + static_cast<size_t>(blockIdx.x) * n;
  for (int i = tid; i < n; i += J_THREADS) ev[rank[i]] = w[i];
  if (want_vectors) {
    float* dst = evecs + static_cast<size_t>(blockIdx.x) * n * n;
    for (int e = tid; e < n * n; e += J_THREADS) {
      const int r = e / n, c = e - r * n;      // source column c goes to column rank[c]
      dst[static_cast<size_t>(r) * n + rank[c]] = V[r * JP + c];
    }
  }
}

}  // namespace

// mats: [batch, n, n] fp32 contiguous (n <= 160); returns (eigenvalues [batch, n] ascending, eigenvectors
// [batch, n, n] as columns, or an empty tensor when `want_vectors` is false).
std::vector<at::Tensor> jacobi_eigh(at::Tensor mats, bool want_vectors) {
  TORCH_CHECK(mats.is_cuda() && mats.scalar_type() == at::kFloat && mats.dim() == 3 && mats.size(1) == mats.size(2) &&
                  mats.is_contiguous(), "mats must be a contiguous fp32 CUDA tensor [batch, n, n]");
  const int64_t batch = mats.size(0), n = mats.size(1);
  TORCH_CHECK(n >= 1 && n <= JN, "the Jacobi kernel handles matrices up to ", JN, " x ", JN);
  const int dev = mats.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto evals = at::empty({batch, n}, mats.options());
  auto evecs = want_vectors ? at::empty({batch, n, n}, mats.options()) : at::empty({0}, mats.options());
  if (batch == 0) return {evals, evecs};
  static bool attr_set_on[64] = {false};
  if (!attr_set_on[dev & 63]) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(jacobi_eigh_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, J_SMEM));
    attr_set_on[dev & 63] = true;
  }
  jacobi_eigh_kernel<<<static_cast<unsigned>(batch), J_THREADS, J_SMEM, at::cuda::getCurrentCUDAStream(dev).stream()>>>(
      mats.data_ptr<float>(), evals.data_ptr<float>(), want_vectors ? evecs.data_ptr<float>() : nullptr,
      static_cast<int>(n), want_vectors ? 1 : 0, device_state(dev).status.data_ptr<int>());
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return {evals, evecs};
}

}  // namespace b200
