// Grouped fp32-accurate inverse of damped symmetric positive-definite matrices on the tensor cores:
//     out_m = (A_m + damping_m * I)^-1        for m = 0 .. count-1, sizes n_m arbitrary.
//
// Blocked right-looking Cholesky with 128-wide panels, triangular inverse by recursive doubling,
// then X^T X.  Every O(n^3) product runs on the persistent tcgen05 GEMM (umma_gemm2.cuh) from
// three-way bf16 splits of the fp32 values (v = hi + mid + lo carries the whole significand; the
// kernel's "split3" flavour issues the six significant part products small-magnitude-first and
// sums the contraction in fp32 registers, one 64-wide K block per TMEM chunk), and every
// subtraction between products happens in fp32 on the CUDA cores: the trailing update of a
// right-looking factorisation is a K = 128 product subtracted from the fp32 matrix in the GEMM
// epilogue.  Only the 128 x 128 diagonal blocks are factored and inverted on the CUDA cores (one
// CTA each, the block held in registers as 8 x 8 cyclic tiles of a 16 x 16 thread grid).
//
//   potrf, step k:  diag(k):   L_kk = chol(A_kk), T_k = L_kk^-1                  (CUDA cores)
//                   panel(k):  L_ik = A_ik T_k^T                  for i > k      (GEMM, K = 128)
//                   trail(k):  A_ij -= L_ik L_jk^T                for k < j <= i (GEMM, K = 128)
//   trtri, level l: blocks of s = 2^l panels are merged pairwise:
//                   W   = L_21 X_11,   X_21 = -X_22 W                            (two GEMM launches)
//   lauum:          out = X^T X  (lower tiles, mirrored)                         (one GEMM launch)
//
// All matrices of a call advance through the same launches ("grouped"): a launch's work list
// holds the tiles of every matrix that has work at that step.  Problem tables, work lists and the
// bf16 split buffers depend only on the addresses and sizes of the matrices; they are built once
// and cached, so a repeated call (the K-FAC state) issues no host-to-device copy and can be
// captured in a CUDA graph.  Inputs are not modified; a non-positive pivot sets the status word to
// ERR_NOT_SPD and the factorisation continues with pivot 1.
//
// Stands in for asdl/utils.py:91-96 (torch.linalg.cholesky + cholesky_inverse).
#include <cstring>
#include <list>

#include "gemm2_host.h"

namespace b200 {

namespace {

constexpr int TB = 128;  // panel width

struct TcMat {
  const float* A;         // input n x n (ld = lda)
  float* L;               // n x n fp32 work matrix (the output buffer)
  __nv_bfloat16* Ls[3];   // splits of L (strictly-lower blocks) / of the current panel column
  __nv_bfloat16* Xs[3];   // splits of X = L^-1 (lower triangular)
  int n, nb, lda, ldp, orig, pad;
};

__device__ __forceinline__ void split3_store(__nv_bfloat16* const* parts, size_t idx, float v) {
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  const float r1 = v - __bfloat162float(h);
  const __nv_bfloat16 m = __float2bfloat16_rn(r1);
  const __nv_bfloat16 l = __float2bfloat16_rn(r1 - __bfloat162float(m));
  parts[0][idx] = h;
  parts[1][idx] = m;
  parts[2][idx] = l;
}

// ---- phase 0: L = A + damping * I, splits of block column 0 -----------------------------------
// grid: (row groups, matrices); a warp walks along one row
__global__ void __launch_bounds__(256) tc_prepare_kernel(const TcMat* mats, const float* damping) {
  const TcMat M = mats[blockIdx.y];
  const float d = damping[M.orig];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = blockIdx.x * 8 + warp; r < M.n; r += gridDim.x * 8) {
    const float* src = M.A + static_cast<size_t>(r) * M.lda;
    float* dst = M.L + static_cast<size_t>(r) * M.n;
    for (int c = lane; c < M.n; c += 32) {
      float v = src[c];
      if (r == c) v += d;
      dst[c] = v;
      if (c < TB && r >= TB) split3_store(M.Ls, static_cast<size_t>(r) * M.ldp + c, v);
    }
  }
}

// ---- diagonal block k: Cholesky factor and its inverse ----------------------------------------
// 256 threads form a 16 x 16 grid; thread (ty, tx) keeps the entries (ty + 16u, tx + 16v), u, v = 0..7,
// of the block and of the inverse in registers (a cyclic layout keeps every thread busy while the
// active part shrinks).  One pass of 128 column steps does both: at step j the owners of column j of
// the block and of row j of the right-hand side publish them through shared memory; everybody scales
// them (L[:, j] and T[j, :] are final now) and updates its own entries of the trailing block and of
// the rows of the right-hand side below j.  One barrier per step: the exchange buffers are
// double-buffered.  This chain of 128 dependent steps is the critical path of every panel step, so
// the pivot's reciprocal square root comes from the fast instruction plus one Newton step.
__global__ void __launch_bounds__(256, 1) tc_diag_kernel(const TcMat* mats, int k, int* status) {
  const TcMat M = mats[blockIdx.x];
  if (k >= M.nb) return;
  __shared__ float colbuf[2][TB];
  __shared__ float rowbuf[2][TB];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int r0 = k * TB;
  float a[8][8], t[8][8];
#pragma unroll
  for (int u = 0; u < 8; ++u)
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      const int r = ty + 16 * u, c = tx + 16 * v;
      const int gr = r0 + r, gc = r0 + c;
      float x = 0.f;
      if (gr < M.n && gc < M.n)
        x = (c <= r) ? M.L[static_cast<size_t>(gr) * M.n + gc] : 0.f;
      else if (r == c)
        x = 1.f;  // identity padding keeps the block factorisable
      a[u][v] = x;
      t[u][v] = (r == c) ? 1.f : 0.f;
    }
  bool bad = false;
#pragma unroll
  for (int vo = 0; vo < 8; ++vo) {
    for (int txo = 0; txo < 16; ++txo) {
      const int j = vo * 16 + txo;
      float* col = colbuf[j & 1];   // column j of the block, before scaling
      float* row = rowbuf[j & 1];   // row j of the right-hand side, before scaling
      if (tx == txo) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (u >= vo) col[ty + 16 * u] = a[u][vo];
      }
      if (ty == txo) {
#pragma unroll
        for (int v = 0; v < 8; ++v)
          if (v <= vo) row[tx + 16 * v] = t[vo][v];
      }
      __syncthreads();
      float d = col[j];
      if (!(d > 0.f)) {
        bad = true;
        d = 1.f;
      }
      float inv = rsqrtf(d);
      inv = inv * fmaf(-0.5f * d, inv * inv, 1.5f);   // one Newton step: full fp32 accuracy
      const float sq = d * inv;
      float rv[8], cv[8], tv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) rv[u] = (u >= vo && ty + 16 * u > j) ? col[ty + 16 * u] * inv : 0.f;
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const int c = tx + 16 * v;
        cv[v] = (v >= vo && c > j) ? col[c] * inv : 0.f;
        tv[v] = (v <= vo && c <= j) ? row[c] * inv : 0.f;
      }
      if (tx == txo) {   // column j of the factor
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (u >= vo) {
            const int i = ty + 16 * u;
            if (i > j)
              a[u][vo] = rv[u];
            else if (i == j)
              a[u][vo] = sq;
          }
      }
      if (ty == txo) {   // row j of the inverse
#pragma unroll
        for (int v = 0; v < 8; ++v)
          if (v <= vo) t[vo][v] = tv[v];
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          if (u >= vo && v >= vo && v <= u) a[u][v] = fmaf(-rv[u], cv[v], a[u][v]);
          if (u >= vo && v <= vo) t[u][v] = fmaf(-rv[u], tv[v], t[u][v]);
        }
    }
  }
  if (bad && tid == 0) set_error(status, ERR_NOT_SPD);
#pragma unroll
  for (int u = 0; u < 8; ++u)
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      const int r = ty + 16 * u, c = tx + 16 * v;
      const int gr = r0 + r, gc = r0 + c;
      if (gr < M.n && gc < M.n) {
        if (c <= r) M.L[static_cast<size_t>(gr) * M.n + gc] = a[u][v];
        split3_store(M.Xs, static_cast<size_t>(gr) * M.ldp + gc, c <= r ? t[u][v] : 0.f);
      }
    }
}

struct Launch {
  int kind;   // 0: diagonal blocks of step `arg`, 1: GEMM work list
  int arg;    // step k (kind 0) / offset into the work list (kind 1)
  int count;  // CTAs (kind 0) / work items (kind 1)
};

struct Prepared {
  std::vector<const void*> key;
  at::Tensor splits;     // bf16 storage of all split buffers
  at::Tensor d_mats;     // TcMat table (sorted by decreasing size)
  at::Tensor d_probs;    // GemmProblem2 table
  at::Tensor d_work;     // all work lists, back to back
  std::vector<Launch> launches;
  int count = 0;
  int prepare_blocks = 1;   // row groups of the prepare kernel: the largest matrix has 8 rows per block
};

std::mutex g_cache_mutex;
std::list<Prepared> g_cache;
constexpr size_t kCacheEntries = 4;

int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// problem indices inside a matrix's group of five
enum { PB_PANEL = 0, PB_TRAIL = 1, PB_W = 2, PB_X21 = 3, PB_LAUUM = 4, PB_COUNT = 5 };

void fill_problem(GemmProblem2& P, __nv_bfloat16* const* a_parts, bool a_k, __nv_bfloat16* const* b_parts, bool b_k,
                  int n, int ldp, float* C, int ldc, float alpha, float beta, int flags,
                  __nv_bfloat16* const* out_parts, int* status) {
  std::memset(&P, 0, sizeof(P));
  for (int s = 0; s < 3; ++s) {  // (hi, mid, lo) parts; the kernel forms the six part products itself
    g2_encode_operand(&P.tmA[s], a_parts[s], n, n, ldp, a_k, G2_BM);
    g2_encode_operand(&P.tmB[s], b_parts[s], n, n, ldp, b_k, 128);
  }
  P.nseg = 3;
  P.M = P.N = P.K = n;
  P.C = C;
  P.Cin = C;
  P.ldc = ldc;
  P.alpha = alpha;
  P.beta = beta;
  P.flags = flags | G2F_SPLIT3 | (a_k ? G2F_A_KMAJOR : 0) | (b_k ? G2F_B_KMAJOR : 0);
  P.nsplit = 1;
  P.tiles_m = P.tiles_n = (n + TB - 1) / TB;
  P.ntiles = 0;
  P.status = status;
  if (out_parts != nullptr) {
    P.out_hi = out_parts[0];
    P.out_mid = out_parts[1];
    P.out_lo = out_parts[2];
    P.ld_out = ldp;
  }
}

GemmWork2 item(int problem, int a_mn, int b_mn, int a_k0, int b_k0, int nkb, int c_row, int c_col, int wflags) {
  GemmWork2 w;
  std::memset(&w, 0, sizeof(w));
  w.problem = problem;
  w.a_mn = a_mn;
  w.b_mn = b_mn;
  w.a_k0 = a_k0;
  w.b_k0 = b_k0;
  w.nkb = nkb;
  w.c_row = c_row;
  w.c_col = c_col;
  w.wflags = wflags;
  return w;
}

}  // namespace

void chol_inverse_tc(std::vector<at::Tensor> mats, std::vector<at::Tensor> outs, at::Tensor damping) {
  const int count = static_cast<int>(mats.size());
  TORCH_CHECK(count > 0 && outs.size() == mats.size(), "mats and outs must have the same length");
  TORCH_CHECK(damping.is_cuda() && damping.scalar_type() == at::kFloat && damping.is_contiguous() &&
                  damping.numel() == count, "damping must be a CUDA fp32 vector with one entry per matrix");
  const int dev = mats[0].get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  std::vector<const void*> key;
  key.reserve(4 * count + 1);
  key.push_back(reinterpret_cast<const void*>(static_cast<intptr_t>(dev)));
  for (int i = 0; i < count; ++i) {
    const at::Tensor& a = mats[i];
    const at::Tensor& o = outs[i];
    TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kFloat && a.dim() == 2 && a.size(0) == a.size(1) &&
                    a.stride(1) == 1 && a.size(0) > 0, "matrices must be square fp32 CUDA tensors with unit column stride");
    TORCH_CHECK(o.is_cuda() && o.scalar_type() == at::kFloat && o.is_contiguous() && o.sizes() == a.sizes(),
                "outputs must be contiguous fp32 tensors of the same shape");
    TORCH_CHECK(o.data_ptr() != a.data_ptr(), "the inverse cannot be written over its input");
    TORCH_CHECK(a.size(0) < (1 << 24), "matrix too large");
    key.push_back(a.data_ptr());
    key.push_back(o.data_ptr());
    key.push_back(reinterpret_cast<const void*>(static_cast<intptr_t>(a.size(0))));
    key.push_back(reinterpret_cast<const void*>(static_cast<intptr_t>(a.stride(0))));
  }

  std::lock_guard<std::mutex> lock(g_cache_mutex);
  Prepared* prep = nullptr;
  for (auto& p : g_cache)
    if (p.key == key) prep = &p;
  if (prep == nullptr) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    B200_CUDA_CHECK(cudaStreamIsCapturing(stream, &cap));
    TORCH_CHECK(cap == cudaStreamCaptureStatusNone, "the first grouped inverse of a set of matrices builds its "
                "tables and cannot run inside a CUDA graph capture; call it once before capturing");
    Prepared P;
    P.key = key;
    P.count = count;
    std::vector<int> order(count);
    for (int i = 0; i < count; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return mats[a].size(0) > mats[b].size(0); });
    // split storage: per matrix Ls, Xs, Ws with three parts each
    int64_t total = 0;
    std::vector<int64_t> base(count);
    for (int s = 0; s < count; ++s) {
      const int64_t n = mats[order[s]].size(0), ldp = round_up(n, 64);
      base[s] = total;
      total += 9 * round_up(n * ldp, 64);
    }
    P.splits = at::zeros({total}, at::TensorOptions().dtype(at::kBFloat16).device(at::kCUDA, dev));
    __nv_bfloat16* sp = reinterpret_cast<__nv_bfloat16*>(P.splits.data_ptr());
    int* status = device_state(dev).status.data_ptr<int>();

    std::vector<TcMat> host(count);
    std::vector<GemmProblem2> probs(static_cast<size_t>(count) * PB_COUNT);
    int nb_max = 0;
    for (int s = 0; s < count; ++s) {
      const int i = order[s];
      TcMat& M = host[s];
      std::memset(&M, 0, sizeof(M));
      M.A = mats[i].data_ptr<float>();
      M.lda = static_cast<int>(mats[i].stride(0));
      M.L = outs[i].data_ptr<float>();
      M.n = static_cast<int>(mats[i].size(0));
      M.nb = (M.n + TB - 1) / TB;
      M.ldp = static_cast<int>(round_up(M.n, 64));
      M.orig = i;
      const int64_t part = round_up(static_cast<int64_t>(M.n) * M.ldp, 64);
      __nv_bfloat16* Ws[3];
      for (int p = 0; p < 3; ++p) {
        M.Ls[p] = sp + base[s] + (0 + p) * part;
        M.Xs[p] = sp + base[s] + (3 + p) * part;
        Ws[p] = sp + base[s] + (6 + p) * part;
      }
      nb_max = std::max(nb_max, M.nb);
      P.prepare_blocks = std::max(P.prepare_blocks, std::min((M.n + 7) / 8, 1024));
      GemmProblem2* pb = &probs[static_cast<size_t>(s) * PB_COUNT];
      // L_ik = A_ik T_k^T : both operands K-major, result to L (fp32) and Ls (splits), in place
      fill_problem(pb[PB_PANEL], M.Ls, true, M.Xs, true, M.n, M.ldp, M.L, M.n, 1.f, 0.f, 0, M.Ls, status);
      // A_ij -= L_ik L_jk^T : lower tiles of the fp32 matrix; splits written for the next panel column only
      fill_problem(pb[PB_TRAIL], M.Ls, true, M.Ls, true, M.n, M.ldp, M.L, M.n, -1.f, 1.f,
                   G2F_SYM | G2F_LOWER, M.Ls, status);
      // W = L_21 X_11 and X_21 = -X_22 W : bf16 splits only
      fill_problem(pb[PB_W], M.Ls, true, M.Xs, false, M.n, M.ldp, nullptr, M.n, 1.f, 0.f, 0, Ws, status);
      fill_problem(pb[PB_X21], M.Xs, true, Ws, false, M.n, M.ldp, nullptr, M.n, -1.f, 0.f, 0, M.Xs, status);
      // out = X^T X : both operands MN-major, lower tiles mirrored
      fill_problem(pb[PB_LAUUM], M.Xs, false, M.Xs, false, M.n, M.ldp, M.L, M.n, 1.f, 0.f,
                   G2F_SYM, nullptr, status);
    }
    std::vector<GemmWork2> work;
    auto push_list = [&](const std::vector<GemmWork2>& items) {
      if (items.empty()) return;
      P.launches.push_back({1, static_cast<int>(work.size()), static_cast<int>(items.size())});
      work.insert(work.end(), items.begin(), items.end());
    };
    auto active = [&](int k) {  // matrices (a prefix of the sorted order) with more than k panels
      int c = 0;
      while (c < count && host[c].nb > k) ++c;
      return c;
    };
    // ---- potrf
    for (int k = 0; k < nb_max; ++k) {
      P.launches.push_back({0, k, active(k)});
      std::vector<GemmWork2> panel, trail;
      for (int s = 0; s < count && host[s].nb > k + 1; ++s) {
        const int nb = host[s].nb, pbase = s * PB_COUNT;
        for (int i = k + 1; i < nb; ++i)
          panel.push_back(item(pbase + PB_PANEL, i * TB, k * TB, k * TB, k * TB, 2, i * TB, k * TB, 0));
        // tiles of the next panel column first: the next diagonal block and panel depend on them
        for (int j = k + 1; j < nb; ++j)
          for (int i = j; i < nb; ++i)
            trail.push_back(item(pbase + PB_TRAIL, i * TB, j * TB, k * TB, k * TB, 2, i * TB, j * TB,
                                 (j == k + 1 && i > j) ? 0 : G2W_NO_SPLIT_OUT));
      }
      push_list(panel);
      push_list(trail);
    }
    // ---- trtri by recursive doubling
    for (int s_blk = 1; s_blk < nb_max; s_blk *= 2) {
      std::vector<GemmWork2> wl, xl;
      for (int s = 0; s < count && host[s].nb > s_blk; ++s) {
        const int nb = host[s].nb, pbase = s * PB_COUNT;
        for (int f0 = 0; f0 + s_blk < nb; f0 += 2 * s_blk) {
          const int e = f0 + s_blk;                       // first = [f0, e), second = [e, s1)
          const int s1 = std::min(e + s_blk, nb);
          for (int r = e; r < s1; ++r)
            for (int c = f0; c < e; ++c) {
              wl.push_back(item(pbase + PB_W, r * TB, c * TB, c * TB, c * TB, 2 * (e - c), r * TB, c * TB, 0));
              xl.push_back(item(pbase + PB_X21, r * TB, c * TB, e * TB, e * TB, 2 * (r - e + 1), r * TB, c * TB, 0));
            }
        }
      }
      auto by_cost = [](const GemmWork2& a, const GemmWork2& b) { return a.nkb > b.nkb; };
      std::stable_sort(wl.begin(), wl.end(), by_cost);
      std::stable_sort(xl.begin(), xl.end(), by_cost);
      push_list(wl);
      push_list(xl);
    }
    // ---- lauum
    {
      std::vector<GemmWork2> ll;
      for (int s = 0; s < count; ++s) {
        const int nb = host[s].nb, pbase = s * PB_COUNT;
        for (int i = 0; i < nb; ++i)
          for (int j = 0; j <= i; ++j)
            ll.push_back(item(pbase + PB_LAUUM, i * TB, j * TB, i * TB, i * TB, 2 * (nb - i), i * TB, j * TB, 0));
      }
      std::stable_sort(ll.begin(), ll.end(), [](const GemmWork2& a, const GemmWork2& b) { return a.nkb > b.nkb; });
      push_list(ll);
    }
    auto upload = [&](const void* src, size_t bytes) {
      at::Tensor hostt = at::empty({static_cast<int64_t>(bytes)}, at::TensorOptions().dtype(at::kByte).pinned_memory(true));
      std::memcpy(hostt.data_ptr(), src, bytes);
      at::Tensor d = hostt.to(at::Device(at::kCUDA, dev));
      return d;
    };
    P.d_mats = upload(host.data(), host.size() * sizeof(TcMat));
    P.d_probs = upload(probs.data(), probs.size() * sizeof(GemmProblem2));
    if (work.empty()) work.push_back(item(0, 0, 0, 0, 0, 0, 0, 0, 0));
    P.d_work = upload(work.data(), work.size() * sizeof(GemmWork2));
    TORCH_CHECK((reinterpret_cast<uintptr_t>(P.d_probs.data_ptr()) & 63) == 0, "problem table is not 64-byte aligned");
    B200_CUDA_CHECK(cudaStreamSynchronize(stream));  // the pinned staging buffers are released after this
    if (g_cache.size() >= kCacheEntries) g_cache.pop_front();
    g_cache.push_back(std::move(P));
    prep = &g_cache.back();
  }

  const TcMat* dm = reinterpret_cast<const TcMat*>(prep->d_mats.data_ptr());
  const GemmProblem2* dp = reinterpret_cast<const GemmProblem2*>(prep->d_probs.data_ptr());
  const GemmWork2* dw = reinterpret_cast<const GemmWork2*>(prep->d_work.data_ptr());
  int* status = device_state(dev).status.data_ptr<int>();
  tc_prepare_kernel<<<dim3(prep->prepare_blocks, count), 256, 0, stream>>>(dm, damping.data_ptr<float>());
  count_launch();
  for (const Launch& l : prep->launches) {
    if (l.kind == 0) {
      tc_diag_kernel<<<l.count, 256, 0, stream>>>(dm, l.arg, status);
      count_launch();
    } else {
      g2_launch_list(dp, dw + l.arg, l.count, G2_SPLIT3, dev, stream);
    }
  }
  B200_CUDA_CHECK(cudaGetLastError());
}

// Drops the cached tables and split buffers of the tensor-core inverse.
void chol_inverse_tc_clear_cache() {
  std::lock_guard<std::mutex> lock(g_cache_mutex);
  g_cache.clear();
}

}  // namespace b200
