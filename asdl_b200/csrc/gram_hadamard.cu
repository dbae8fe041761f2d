// Hadamard-factored Gram matrix of one layer on the tensor cores:
//     kernel[n1 x n2]  +=  alpha * (A1 A2^T + one) o (G1 G2^T)
// A1 / A2: layer inputs of the two example sets ([n, d_in], examples are rows), G1 / G2: output
// gradients ([n, d_out]); `one` is 1 when the layer has a bias (its per-example gradient adds
// g_i . g_j to the entry), `alpha` carries the 1 / spatial-size factor of a convolution.
// This is what asdl/operations/operation.py:335-351 (OP_GRAM_HADAMARD) computes with two matmuls,
// an add and a multiply; here one CTA per 128 x 128 tile forms both Gram tiles in its two TMEM
// accumulators (tcgen05.mma, operands staged by TMA) and the epilogue multiplies them out of TMEM,
// so neither Gram matrix exists in memory.
//
// Operands arrive as bf16 parts: one part per matrix, or (hi, lo) pairs for fp32 inputs, in which
// case every Gram tile is the sum of the three significant part products ("bf16x3").
#include "host_utils.h"
#include "sm100_ptx.cuh"

namespace b200 {

namespace {

constexpr int GH_BM = 128, GH_BN = 128, GH_BK = 64;
constexpr int GH_STAGES = 4;
constexpr int GH_TILE_BYTES = GH_BM * GH_BK * 2;          // 16 KiB
constexpr int GH_STAGE_BYTES = 2 * GH_TILE_BYTES;
constexpr int GH_THREADS = 64 + 32 * 4;
constexpr int GH_SMEM = GH_STAGES * GH_STAGE_BYTES + 1024 + 128;

struct alignas(64) HadamardProblem {
  CUtensorMap tmL[6];   // left operand of every part product (rows of the first example set)
  CUtensorMap tmR[6];   // right operand (rows of the second example set)
  float* C;
  int* status;
  int M, N, ldc;
  int K[2];             // d_in, d_out
  int nseg[2];          // part products of the input Gram / of the gradient Gram
  float alpha, one;
};

__global__ void __launch_bounds__(GH_THREADS, 1)
gram_hadamard_kernel(const __grid_constant__ HadamardProblem P) {
  extern __shared__ uint8_t gh_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gh_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + GH_STAGES * GH_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + GH_STAGES;
  uint64_t* acc_full = empty_bar + GH_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.y * GH_BM, col0 = blockIdx.x * GH_BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GH_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * GH_BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int kb_of[2] = {(P.K[0] + GH_BK - 1) / GH_BK, (P.K[1] + GH_BK - 1) / GH_BK};

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int seg = 0;
      for (int which = 0; which < 2 && ok; ++which) {
        for (int sg = 0; sg < P.nseg[which] && ok; ++sg, ++seg) {
          for (int kb = 0; kb < kb_of[which]; ++kb, ++it) {
            const int s = it % GH_STAGES;
            if (!mbar_wait(&empty_bar[s], ((it / GH_STAGES) & 1) ^ 1)) {
              set_error(P.status, ERR_WAIT_EMPTY);
              ok = false;
              break;
            }
            uint8_t* stage = smem + s * GH_STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], GH_STAGE_BYTES);
            tma_load_2d(stage, &P.tmL[seg], &full_bar[s], kb * GH_BK, row0);
            tma_load_2d(stage + GH_TILE_BYTES, &P.tmR[seg], &full_bar[s], kb * GH_BK, col0);
          }
        }
      }
      if (!ok) {
        const uint32_t pending = it < static_cast<uint32_t>(GH_STAGES) ? it : static_cast<uint32_t>(GH_STAGES);
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t jt = it - 1 - j;
          mbar_wait(&full_bar[jt % GH_STAGES], (jt / GH_STAGES) & 1);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(GH_BM, GH_BN, false, false);   // both operands K-major
      uint32_t it = 0;
      bool ok = true;
      for (int which = 0; which < 2 && ok; ++which) {
        const uint32_t tacc = tmem_base + which * GH_BN;
        uint32_t first = 1;
        for (int sg = 0; sg < P.nseg[which] && ok; ++sg) {
          for (int kb = 0; kb < kb_of[which]; ++kb, ++it) {
            const int s = it % GH_STAGES;
            if (!mbar_wait(&full_bar[s], (it / GH_STAGES) & 1)) {
              set_error(P.status, ERR_WAIT_FULL);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t aL = smem_u32(smem + s * GH_STAGE_BYTES);
            const uint32_t aR = aL + GH_TILE_BYTES;
#pragma unroll
            for (int k = 0; k < GH_BK / 16; ++k) {
              umma_bf16(tacc, make_smem_desc_sw128(aL + k * 32, 16, 1024), make_smem_desc_sw128(aR + k * 32, 16, 1024),
                        idesc, first ? 0u : 1u);
              first = 0;
            }
            umma_commit(&empty_bar[s]);
          }
        }
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int gr = row0 + row;
    bool ok = mbar_wait(acc_full, 0);
    if (!ok) set_error(P.status, ERR_WAIT_ACC);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after_sync();
      const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
      const bool have_a = P.nseg[0] > 0 && kb_of[0] > 0;
#pragma unroll 1
      for (int c = 0; c < GH_BN / 32; ++c) {
        uint32_t ra[32], rg[32];
        if (have_a) tmem_ld_32x32(tmem_base + lane_addr + c * 32, ra);
        tmem_ld_32x32(tmem_base + lane_addr + GH_BN + c * 32, rg);
        tmem_ld_wait();
        if (gr < P.M) {
          float* dst = P.C + static_cast<size_t>(gr) * P.ldc + col0 + c * 32;
          float upd[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float a = have_a ? __uint_as_float(ra[j]) : 0.f;
            upd[j] = P.alpha * (a + P.one) * __uint_as_float(rg[j]);
          }
          const bool vec = (col0 + c * 32 + 32 <= P.N) && ((P.ldc & 3) == 0) &&
                           ((reinterpret_cast<uintptr_t>(P.C) & 15) == 0);
          if (vec) {
            // all eight 16-byte loads of the row segment are in flight before the first store
            float4 cur[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) cur[j] = *reinterpret_cast<const float4*>(dst + 4 * j);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4*>(dst + 4 * j) = make_float4(cur[j].x + upd[4 * j], cur[j].y + upd[4 * j + 1],
                                                                    cur[j].z + upd[4 * j + 2], cur[j].w + upd[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + c * 32 + j < P.N) dst[j] += upd[j];
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 2 * GH_BN);
  }
}

void check_part(const at::Tensor& t, int64_t rows, int64_t cols, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1 &&
                  t.size(0) == rows && t.size(1) == cols,
              name, " parts must be bf16 CUDA matrices of one shape with unit column stride");
  TORCH_CHECK((t.stride(0) * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name,
              " parts need 16-byte aligned rows");
}

}  // namespace

// kernel += alpha * (A1 A2^T + one) o (G1 G2^T).  a1 / a2 / g1 / g2: one bf16 part each, or (hi, lo)
// pairs; a1 / a2 may be empty (the factor is then `one` alone).  kernel: fp32 [n1, n2].
void gram_hadamard(std::vector<at::Tensor> a1, std::vector<at::Tensor> a2, std::vector<at::Tensor> g1,
                   std::vector<at::Tensor> g2, at::Tensor kernel, double alpha, double one) {
  TORCH_CHECK(kernel.is_cuda() && kernel.scalar_type() == at::kFloat && kernel.dim() == 2 && kernel.stride(1) == 1,
              "kernel must be an fp32 CUDA matrix with unit column stride");
  TORCH_CHECK(a1.size() == a2.size() && g1.size() == g2.size() && !g1.empty() && g1.size() <= 2 && a1.size() <= 2,
              "operands are one bf16 part or a (hi, lo) pair per matrix");
  const int64_t n1 = kernel.size(0), n2 = kernel.size(1);
  if (n1 == 0 || n2 == 0) return;
  const int dev = kernel.get_device();
  c10::cuda::CUDAGuard guard(dev);
  HadamardProblem P;
  std::memset(&P, 0, sizeof(P));
  int seg = 0;
  auto add = [&](const std::vector<at::Tensor>& l, const std::vector<at::Tensor>& r, int which) {
    if (l.empty()) return;
    const int64_t k = l[0].size(1);
    for (auto& t : l) check_part(t, n1, k, "left");
    for (auto& t : r) check_part(t, n2, k, "right");
    P.K[which] = static_cast<int>(k);
    // part products, small magnitudes first: (lo, hi), (hi, lo), (hi, hi)
    const int pairs[3][2] = {{1, 0}, {0, 1}, {0, 0}};
    for (int p = (l.size() == 2 ? 0 : 2); p < 3; ++p, ++seg) {
      const at::Tensor& lt = l[pairs[p][0]];
      const at::Tensor& rt = r[pairs[p][1]];
      encode_tmap_bf16_2d(&P.tmL[seg], lt.data_ptr(), k, n1, lt.stride(0), 64, GH_BM);
      encode_tmap_bf16_2d(&P.tmR[seg], rt.data_ptr(), k, n2, rt.stride(0), 64, GH_BN);
      ++P.nseg[which];
    }
  };
  add(a1, a2, 0);
  add(g1, g2, 1);
  P.C = kernel.data_ptr<float>();
  P.status = device_state(dev).status.data_ptr<int>();
  P.M = static_cast<int>(n1);
  P.N = static_cast<int>(n2);
  P.ldc = static_cast<int>(kernel.stride(0));
  P.alpha = static_cast<float>(alpha);
  P.one = static_cast<float>(one);
  static bool attr_set_on[64] = {false};
  if (!attr_set_on[dev & 63]) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(gram_hadamard_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GH_SMEM));
    attr_set_on[dev & 63] = true;
  }
  const dim3 grid(static_cast<unsigned>((n2 + GH_BN - 1) / GH_BN), static_cast<unsigned>((n1 + GH_BM - 1) / GH_BM));
  gram_hadamard_kernel<<<grid, GH_THREADS, GH_SMEM, at::cuda::getCurrentCUDAStream(dev).stream()>>>(P);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

}  // namespace b200
