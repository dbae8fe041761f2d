// tcgen05 "TN" GEMM / SYRK for sm_100a.
//
//   C[M x N] (fp32)  =  alpha * sum_seg  op(A_seg)^T-contract-K  op(B_seg)   (+ beta * Cin)
//
// Both operands are bf16 and are contracted over K.  Each operand may be stored either
//   * MN-major: a [K, M] row-major matrix (the layout of activations / output-gradients,
//     rows = samples, so that C = X^T Y needs no transpose copy), or
//   * K-major : a [M, K] row-major matrix.
// Up to three (A_seg, B_seg) pairs are accumulated into the same TMEM accumulator.  With
// A = (hi, hi, lo) and B = (hi, lo, hi) this evaluates an fp32-grade product out of bf16
// tensor-core instructions ("bf16x3").
//
// One CTA computes one 128x128 output tile for one K-split:
//   warp 0      : TMA producer (cp.async.bulk.tensor, 128B swizzle, 3-stage ring)
//   warp 1      : TMEM allocator + single-thread tcgen05.mma issuer
//   warps 2..5  : epilogue (tcgen05.ld -> registers -> global), split-K fix-up, EMA (beta),
//                 symmetric mirror store, optional bf16 hi/lo outputs.
// Split-K partial tiles go to a scratch buffer; `splitk_reduce_kernel` then sums the partials
// in split order (deterministic) and runs the same epilogue with fully coalesced traffic.
// SYM mode (SYRK) schedules only tiles on or below the diagonal and mirrors them.
//
// Epilogue variants for destinations in other GPUs' memory (peer pointers from a symmetric
// allocation): plain stores of the lower-triangular tiles only (GF_LOWER: the owner of the matrix
// sums and mirrors what the ranks sent), `red.global.add` reductions (GF_ATOMIC, optionally
// lower-only), and up to G_MAX_EXTRA additional plain copies of the result (C_extra: the
// preconditioned gradient replicated to every rank).  Peer memory is only ever written with
// per-thread stores / reductions from the epilogue; TMA loads always read local memory.
// A grouped launch (`work` != nullptr) runs one tile of one problem of a plan per CTA.
#pragma once
#include "sm100_ptx.cuh"

namespace b200 {

constexpr int G_BM = 128;
constexpr int G_BN = 128;
constexpr int G_BK = 64;
constexpr int G_STAGES = 3;
constexpr int G_THREADS = 192;
constexpr int G_TMEM_COLS = 128;
constexpr int G_OPERAND_BYTES = G_BM * G_BK * 2;  // 16 KiB per operand per stage
constexpr int G_STAGE_BYTES = 2 * G_OPERAND_BYTES;
constexpr int G_SMEM_BYTES = G_STAGES * G_STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

enum : int {
  GF_SYM = 1,        // symmetric output: lower tiles only, mirrored
  GF_A_KMAJOR = 2,   // A given as [M, K] row-major
  GF_B_KMAJOR = 4,   // B given as [N, K] row-major
  GF_SAME_AB = 8,    // A and B are the same matrix (diagonal tiles load once)
  GF_ATOMIC = 16,    // C += alpha * result with reductions (C may live on another GPU); beta unused
  GF_LOWER = 32,     // with GF_SYM: write / add the lower triangle only (the owner of the matrix mirrors it)
};

constexpr int G_MAX_EXTRA = 7;  // additional destinations of the result (peer copies)

struct alignas(64) GemmProblem {
  CUtensorMap tmA[3];
  CUtensorMap tmB[3];
  float* C;              // may be null when only bf16 outputs are wanted
  const float* Cin;      // read when beta != 0 (may alias C)
  __nv_bfloat16* out_hi; // optional bf16 copy of the result
  __nv_bfloat16* out_lo; // optional bf16 residual (result - hi)
  float* ws;             // split-K scratch: [tiles][nsplit][128][128] fp32
  int* status;           // device error word
  float* C_extra[G_MAX_EXTRA];  // the fp32 result is also stored here (same ldc), e.g. peer GPUs
  int n_extra;
  int M, N, K;
  int ldc, ld_out;
  int nseg;
  int tiles_m, tiles_n, ntiles, nsplit;
  int flags;
  float alpha, beta;
};

struct GemmWork {  // grouped mode: one entry per CTA
  int problem, tm, tn, split;
};

__device__ __forceinline__ void gemm_decode_tile(const GemmProblem& P, int t, int& tm, int& tn) {
  if (P.flags & GF_SYM) {
    int r = static_cast<int>((sqrtf(8.f * static_cast<float>(t) + 1.f) - 1.f) * 0.5f);
    while ((r + 1) * (r + 2) / 2 <= t) ++r;
    while (r * (r + 1) / 2 > t) --r;
    tm = r;
    tn = t - r * (r + 1) / 2;
  } else {
    tm = t / P.tiles_n;
    tn = t - tm * P.tiles_n;
  }
}

__device__ __forceinline__ int gemm_tile_id(const GemmProblem& P, int tm, int tn) {
  return (P.flags & GF_SYM) ? tm * (tm + 1) / 2 + tn : tm * P.tiles_n + tn;
}

__device__ __forceinline__ void red_add_f32(float* p, float v) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

// Accumulating variant of the final store (GF_ATOMIC): every element is added to C with a
// reduction instruction, lower tile and mirror image alike, so that several CTAs / GPUs can
// contribute to the same matrix.
__device__ __forceinline__ void gemm_reduce_chunk(const GemmProblem& P, const float (&v)[32], int gr,
                                                  int gc0, bool diag_tile) {
  if (gr >= P.M) return;
  const bool sym = (P.flags & GF_SYM) != 0;
  const float alpha = P.alpha;
  float* c = P.C + static_cast<size_t>(gr) * P.ldc + gc0;
  const bool vec_ok = (gc0 + 32 <= P.N) && ((P.ldc & 3) == 0) && !(sym && diag_tile);
  if (vec_ok) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      red_add_v4_f32(c + 4 * j, alpha * v[4 * j], alpha * v[4 * j + 1], alpha * v[4 * j + 2],
                     alpha * v[4 * j + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int gc = gc0 + j;
      if (gc < P.N && !(sym && diag_tile && gc > gr)) red_add_f32(c + j, alpha * v[j]);
    }
  }
  if (sym && !(P.flags & GF_LOWER)) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int gc = gc0 + j;
      if (gc < P.N && (!diag_tile || gc < gr))
        red_add_f32(P.C + static_cast<size_t>(gc) * P.ldc + gr, alpha * v[j]);
    }
  }
}

// Final store of one 32-column chunk held by this thread (row `gr`, columns gc0..gc0+31).
__device__ __forceinline__ void gemm_store_chunk(const GemmProblem& P, const float (&v)[32], int gr,
                                                 int gc0, bool diag_tile) {
  if (gr >= P.M) return;
  const bool sym = (P.flags & GF_SYM) != 0;
  const float alpha = P.alpha, beta = P.beta;
  float out[32];
  const bool full = (gc0 + 32 <= P.N);
  const bool vec_ok = full && ((P.ldc & 3) == 0);
  if (beta != 0.f) {
    const float* cin = P.Cin + static_cast<size_t>(gr) * P.ldc + gc0;
    if (vec_ok) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 c4 = *reinterpret_cast<const float4*>(cin + 4 * j);
        out[4 * j + 0] = alpha * v[4 * j + 0] + beta * c4.x;
        out[4 * j + 1] = alpha * v[4 * j + 1] + beta * c4.y;
        out[4 * j + 2] = alpha * v[4 * j + 2] + beta * c4.z;
        out[4 * j + 3] = alpha * v[4 * j + 3] + beta * c4.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        out[j] = (gc0 + j < P.N) ? alpha * v[j] + beta * cin[j] : 0.f;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) out[j] = alpha * v[j];
  }
  if (P.C != nullptr) {
    float* c = P.C + static_cast<size_t>(gr) * P.ldc + gc0;
    if (!sym) {
      if (vec_ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(c + 4 * j) =
              make_float4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gc0 + j < P.N) c[j] = out[j];
      }
    } else if (!diag_tile) {
      // strictly-lower tile: direct store plus mirrored (transposed) store
      if (vec_ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(c + 4 * j) =
              make_float4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gc0 + j < P.N) c[j] = out[j];
      }
      if (!(P.flags & GF_LOWER)) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gc0 + j < P.N) P.C[static_cast<size_t>(gc0 + j) * P.ldc + gr] = out[j];
      }
    } else {
      // diagonal tile: keep the lower triangle, mirror it so the result is exactly symmetric
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int gc = gc0 + j;
        if (gc <= gr && gc < P.N) {
          c[j] = out[j];
          if (gc < gr && !(P.flags & GF_LOWER)) P.C[static_cast<size_t>(gc) * P.ldc + gr] = out[j];
        }
      }
    }
  }
  for (int e = 0; e < P.n_extra; ++e) {  // plain (non-symmetric) result replicated to peers
    float* c = P.C_extra[e] + static_cast<size_t>(gr) * P.ldc + gc0;
    if (vec_ok) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(c + 4 * j) =
            make_float4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (gc0 + j < P.N) c[j] = out[j];
    }
  }
  if (P.out_hi != nullptr) {
    __nv_bfloat16* oh = P.out_hi + static_cast<size_t>(gr) * P.ld_out + gc0;
    __nv_bfloat16* ol =
        P.out_lo ? P.out_lo + static_cast<size_t>(gr) * P.ld_out + gc0 : nullptr;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (gc0 + j < P.N) {
        __nv_bfloat16 h = __float2bfloat16_rn(out[j]);
        oh[j] = h;
        if (ol) ol[j] = __float2bfloat16_rn(out[j] - __bfloat162float(h));
      }
    }
  }
}

__global__ void __launch_bounds__(G_THREADS, 2)
umma_gemm_kernel(const __grid_constant__ GemmProblem single, const GemmProblem* __restrict__ probs,
                 const GemmWork* __restrict__ work) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128B swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + G_STAGES * G_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + G_STAGES;
  uint64_t* acc_bar = empty_bar + G_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const GemmProblem* Pp;
  int tm, tn, split;
  if (work != nullptr) {
    const GemmWork w = work[blockIdx.x];
    Pp = probs + w.problem;
    tm = w.tm;
    tn = w.tn;
    split = w.split;
  } else {
    Pp = &single;
    gemm_decode_tile(single, blockIdx.x, tm, tn);
    split = blockIdx.y;
  }
  const GemmProblem& P = *Pp;

  const bool a_k = (P.flags & GF_A_KMAJOR) != 0;
  const bool b_k = (P.flags & GF_B_KMAJOR) != 0;
  const bool diag_tile = (P.flags & GF_SYM) && tm == tn;
  const bool shared_ab = diag_tile && (P.flags & GF_SAME_AB);
  const int kb_total = (P.K + G_BK - 1) / G_BK;
  const int kb0 = static_cast<int>((static_cast<long long>(split) * kb_total) / P.nsplit);
  const int kb1 = static_cast<int>((static_cast<long long>(split + 1) * kb_total) / P.nsplit);
  const int iters = P.nseg * (kb1 - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < G_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, G_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------
    if (lane == 0) {
      for (int s = 0; s < P.nseg; ++s) {
        tma_prefetch_desc(&P.tmA[s]);
        tma_prefetch_desc(&P.tmB[s]);
      }
      const uint32_t bytes = shared_ab ? G_OPERAND_BYTES : 2 * G_OPERAND_BYTES;
      int it = 0;
      bool ok = true;
      for (int seg = 0; seg < P.nseg && ok; ++seg) {
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % G_STAGES;
          const uint32_t ph = (it / G_STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            set_error(P.status, ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * G_STAGE_BYTES;
          uint8_t* sB = sA + G_OPERAND_BYTES;
          mbar_expect_tx(&full_bar[s], bytes);
          if (a_k) {
            tma_load_2d(sA, &P.tmA[seg], &full_bar[s], kb * G_BK, tm * G_BM);
          } else {
            tma_load_2d(sA, &P.tmA[seg], &full_bar[s], tm * G_BM, kb * G_BK);
            tma_load_2d(sA + G_BK * 128, &P.tmA[seg], &full_bar[s], tm * G_BM + 64, kb * G_BK);
          }
          if (!shared_ab) {
            if (b_k) {
              tma_load_2d(sB, &P.tmB[seg], &full_bar[s], kb * G_BK, tn * G_BN);
            } else {
              tma_load_2d(sB, &P.tmB[seg], &full_bar[s], tn * G_BN, kb * G_BK);
              tma_load_2d(sB + G_BK * 128, &P.tmB[seg], &full_bar[s], tn * G_BN + 64, kb * G_BK);
            }
          }
        }
      }
      if (!ok) {
        // give copies that are still in flight a bounded chance to land before teardown
        const int pending = it < G_STAGES ? it : G_STAGES;
        for (int j = 0; j < pending; ++j) {
          const int jt = it - 1 - j;
          mbar_wait(&full_bar[jt % G_STAGES], (jt / G_STAGES) & 1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(G_BM, G_BN, !a_k, !b_k);
      bool ok = true;
      for (int it = 0; it < iters; ++it) {
        const int s = it % G_STAGES;
        const uint32_t ph = (it / G_STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph)) {
          set_error(P.status, ERR_WAIT_FULL);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t aA = smem_u32(smem + s * G_STAGE_BYTES);
        const uint32_t aB = shared_ab ? aA : aA + G_OPERAND_BYTES;
#pragma unroll
        for (int k = 0; k < G_BK / 16; ++k) {
          // MN-major: 16 K-rows of 128 B each per MMA; K-major: 16 K-elements = 32 B per MMA.
          const uint64_t da = a_k ? make_smem_desc_sw128(aA + k * 32, 16, 1024)
                                  : make_smem_desc_sw128(aA + k * 16 * 128, G_BK * 128, 1024);
          const uint64_t db = b_k ? make_smem_desc_sw128(aB + k * 32, 16, 1024)
                                  : make_smem_desc_sw128(aB + k * 16 * 128, G_BK * 128, 1024);
          umma_bf16(tmem_base, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(acc_bar);
    }
  } else {
    // ------------------------------ epilogue ----------------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;
    const int gr = tm * G_BM + row;
    const int tile_id = gemm_tile_id(P, tm, tn);
    bool ok = true;
    if (iters > 0) {
      ok = mbar_wait(acc_bar, 0);
      if (!ok) set_error(P.status, ERR_WAIT_ACC);
    }
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after_sync();
    if (ok) {
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      const bool atomic = (P.flags & GF_ATOMIC) != 0;
      if (P.nsplit == 1 || atomic) {
#pragma unroll 1
        for (int c = 0; c < G_BN / 32; ++c) {
          float v[32];
          if (iters > 0) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
          const int gc0 = tn * G_BN + c * 32;
          if (gc0 < P.N && !(diag_tile && gc0 > gr)) {
            if (atomic)
              gemm_reduce_chunk(P, v, gr, gc0, diag_tile);
            else
              gemm_store_chunk(P, v, gr, gc0, diag_tile);
          }
        }
      } else {
        float* part = P.ws + (static_cast<size_t>(tile_id) * P.nsplit + split) * (G_BM * G_BN) +
                      static_cast<size_t>(row) * G_BN;
#pragma unroll 1
        for (int c = 0; c < G_BN / 32; ++c) {
          uint32_t r[32];
          if (iters > 0) {
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(part + c * 32 + 4 * j) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, G_TMEM_COLS);
  }
}


// Sums split-K partials and applies the epilogue.  One block handles a 32x32 patch of one tile:
// reads and direct stores are 128-byte coalesced, the mirrored store goes through shared memory.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const __grid_constant__ GemmProblem single, const GemmProblem* __restrict__ probs,
                     const GemmWork* __restrict__ work) {
  __shared__ float tile[32][33];
  const GemmProblem* Pp;
  int tm, tn;
  if (work != nullptr) {
    const GemmWork w = work[blockIdx.x];
    Pp = probs + w.problem;
    tm = w.tm;
    tn = w.tn;
  } else {
    Pp = &single;
    gemm_decode_tile(single, blockIdx.x, tm, tn);
  }
  const GemmProblem& P = *Pp;
  const int tile_id = gemm_tile_id(P, tm, tn);
  const bool sym = (P.flags & GF_SYM) != 0;
  const bool diag_tile = sym && tm == tn;
  const int sub_r = blockIdx.y >> 2, sub_c = blockIdx.y & 3;  // 4x4 patches of 32x32
  if (diag_tile && sub_c > sub_r) return;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  // patches that lie completely outside the matrix (edge tiles of small problems) have no work
  if (tm * G_BM + sub_r * 32 >= P.M || tn * G_BN + sub_c * 32 >= P.N) return;
  const float* base = P.ws + static_cast<size_t>(tile_id) * P.nsplit * (G_BM * G_BN);
  const int gc = tn * G_BN + sub_c * 32 + tx;
  // sum the partials in split order; the loads of the four rows of a thread and of four splits are
  // issued together (16 independent loads in flight per thread)
  float accs[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const float* p0 = base + static_cast<size_t>(sub_r * 32 + ty) * G_BN + sub_c * 32 + tx;
    int s = 0;
    for (; s + 4 <= P.nsplit; s += 4) {
      float v[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u)
          v[i][u] = __ldcg(p0 + static_cast<size_t>(8 * i) * G_BN + static_cast<size_t>(s + u) * (G_BM * G_BN));
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u) accs[i] += v[i][u];
    }
    for (; s < P.nsplit; ++s)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        accs[i] += __ldcg(p0 + static_cast<size_t>(8 * i) * G_BN + static_cast<size_t>(s) * (G_BM * G_BN));
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = ty + 8 * i;
    const int row = sub_r * 32 + lr;
    const int gr = tm * G_BM + row;
    const float acc = accs[i];
    float val = P.alpha * acc;
    const bool inb = gr < P.M && gc < P.N;
    if (inb && P.beta != 0.f) val += P.beta * P.Cin[static_cast<size_t>(gr) * P.ldc + gc];
    tile[lr][tx] = val;
    const bool keep = inb && !(diag_tile && gc > gr);
    if (keep) {
      if (P.C != nullptr) P.C[static_cast<size_t>(gr) * P.ldc + gc] = val;
      for (int e = 0; e < P.n_extra; ++e) P.C_extra[e][static_cast<size_t>(gr) * P.ldc + gc] = val;
      if (P.out_hi != nullptr) {
        const __nv_bfloat16 h = __float2bfloat16_rn(val);
        P.out_hi[static_cast<size_t>(gr) * P.ld_out + gc] = h;
        if (P.out_lo != nullptr)
          P.out_lo[static_cast<size_t>(gr) * P.ld_out + gc] =
              __float2bfloat16_rn(val - __bfloat162float(h));
      }
    }
  }
  if (!sym || P.C == nullptr || (P.flags & GF_LOWER)) return;
  __syncthreads();
  // mirrored store: element (r, c) of the patch goes to C[c][r]
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lc = ty + 8 * i;                       // patch column -> destination row
    const int dst_r = tn * G_BN + sub_c * 32 + lc;   // global column index of the source
    const int dst_c = tm * G_BM + sub_r * 32 + tx;   // global row index of the source
    if (dst_r < P.N && dst_c < P.M && dst_r < dst_c)
      P.C[static_cast<size_t>(dst_r) * P.ldc + dst_c] = tile[tx][lc];
  }
}

}  // namespace b200
