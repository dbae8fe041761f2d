// CTA-pair flavour of the persistent tcgen05 GEMM / SYRK (umma_gemm2.cuh): `tcgen05.mma.cta_group::2`.
//
// Two CTAs of a cluster - on the two SMs of one TPC - share every tile.  A pair tile is 256 x 256:
// CTA r of the pair stages rows [128 r, 128 r + 128) of the A tile and columns [128 r, 128 r + 128) of
// the B tile in its own shared memory (32 KiB per 64-wide K block, a six-stage ring), the leader CTA
// (rank 0) issues one 256 x 256 x 16 MMA per K step that reads both CTAs' shared memory, and every
// CTA ends up with its 128 rows of the 256-column accumulator in its own TMEM.  Per FLOP a pair
// moves two thirds of the shared-memory bytes of a 128 x 256 tile and half those of a 128 x 128 tile.
//
// Signals inside a pair:
//   full[s]      lives in the leader.  The leader's producer arms it with the bytes of BOTH CTAs'
//                loads; each CTA's TMA loads (no cluster multicast: every CTA fetches its own
//                tiles) complete on it.
//   empty[s]     one per CTA; `tcgen05.commit` with a CTA mask arrives on both when the MMAs that
//                read the stage have finished.
//   acc_full[b]  one per CTA, signalled the same way when a tile's last MMA has finished.
//   acc_empty[b] lives in the leader and counts the epilogue warps of both CTAs (the peer's arrive
//                through the cluster's shared-memory window).
// Every wait is bounded in wall time as in the other flavours; the cluster barriers at the start
// and the end are reached by every thread on every path, error paths included.
//
// A problem of this flavour uses the tensor maps of the 128-wide flavour (boxes of 128 rows) and
// the tile grid and split-K scratch layout of the 256-wide flavour: the two halves of a pair tile
// are exactly the 128 x 256 tiles (2 TM + r, TN) of that grid, so the split-K reduction kernel of
// the wide flavour finishes a pair launch unchanged.
#pragma once
#include "umma_gemm2.cuh"

namespace b200 {

constexpr int G2P_STAGES = 6;
constexpr int G2P_STAGE_BYTES = 2 * G2_A_BYTES;             // this CTA's A rows and B columns of one K block
constexpr int G2P_EPI_WARPS = 8;
constexpr int G2P_THREADS = 64 + 32 * G2P_EPI_WARPS;
constexpr int G2P_TMEM_COLS = 512;                          // two 256-column accumulators
constexpr int G2P_SMEM_BYTES = G2P_STAGES * G2P_STAGE_BYTES + 1024 + 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the same shared-memory object in CTA `rank` of the cluster (shared::cluster window)
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled load into this CTA's shared memory whose completion is counted on a barrier that may
// live in the other CTA of the pair (`bar_cluster_addr` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// `bar` (same offset in both CTAs of the pair) observes completion of all MMAs issued so far.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

struct G2PairItem {
  int TM, TN;        // pair tile (256 x 256 units)
  int kb0, nkb;      // K blocks of this split
  int split;
};

__device__ __forceinline__ G2PairItem g2_pair_decode(const GemmProblem2& P, int idx) {
  G2PairItem it;
  const int t = idx / P.nsplit;
  it.split = idx - t * P.nsplit;
  if (P.flags & G2F_SYM) {
    int TM = 0, rem = t;
    while (rem > TM) {   // row TM of the pair grid holds TM + 1 tiles
      rem -= TM + 1;
      ++TM;
    }
    it.TM = TM;
    it.TN = rem;
  } else {
    it.TM = t / P.tiles_n;
    it.TN = t - it.TM * P.tiles_n;
  }
  const int kb_total = (P.K + G2_BK - 1) / G2_BK;
  it.kb0 = static_cast<int>((static_cast<long long>(it.split) * kb_total) / P.nsplit);
  const int kb1 = static_cast<int>((static_cast<long long>(it.split + 1) * kb_total) / P.nsplit);
  it.nkb = kb1 - it.kb0;
  return it;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2P_THREADS, 1)
umma_gemm2_pair_kernel(const __grid_constant__ GemmProblem2 P0, int n_work) {
  constexpr int STAGES = G2P_STAGES;
  constexpr int BN = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * G2P_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const GemmProblem2& P = P0;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * G2P_EPI_WARPS);  // the epilogue warps of both CTAs
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, G2P_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();   // barriers of both CTAs are initialised before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) --------------------------
    if (lane == 0) {
      const bool a_k = (P.flags & G2F_A_KMAJOR) != 0;
      const bool b_k = (P.flags & G2F_B_KMAJOR) != 0;
      uint32_t it = 0;
      bool ok = true;
      for (int wi = pair_id; wi < n_work && ok; wi += n_pairs) {
        const G2PairItem w = g2_pair_decode(P, wi);
        const int a_mn = w.TM * 256 + static_cast<int>(rank) * G2_BM;
        const int b_mn = w.TN * 256 + static_cast<int>(rank) * G2_BM;
        for (int seg = 0; seg < P.nseg && ok; ++seg) {
          for (int kb = 0; kb < w.nkb; ++kb, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
              set_error(P.status, ERR_WAIT_EMPTY);
              ok = false;
              break;
            }
            uint8_t* sA = smem + s * G2P_STAGE_BYTES;
            uint8_t* sB = sA + G2_A_BYTES;
            if (leader) mbar_expect_tx(&full_bar[s], 2 * G2P_STAGE_BYTES);
            const uint32_t bar = mapa_shared(smem_u32(&full_bar[s]), 0);
            const int k = (w.kb0 + kb) * G2_BK;
            if (a_k) {
              tma_load_2d_pair(sA, &P.tmA[seg], bar, k, a_mn);
            } else {
              tma_load_2d_pair(sA, &P.tmA[seg], bar, a_mn, k);
              tma_load_2d_pair(sA + G2_BK * 128, &P.tmA[seg], bar, a_mn + 64, k);
            }
            if (b_k) {
              tma_load_2d_pair(sB, &P.tmB[seg], bar, k, b_mn);
            } else {
              tma_load_2d_pair(sB, &P.tmB[seg], bar, b_mn, k);
              tma_load_2d_pair(sB + G2_BK * 128, &P.tmB[seg], bar, b_mn + 64, k);
            }
          }
        }
      }
      if (!ok && leader) {
        // give copies that are still in flight a bounded chance to land before teardown
        const uint32_t pending = it < static_cast<uint32_t>(STAGES) ? it : static_cast<uint32_t>(STAGES);
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t jt = it - 1 - j;
          mbar_wait(&full_bar[jt % STAGES], (jt / STAGES) & 1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ----------------------
    if (leader && lane == 0) {
      const bool a_k = (P.flags & G2F_A_KMAJOR) != 0;
      const bool b_k = (P.flags & G2F_B_KMAJOR) != 0;
      const uint32_t idesc = make_idesc_bf16(256, BN, !a_k, !b_k);
      uint32_t it = 0, ch = 0;
      bool ok = true;
      for (int wi = pair_id; wi < n_work && ok; wi += n_pairs) {
        const G2PairItem w = g2_pair_decode(P, wi);
        if (w.nkb <= 0) continue;
        const uint32_t ab = ch & 1;
        if (!mbar_wait(&acc_empty[ab], ((ch >> 1) & 1) ^ 1)) {
          set_error(P.status, ERR_WAIT_ACC);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tacc = tmem_base + ab * BN;
        uint32_t first = 1;
        for (int seg = 0; seg < P.nseg && ok; ++seg) {
          for (int kb = 0; kb < w.nkb; ++kb, ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
              set_error(P.status, ERR_WAIT_FULL);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t aA = smem_u32(smem + s * G2P_STAGE_BYTES);
            const uint32_t aB = aA + G2_A_BYTES;
#pragma unroll
            for (int k = 0; k < G2_BK / 16; ++k) {
              const uint64_t da = a_k ? make_smem_desc_sw128(aA + k * 32, 16, 1024)
                                      : make_smem_desc_sw128(aA + k * 16 * 128, G2_BK * 128, 1024);
              const uint64_t db = b_k ? make_smem_desc_sw128(aB + k * 32, 16, 1024)
                                      : make_smem_desc_sw128(aB + k * 16 * 128, G2_BK * 128, 1024);
              umma_bf16_pair(tacc, da, db, idesc, first ? 0u : 1u);
              first = 0;
            }
            umma_commit_pair(&empty_bar[s]);
          }
        }
        if (ok) umma_commit_pair(&acc_full[ab]);
        ++ch;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int q = warp & 3;                                   // TMEM lane quarter this warp may access
    constexpr int COLS = BN / (G2P_EPI_WARPS / 4);            // 128 columns per warp
    const int col_base = ((warp - 2) >> 2) * COLS;
    constexpr int PASSES = COLS / 64;
    const int row = q * 32 + lane;
    const G2Epi E = g2_epi(P);
    const bool sym = (E.flags & G2F_SYM) != 0;
    const bool atomic = (E.flags & G2F_ATOMIC) != 0;
    const bool to_ws = E.nsplit > 1 && !atomic;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    uint32_t ch = 0;
    bool ok = true;
    for (int wi = pair_id; wi < n_work && ok; wi += n_pairs) {
      const G2PairItem w = g2_pair_decode(P, wi);
      const int c_row = w.TM * 256 + static_cast<int>(rank) * G2_BM;
      const int c_col = w.TN * 256;
      const int tm = 2 * w.TM + static_cast<int>(rank);
      const int tile_id = sym ? w.TM * (w.TM + 1) + static_cast<int>(rank) * (w.TM + 1) + w.TN : tm * E.full->tiles_n + w.TN;
      const int gr = c_row + row;
      const bool have = w.nkb > 0;
      const uint32_t ab = ch & 1;
      if (have) {
        ok = mbar_wait(&acc_full[ab], (ch >> 1) & 1);
        if (!ok) set_error(P.status, ERR_WAIT_ACC);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
      }
#pragma unroll
      for (int pass = 0; pass < PASSES; ++pass) {
        float v[64];
        const int col0 = col_base + pass * 64;
        if (have) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(tmem_base + lane_addr + ab * BN + col0, r0);
          tmem_ld_32x32(tmem_base + lane_addr + ab * BN + col0 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __uint_as_float(r0[j]);
            v[32 + j] = __uint_as_float(r1[j]);
          }
          if (pass == PASSES - 1) {  // this warp's share is in registers: hand the accumulator back to the leader
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[ab]), 0));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 64; ++j) v[j] = 0.f;
        }
        if (c_row >= E.M) continue;   // the lower half of the last pair row of an odd tile count: nothing to write
        if (to_ws) {
          float* part = E.ws + (static_cast<size_t>(tile_id) * E.nsplit + w.split) * (G2_BM * BN) +
                        static_cast<size_t>(row) * BN + col0;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            *reinterpret_cast<float4*>(part + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          continue;
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int gc0 = c_col + col0 + c * 32;
          // a symmetric problem's pair tile on the diagonal reaches past the diagonal block: skip that part
          const bool beyond = sym && (gc0 / G2_BM) > (c_row / G2_BM);
          const bool diag = sym && (gc0 / G2_BM) == (c_row / G2_BM);
          if (gc0 < E.N && !beyond && !(diag && gc0 > gr)) {
            if (atomic)
              g2_reduce_chunk(E, v + c * 32, gr, gc0, diag);
            else
              g2_store_chunk(E, v + c * 32, gr, gc0, diag, true);
          }
        }
      }
      if (have) ++ch;
    }
  }

  tc_fence_before_sync();
  cluster_sync_all();   // nobody frees TMEM or leaves while the other CTA may still signal it
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, G2P_TMEM_COLS);
  }
}

}  // namespace b200
