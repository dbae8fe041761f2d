// Persistent tcgen05 "TN" GEMM / SYRK for sm_100a (second generation of umma_gemm.cuh).
//
//   C[M x N] (fp32)  =  alpha * sum_seg  op(A_seg)^T-contract-K  op(B_seg)   (+ beta * Cin)
//
// Operands are bf16 matrices contracted over K, each either MN-major ([K, M] row-major, the layout
// of activations, so that X^T Y needs no transpose copy) or K-major ([M, K] row-major).
//
// Persistent CTAs walk a list of work items - tiles of one problem or of a whole plan of problems -
// so a grouped launch pays one prologue per CTA, not one per tile.  Every CTA owns two TMEM
// accumulators: the MMA warp fills one while the epilogue warps drain the other, so stores
// (including stores into other GPUs' memory) overlap the next tile's main loop.  A work item
// carries its own operand origins and K range, so triangular operands (Cholesky panels,
// triangular inverses) skip their zero blocks and sub-matrices of one tensor map serve as operands.
//
// Four flavours of one kernel template:
//   plain   128 x 128 tiles, two CTAs per SM with a 3-stage ring each (two independent pipelines
//           per SM hide each other's load latency), four epilogue warps; up to six (A_seg, B_seg)
//           pairs accumulate into one TMEM accumulator (bf16, or "bf16x3" from hi/lo splits);
//   wide    128 x 256 tiles (a third less operand traffic per FLOP), one CTA per SM, 4 stages,
//           eight epilogue warps;
//   x3wide  "bf16x3" products on 128 x 256 tiles: a stage holds the hi and lo parts of both operands
//           of one K block (96 KiB, loaded once) and the MMA warp issues (lo,hi), (hi,lo), (hi,hi) from
//           them - half the operand traffic per FLOP of three separately loaded segments;
//   split3  fp32-grade products from three-way splits v = hi + mid + lo of both operands: a stage
//           holds the three A parts and the three B parts of one 64-wide K block (96 KiB, loaded
//           once) and the MMA warp issues the six significant part products from them,
//           small magnitudes first.  Every K block is its own accumulation chunk: it goes to a
//           fresh TMEM accumulator that the eight epilogue warps read back and add to a running
//           fp32 sum in registers with round-to-nearest adds.  The tensor core truncates when it
//           adds into its accumulator, which biases long sums (about 1e-6 of the largest term at
//           K = 1024); with one K block per chunk the bias stays at a few 2^-24.
//
// Roles inside a CTA: warp 0 TMA producer (cp.async.bulk.tensor, 128B swizzle), warp 1 TMEM
// allocator + single-thread tcgen05.mma issuer, warps 2.. epilogue (tcgen05.ld -> registers ->
// global; warp w reads TMEM lanes 32*(w%4)..+31, a hardware rule).  Every wait is bounded in wall
// time; on expiry the status word is set and the CTA unwinds.  TMA loads only ever read this GPU's
// memory; peer memory is written with per-thread stores from the epilogue.
#pragma once
#include "sm100_ptx.cuh"

namespace b200 {

constexpr int G2_BM = 128;
constexpr int G2_BK = 64;
constexpr int G2_MAX_SEG = 6;
constexpr int G2_MAX_EXTRA = 7;
constexpr int G2_MAX_BATCH = 256;   // problems of one launch in batch mode
constexpr int G2_A_BYTES = G2_BM * G2_BK * 2;  // 16 KiB

template <int BN, int EPI_WARPS, int MINB, int PARTS>
struct G2Cfg {
  static constexpr int STAGES = PARTS > 1 ? 2 : (BN == 256 ? 4 : (MINB == 2 ? 3 : 6));
  static constexpr int B_BYTES = BN * G2_BK * 2;
  static constexpr int STAGE_BYTES = PARTS * (G2_A_BYTES + B_BYTES);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/ +
                                    4 * (G2_MAX_BATCH + 4) /*item prefix of a batch*/;
};
using G2Plain = G2Cfg<128, 4, 2, 1>;
using G2Wide = G2Cfg<256, 8, 1, 1>;
using G2X3Wide = G2Cfg<256, 8, 1, 2>;
using G2Split3 = G2Cfg<128, 8, 1, 3>;

enum : int {
  G2F_SYM = 1,        // symmetric output: tiles on or below the diagonal only, mirrored
  G2F_A_KMAJOR = 2,   // A given as [M, K] row-major
  G2F_B_KMAJOR = 4,   // B given as [N, K] row-major
  G2F_SAME_AB = 8,    // A and B are the same matrix (diagonal tiles load once; BN = 128 only)
  G2F_ATOMIC = 16,    // C += alpha * result with reductions (C may live on another GPU); beta unused
  G2F_LOWER = 32,     // with G2F_SYM: write / add the lower triangle only
  G2F_WIDE = 64,      // the problem's tensor maps and tile grid are laid out for BN = 256
  G2F_SPLIT3 = 128,   // tmA[0..2] / tmB[0..2] are the (hi, mid, lo) parts of the operands
  G2F_SPLIT2 = 256,   // tmA[0..1] / tmB[0..1] are the (hi, lo) parts of the operands ("bf16x3", wide tiles)
  G2F_MCAST = 512,    // C_extra[] are NVLS multicast addresses: one multimem.st reaches every GPU of the group
  G2F_PAIR = 1024,    // CTA-pair flavour (umma_gemm2_pair.cuh): 128-row tensor maps, tile grid of BN = 256
  G2F_CONV = 2048,    // implicit im2col SYRK: both operands are patch matrices gathered by 4-D TMA loads (below)
};

// Implicit im2col (G2F_CONV): the operand is the patch matrix of a stride-1 convolution input x [N, H, W, C] (bf16,
// channels innermost, C a multiple of 64), columns ordered (kh, kw, c), rows = output pixels.  It never exists in
// memory: a K block is a bw x bh rectangle of output pixels of bi consecutive images (bw * bh * bi = 64, chosen per
// layer so that the blocks cover the output with the least overhang: 8 x 8 x 1 for a 56 x 56 output, 2 x 2 x 16 for
// 14 x 14), a 64-column chunk is 64 channels of one filter tap, and the [64 pixels] x [64 channels] tile of a chunk is
// one 4-D TMA box {64, bw, bh, bi} of x, shifted by the tap offset minus the padding.  Tap q has its own tensor map (slots tmA[0..5], tmB[0..5]) whose W and H extents end
// where the tap's last valid output pixel reads: coordinates before the image are the padding and coordinates past
// the extents belong to output pixels that do not exist - TMA fills both with zeros.  The shared-memory image of a
// box is exactly the MN-major tile of the explicit patch matrix, so the MMA side does not change.


enum : int {
  G2W_NO_SPLIT_OUT = 1,  // work item: do not write the bf16 outputs of the problem for this tile
};

struct alignas(64) GemmProblem2 {
  CUtensorMap tmA[G2_MAX_SEG];
  CUtensorMap tmB[G2_MAX_SEG];
  float* C;               // may be null when only bf16 outputs are wanted
  const float* Cin;       // read when beta != 0 (may alias C)
  __nv_bfloat16* out_hi;  // optional bf16 image of the result
  __nv_bfloat16* out_mid; // optional second part of a three-way split (needs out_hi and out_lo)
  __nv_bfloat16* out_lo;  // optional residual
  float* ws;              // split-K scratch: [tile][split][128][BN] fp32
  int* status;            // device error word
  float* C_extra[G2_MAX_EXTRA];  // plain copies of the fp32 result (same ldc), e.g. peer GPUs
  int n_extra;
  int M, N, K;
  int ldc, ld_out;
  int nseg;
  int tiles_m, tiles_n, ntiles, nsplit;
  int flags;
  int reserved;
  float alpha, beta;
  // G2F_CONV geometry
  int conv_c, conv_kw, conv_taps;   // channels, filter width, kh * kw
  int conv_ph, conv_pw;             // padding
  int conv_th, conv_tw;             // pixel blocks per image column / row
  int conv_box;                     // bw | bh << 8 | bi << 16
};

struct GemmWork2 {
  int problem;
  int a_mn, b_mn;   // first M / N element of the operand tiles
  int a_k0, b_k0;   // first K element of the operand tiles
  int nkb;          // number of 64-wide K blocks
  int c_row, c_col; // output origin
  int tile_id;      // index of the tile inside the problem's split-K scratch
  int split;        // split-K slice
  int wflags;
  int pad;
};

// What the epilogue needs of a problem, read once per work item into registers: a problem of a
// grouped launch lives in global memory, and reading its fields through the pointer between the
// stores would force the compiler to reload them after every store.
struct G2Epi {
  float* C;
  const float* Cin;
  __nv_bfloat16 *out_hi, *out_mid, *out_lo;
  float* ws;
  const GemmProblem2* full;   // for the rarely used fields (extra destinations)
  int M, N, ldc, ld_out, flags, n_extra, nsplit;
  float alpha, beta;
};

__device__ __forceinline__ G2Epi g2_epi(const GemmProblem2& P) {
  G2Epi e;
  e.C = P.C;
  e.Cin = P.Cin;
  e.out_hi = P.out_hi;
  e.out_mid = P.out_mid;
  e.out_lo = P.out_lo;
  e.ws = P.ws;
  e.full = &P;
  e.M = P.M;
  e.N = P.N;
  e.ldc = P.ldc;
  e.ld_out = P.ld_out;
  e.flags = P.flags;
  e.n_extra = P.n_extra;
  e.nsplit = P.nsplit;
  e.alpha = P.alpha;
  e.beta = P.beta;
  return e;
}

// number of column tiles scheduled in tile row tm
template <int BN>
__device__ __forceinline__ int g2_tiles_in_row(const GemmProblem2& P, int tm) {
  return (P.flags & G2F_SYM) ? (tm * G2_BM) / BN + 1 : P.tiles_n;
}

// Work item `idx` of a single-problem launch: idx = tile * nsplit + split.
template <int BN>
__device__ __forceinline__ GemmWork2 g2_decode(const GemmProblem2& P, int idx) {
  GemmWork2 w;
  const int t = idx / P.nsplit;
  w.split = idx - t * P.nsplit;
  int tm = 0, rem = t;
  while (true) {
    const int cnt = g2_tiles_in_row<BN>(P, tm);
    if (rem < cnt) break;
    rem -= cnt;
    ++tm;
  }
  const int kb_total = (P.K + G2_BK - 1) / G2_BK;
  const int kb0 = static_cast<int>((static_cast<long long>(w.split) * kb_total) / P.nsplit);
  const int kb1 = static_cast<int>((static_cast<long long>(w.split + 1) * kb_total) / P.nsplit);
  w.problem = 0;
  w.a_mn = tm * G2_BM;
  w.b_mn = rem * BN;
  w.a_k0 = w.b_k0 = kb0 * G2_BK;
  w.nkb = kb1 - kb0;
  w.c_row = w.a_mn;
  w.c_col = w.b_mn;
  w.tile_id = t;
  w.wflags = 0;
  w.pad = 0;
  return w;
}

// Work item `wi` of a launch, in any of the three ways a launch describes its work:
//   * a work list (plans, the Cholesky steps): item wi is work[wi];
//   * a batch of problems without a list: prefix[p] is the first item of problem p (prefix has
//     n_probs + 1 entries and sits in shared memory); the item is decoded like a single problem's;
//   * one problem passed by value.
template <int BN>
__device__ __forceinline__ const GemmProblem2* g2_item(const GemmProblem2& single, const GemmProblem2* probs,
                                                       const GemmWork2* work, const int* prefix, int n_probs,
                                                       int wi, GemmWork2& w) {
  if (work != nullptr) {
    w = work[wi];
    return probs + w.problem;
  }
  if (probs != nullptr) {
    int lo = 0, hi = n_probs;   // largest p with prefix[p] <= wi
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid] <= wi)
        lo = mid;
      else
        hi = mid;
    }
    w = g2_decode<BN>(probs[lo], wi - prefix[lo]);
    w.problem = lo;
    return probs + lo;
  }
  w = g2_decode<BN>(single, wi);
  return &single;
}

__device__ __forceinline__ void g2_red_add_f32(float* p, float v) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void g2_red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

__device__ __forceinline__ void g2_multimem_st_v4(float* mc, float a, float b, float c, float d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}
__device__ __forceinline__ void g2_multimem_st_f32(float* mc, float a) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(a) : "memory");
}

// 16-byte accesses need a 16-byte aligned row start: ldc a multiple of 4 and an aligned base
__device__ __forceinline__ bool g2_vec_ok(const float* base, int ldc) {
  return ((ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(base) & 15) == 0);
}

// Accumulating variant of the final store (G2F_ATOMIC): every element is added to C with a
// reduction instruction, so that several CTAs / GPUs can contribute to the same matrix.
__device__ __forceinline__ void g2_reduce_chunk(const G2Epi& P, const float* v, int gr, int gc0,
                                                bool diag_tile) {
  if (gr >= P.M) return;
  const bool sym = (P.flags & G2F_SYM) != 0;
  const float alpha = P.alpha;
  float* c = P.C + static_cast<size_t>(gr) * P.ldc + gc0;
  const bool vec_ok = (gc0 + 32 <= P.N) && g2_vec_ok(P.C, P.ldc) && !(sym && diag_tile);
  if (vec_ok) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      g2_red_add_v4_f32(c + 4 * j, alpha * v[4 * j], alpha * v[4 * j + 1], alpha * v[4 * j + 2],
                        alpha * v[4 * j + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int gc = gc0 + j;
      if (gc < P.N && !(sym && diag_tile && gc > gr)) g2_red_add_f32(c + j, alpha * v[j]);
    }
  }
  if (sym && !(P.flags & G2F_LOWER)) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int gc = gc0 + j;
      if (gc < P.N && (!diag_tile || gc < gr))
        g2_red_add_f32(P.C + static_cast<size_t>(gc) * P.ldc + gr, alpha * v[j]);
    }
  }
}

// Final store of 32 consecutive columns of one row held by this thread.
__device__ __forceinline__ void g2_store_chunk(const G2Epi& P, const float* v, int gr, int gc0,
                                               bool diag_tile, bool split_out) {
  if (gr >= P.M) return;
  const bool sym = (P.flags & G2F_SYM) != 0;
  const float alpha = P.alpha, beta = P.beta;
  float out[32];
  const bool full = (gc0 + 32 <= P.N);
  const bool vec_ok = full && g2_vec_ok(P.C != nullptr ? P.C : P.Cin, P.ldc);
  if (beta != 0.f) {
    const float* cin = P.Cin + static_cast<size_t>(gr) * P.ldc + gc0;
    if (vec_ok && g2_vec_ok(P.Cin, P.ldc)) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 c4 = *reinterpret_cast<const float4*>(cin + 4 * j);
        out[4 * j + 0] = alpha * v[4 * j + 0] + beta * c4.x;
        out[4 * j + 1] = alpha * v[4 * j + 1] + beta * c4.y;
        out[4 * j + 2] = alpha * v[4 * j + 2] + beta * c4.z;
        out[4 * j + 3] = alpha * v[4 * j + 3] + beta * c4.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) out[j] = (gc0 + j < P.N) ? alpha * v[j] + beta * cin[j] : 0.f;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) out[j] = alpha * v[j];
  }
  if (P.C != nullptr) {
    float* c = P.C + static_cast<size_t>(gr) * P.ldc + gc0;
    if (!sym || !diag_tile) {
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
      if (sym && !(P.flags & G2F_LOWER)) {  // strictly-lower tile: mirrored (transposed) store
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
          if (gc < gr && !(P.flags & G2F_LOWER)) P.C[static_cast<size_t>(gc) * P.ldc + gr] = out[j];
        }
      }
    }
  }
  for (int e = 0; e < P.n_extra; ++e) {  // plain (non-symmetric) result replicated to peers
    float* const extra = P.full->C_extra[e];
    float* c = extra + static_cast<size_t>(gr) * P.ldc + gc0;
    if (P.flags & G2F_MCAST) {   // through the switch: the store lands in every GPU's copy
      if (full && g2_vec_ok(extra, P.ldc)) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          g2_multimem_st_v4(c + 4 * j, out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gc0 + j < P.N) g2_multimem_st_f32(c + j, out[j]);
      }
    } else if (full && g2_vec_ok(extra, P.ldc)) {
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
  if (P.out_hi != nullptr && split_out) {
    const size_t o = static_cast<size_t>(gr) * P.ld_out + gc0;
    // a symmetric problem's bf16 images are consumed as full matrices: write the mirror image too
    const bool mirror = sym && !(P.flags & G2F_LOWER);
    const bool masked = sym && diag_tile;   // entries above the diagonal are not this tile's to write
    const bool vec = full && !masked && ((P.ld_out & 7) == 0) &&
                     (((reinterpret_cast<uintptr_t>(P.out_hi) | reinterpret_cast<uintptr_t>(P.out_mid) |
                        reinterpret_cast<uintptr_t>(P.out_lo)) & 15) == 0);
    if (vec) {
      // 32 consecutive bf16 per part: four 16-byte stores instead of 32 two-byte ones (a warp's
      // lanes hold different rows, so every store instruction touches 32 sectors either way)
      uint32_t ph[16], pm[16], pl[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float x0 = out[2 * j], x1 = out[2 * j + 1];
        const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
        const float r0 = x0 - __bfloat162float(h0), r1 = x1 - __bfloat162float(h1);
        const __nv_bfloat16 m0 = __float2bfloat16_rn(r0), m1 = __float2bfloat16_rn(r1);
        ph[j] = static_cast<uint32_t>(__bfloat16_as_ushort(h0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h1)) << 16);
        if (P.out_mid != nullptr) {
          const __nv_bfloat16 l0 = __float2bfloat16_rn(r0 - __bfloat162float(m0));
          const __nv_bfloat16 l1 = __float2bfloat16_rn(r1 - __bfloat162float(m1));
          pm[j] = static_cast<uint32_t>(__bfloat16_as_ushort(m0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(m1)) << 16);
          pl[j] = static_cast<uint32_t>(__bfloat16_as_ushort(l0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(l1)) << 16);
        } else {
          pm[j] = 0u;   // two-way split: the residual goes to out_lo
          pl[j] = static_cast<uint32_t>(__bfloat16_as_ushort(m0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(m1)) << 16);
        }
      }
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        *reinterpret_cast<uint4*>(P.out_hi + o + 8 * q4) = make_uint4(ph[4 * q4], ph[4 * q4 + 1], ph[4 * q4 + 2], ph[4 * q4 + 3]);
        if (P.out_mid != nullptr)
          *reinterpret_cast<uint4*>(P.out_mid + o + 8 * q4) = make_uint4(pm[4 * q4], pm[4 * q4 + 1], pm[4 * q4 + 2], pm[4 * q4 + 3]);
        if (P.out_lo != nullptr)
          *reinterpret_cast<uint4*>(P.out_lo + o + 8 * q4) = make_uint4(pl[4 * q4], pl[4 * q4 + 1], pl[4 * q4 + 2], pl[4 * q4 + 3]);
      }
      if (mirror) {   // transposed image: consecutive lanes write consecutive addresses
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const size_t om = static_cast<size_t>(gc0 + j) * P.ld_out + gr;
          const uint32_t wh = ph[j >> 1], wm = pm[j >> 1], wl = pl[j >> 1];
          const unsigned short sh = (j & 1) ? static_cast<unsigned short>(wh >> 16) : static_cast<unsigned short>(wh & 0xffffu);
          const unsigned short sm = (j & 1) ? static_cast<unsigned short>(wm >> 16) : static_cast<unsigned short>(wm & 0xffffu);
          const unsigned short sl = (j & 1) ? static_cast<unsigned short>(wl >> 16) : static_cast<unsigned short>(wl & 0xffffu);
          P.out_hi[om] = __ushort_as_bfloat16(sh);
          if (P.out_mid != nullptr) P.out_mid[om] = __ushort_as_bfloat16(sm);
          if (P.out_lo != nullptr) P.out_lo[om] = __ushort_as_bfloat16(sl);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int gc = gc0 + j;
        if (gc >= P.N || (masked && gc > gr)) continue;
        const float x = out[j];
        const __nv_bfloat16 h = __float2bfloat16_rn(x);
        P.out_hi[o + j] = h;
        const size_t om = static_cast<size_t>(gc) * P.ld_out + gr;
        if (mirror && gc != gr) P.out_hi[om] = h;
        if (P.out_lo != nullptr) {
          const float r1 = x - __bfloat162float(h);
          if (P.out_mid != nullptr) {
            const __nv_bfloat16 m = __float2bfloat16_rn(r1);
            const __nv_bfloat16 l = __float2bfloat16_rn(r1 - __bfloat162float(m));
            P.out_mid[o + j] = m;
            P.out_lo[o + j] = l;
            if (mirror && gc != gr) {
              P.out_mid[om] = m;
              P.out_lo[om] = l;
            }
          } else {
            const __nv_bfloat16 l = __float2bfloat16_rn(r1);
            P.out_lo[o + j] = l;
            if (mirror && gc != gr) P.out_lo[om] = l;
          }
        }
      }
    }
  }
}

template <int BN, int EPI_WARPS, int MINB, int PARTS>
__global__ void __launch_bounds__(64 + 32 * EPI_WARPS, MINB)
umma_gemm2_kernel(const __grid_constant__ GemmProblem2 single, const GemmProblem2* __restrict__ probs,
                  const GemmWork2* __restrict__ work, int n_work, const int* __restrict__ prefix_g, int n_probs) {
  using Cfg = G2Cfg<BN, EPI_WARPS, MINB, PARTS>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr bool SPLIT3 = PARTS == 3;   // fp32-grade products, one accumulation chunk per K block
  constexpr bool SPLIT2 = PARTS == 2;   // bf16x3 products from (hi, lo) parts loaded once per K block
  static_assert(!SPLIT3 || (BN == 128 && EPI_WARPS == 8), "the split3 flavour runs 128-wide tiles with 8 epilogue warps");
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128B swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* prefix = reinterpret_cast<int*>(smem + STAGES * Cfg::STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (prefix_g != nullptr)
    for (int i = threadIdx.x; i <= n_probs && i <= G2_MAX_BATCH; i += blockDim.x) prefix[i] = prefix_g[i];

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], EPI_WARPS);  // one arrival per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int wi = blockIdx.x; wi < n_work && ok; wi += gridDim.x) {
        GemmWork2 w;
        const GemmProblem2& P = *g2_item<BN>(single, probs, work, prefix, n_probs, wi, w);
        const bool a_k = (P.flags & G2F_A_KMAJOR) != 0;
        const bool b_k = (P.flags & G2F_B_KMAJOR) != 0;
        const bool shared_ab = PARTS == 1 && BN == 128 && (P.flags & G2F_SAME_AB) && w.a_mn == w.b_mn &&
                               w.a_k0 == w.b_k0;
        const uint32_t bytes = shared_ab ? G2_A_BYTES : Cfg::STAGE_BYTES;
        const int nseg = PARTS > 1 ? 1 : P.nseg;
        for (int seg = 0; seg < nseg && ok; ++seg) {
          for (int kb = 0; kb < w.nkb; ++kb, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
              set_error(P.status, ERR_WAIT_EMPTY);
              ok = false;
              break;
            }
            uint8_t* stage = smem + s * Cfg::STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], bytes);
            const int ka = w.a_k0 + kb * G2_BK, kbb = w.b_k0 + kb * G2_BK;
            if constexpr (PARTS == 1 && BN == 128) {
              if (P.flags & G2F_CONV) {
                // K block -> (group of images, block of output pixels); 64-column chunk -> (filter tap, channel offset)
                const int pb = ka >> 6, per_img = P.conv_th * P.conv_tw;
                const int bw = P.conv_box & 0xff, bh = (P.conv_box >> 8) & 0xff, bi = P.conv_box >> 16;
                const int ib = pb / per_img, rem = pb - ib * per_img;
                const int img = ib * bi, oy0 = (rem / P.conv_tw) * bh, ox0 = (rem % P.conv_tw) * bw;
                auto gather = [&](uint8_t* dst, int col) {
                  const int q = col / P.conv_c, c0 = col - q * P.conv_c;
                  if (q < P.conv_taps) {
                    const CUtensorMap* tm = q < G2_MAX_SEG ? &P.tmA[q] : &P.tmB[q - G2_MAX_SEG];
                    const int khh = q / P.conv_kw, kww = q - khh * P.conv_kw;
                    tma_load_4d(dst, tm, &full_bar[s], c0, ox0 + kww - P.conv_pw, oy0 + khh - P.conv_ph, img);
                  } else {   // columns past the matrix: a box that lies outside the tensor reads zeros
                    tma_load_4d(dst, &P.tmA[0], &full_bar[s], 0, 0, 1 << 20, img);
                  }
                };
                gather(stage, w.a_mn);
                gather(stage + G2_BK * 128, w.a_mn + 64);
                if (!shared_ab) {
                  gather(stage + G2_A_BYTES, w.b_mn);
                  gather(stage + G2_A_BYTES + G2_BK * 128, w.b_mn + 64);
                }
                continue;
              }
            }
            constexpr int NPART = PARTS;
#pragma unroll
            for (int part = 0; part < NPART; ++part) {
              const CUtensorMap* ta = PARTS > 1 ? &P.tmA[part] : &P.tmA[seg];
              const CUtensorMap* tb = PARTS > 1 ? &P.tmB[part] : &P.tmB[seg];
              uint8_t* sA = stage + part * G2_A_BYTES;
              uint8_t* sB = stage + NPART * G2_A_BYTES + part * Cfg::B_BYTES;
              if (a_k) {
                tma_load_2d(sA, ta, &full_bar[s], ka, w.a_mn);
              } else {
                tma_load_2d(sA, ta, &full_bar[s], w.a_mn, ka);
                tma_load_2d(sA + G2_BK * 128, ta, &full_bar[s], w.a_mn + 64, ka);
              }
              if (!shared_ab) {
                if (b_k) {
                  tma_load_2d(sB, tb, &full_bar[s], kbb, w.b_mn);
                } else {
#pragma unroll
                  for (int h = 0; h < BN / 64; ++h)
                    tma_load_2d(sB + h * G2_BK * 128, tb, &full_bar[s], w.b_mn + 64 * h, kbb);
                }
              }
            }
          }
        }
      }
      if (!ok) {
        // give copies that are still in flight a bounded chance to land before teardown
        const uint32_t pending = it < static_cast<uint32_t>(STAGES) ? it : static_cast<uint32_t>(STAGES);
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t jt = it - 1 - j;
          mbar_wait(&full_bar[jt % STAGES], (jt / STAGES) & 1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------------
    if (lane == 0) {
      uint32_t it = 0, ch = 0;
      bool ok = true;
      for (int wi = blockIdx.x; wi < n_work && ok; wi += gridDim.x) {
        GemmWork2 w;
        const GemmProblem2& P = *g2_item<BN>(single, probs, work, prefix, n_probs, wi, w);
        const bool a_k = (P.flags & G2F_A_KMAJOR) != 0;
        const bool b_k = (P.flags & G2F_B_KMAJOR) != 0;
        const bool shared_ab = PARTS == 1 && BN == 128 && (P.flags & G2F_SAME_AB) && w.a_mn == w.b_mn &&
                               w.a_k0 == w.b_k0;
        const uint32_t idesc = make_idesc_bf16(G2_BM, BN, !a_k, !b_k);
        if (w.nkb <= 0) continue;
        if constexpr (SPLIT3) {
          for (int kb = 0; kb < w.nkb && ok; ++kb, ++it, ++ch) {
            const uint32_t ab = ch & 1;
            if (!mbar_wait(&acc_empty[ab], ((ch >> 1) & 1) ^ 1)) {
              set_error(P.status, ERR_WAIT_ACC);
              ok = false;
              break;
            }
            const int s = it % STAGES;
            if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
              set_error(P.status, ERR_WAIT_FULL);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t tacc = tmem_base + ab * BN;
            const uint32_t base = smem_u32(smem + s * Cfg::STAGE_BYTES);
            // part products in issue order: (lo,hi) (hi,lo) (mid,mid) (mid,hi) (hi,mid) (hi,hi)
            constexpr int PART_A[6] = {2, 0, 1, 1, 0, 0};
            constexpr int PART_B[6] = {0, 2, 1, 0, 1, 0};
#pragma unroll
            for (int pr = 0; pr < 6; ++pr) {
              const uint32_t aA = base + PART_A[pr] * G2_A_BYTES;
              const uint32_t aB = base + 3 * G2_A_BYTES + PART_B[pr] * Cfg::B_BYTES;
#pragma unroll
              for (int k = 0; k < G2_BK / 16; ++k) {
                const uint64_t da = a_k ? make_smem_desc_sw128(aA + k * 32, 16, 1024)
                                        : make_smem_desc_sw128(aA + k * 16 * 128, G2_BK * 128, 1024);
                const uint64_t db = b_k ? make_smem_desc_sw128(aB + k * 32, 16, 1024)
                                        : make_smem_desc_sw128(aB + k * 16 * 128, G2_BK * 128, 1024);
                umma_bf16(tacc, da, db, idesc, (pr | k) ? 1u : 0u);
              }
            }
            umma_commit(&empty_bar[s]);
            umma_commit(&acc_full[ab]);
          }
        } else if constexpr (SPLIT2) {
          const uint32_t ab = ch & 1;
          if (!mbar_wait(&acc_empty[ab], ((ch >> 1) & 1) ^ 1)) {
            set_error(P.status, ERR_WAIT_ACC);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t tacc = tmem_base + ab * BN;
          for (int kb = 0; kb < w.nkb; ++kb, ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
              set_error(P.status, ERR_WAIT_FULL);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t base = smem_u32(smem + s * Cfg::STAGE_BYTES);
            // part products in issue order: (lo,hi) (hi,lo) (hi,hi)
            constexpr int PART_A[3] = {1, 0, 0};
            constexpr int PART_B[3] = {0, 1, 0};
#pragma unroll
            for (int pr = 0; pr < 3; ++pr) {
              const uint32_t aA = base + PART_A[pr] * G2_A_BYTES;
              const uint32_t aB = base + 2 * G2_A_BYTES + PART_B[pr] * Cfg::B_BYTES;
#pragma unroll
              for (int k = 0; k < G2_BK / 16; ++k) {
                const uint64_t da = a_k ? make_smem_desc_sw128(aA + k * 32, 16, 1024)
                                        : make_smem_desc_sw128(aA + k * 16 * 128, G2_BK * 128, 1024);
                const uint64_t db = b_k ? make_smem_desc_sw128(aB + k * 32, 16, 1024)
                                        : make_smem_desc_sw128(aB + k * 16 * 128, G2_BK * 128, 1024);
                umma_bf16(tacc, da, db, idesc, (kb | pr | k) ? 1u : 0u);
              }
            }
            umma_commit(&empty_bar[s]);
          }
          if (ok) umma_commit(&acc_full[ab]);
          ++ch;
        } else {
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
              const uint32_t ph = (it / STAGES) & 1;
              if (!mbar_wait(&full_bar[s], ph)) {
                set_error(P.status, ERR_WAIT_FULL);
                ok = false;
                break;
              }
              tc_fence_after_sync();
              const uint32_t aA = smem_u32(smem + s * Cfg::STAGE_BYTES);
              const uint32_t aB = shared_ab ? aA : aA + G2_A_BYTES;
#pragma unroll
              for (int k = 0; k < G2_BK / 16; ++k) {
                // MN-major: 16 K-rows of 128 B each per MMA; K-major: 16 K-elements = 32 B per MMA.
                const uint64_t da = a_k ? make_smem_desc_sw128(aA + k * 32, 16, 1024)
                                        : make_smem_desc_sw128(aA + k * 16 * 128, G2_BK * 128, 1024);
                const uint64_t db = b_k ? make_smem_desc_sw128(aB + k * 32, 16, 1024)
                                        : make_smem_desc_sw128(aB + k * 16 * 128, G2_BK * 128, 1024);
                umma_bf16(tacc, da, db, idesc, first ? 0u : 1u);
                first = 0;
              }
              umma_commit(&empty_bar[s]);
            }
          }
          if (ok) umma_commit(&acc_full[ab]);
          ++ch;
        }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------------
    const int q = warp & 3;                                   // TMEM lane quarter this warp may access
    constexpr int COLS = BN / (EPI_WARPS / 4);                // columns per warp
    const int col_base = ((warp - 2) >> 2) * COLS;            // first column of this warp's share
    constexpr int PASSES = COLS / 64;
    const int row = q * 32 + lane;
    uint32_t ch = 0;
    bool ok = true;
    for (int wi = blockIdx.x; wi < n_work && ok; wi += gridDim.x) {
      GemmWork2 w;
      const GemmProblem2& Pg = *g2_item<BN>(single, probs, work, prefix, n_probs, wi, w);
      const G2Epi P = g2_epi(Pg);
      int* const status = Pg.status;
      const int nchunks = SPLIT3 ? w.nkb : (w.nkb > 0 ? 1 : 0);
      const int gr = w.c_row + row;
      const bool sym = (P.flags & G2F_SYM) != 0;
      const bool atomic = (P.flags & G2F_ATOMIC) != 0;
      const bool to_ws = P.nsplit > 1 && !atomic;
      const bool split_out = !(w.wflags & G2W_NO_SPLIT_OUT);
      const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;

      auto finish = [&](const float* v, int col0) {
        // v: 64 consecutive columns of this thread's row starting at tile column col0
        if (to_ws) {
          float* part = P.ws + (static_cast<size_t>(w.tile_id) * P.nsplit + w.split) * (G2_BM * BN) +
                        static_cast<size_t>(row) * BN + col0;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            *reinterpret_cast<float4*>(part + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          return;
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int gc0 = w.c_col + col0 + c * 32;
          // with wide tiles a symmetric problem's tile may reach past the diagonal block: skip that part
          const bool beyond = sym && (gc0 / G2_BM) > (w.c_row / G2_BM);
          const bool diag = sym && (gc0 / G2_BM) == (w.c_row / G2_BM);
          if (gc0 < P.N && !beyond && !(diag && gc0 > gr)) {
            if (atomic)
              g2_reduce_chunk(P, v + c * 32, gr, gc0, diag);
            else
              g2_store_chunk(P, v + c * 32, gr, gc0, diag, split_out);
          }
        }
      };

      if constexpr (!SPLIT3) {
        const uint32_t ab = ch & 1;
        if (nchunks == 1) {
          ok = mbar_wait(&acc_full[ab], (ch >> 1) & 1);
          if (!ok) set_error(status, ERR_WAIT_ACC);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
        }
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) {
          float v[64];
          const int col0 = col_base + pass * 64;
          if (nchunks == 1) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(tmem_base + lane_addr + ab * BN + col0, r0);
            tmem_ld_32x32(tmem_base + lane_addr + ab * BN + col0 + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[j] = __uint_as_float(r0[j]);
              v[32 + j] = __uint_as_float(r1[j]);
            }
            if (pass == PASSES - 1) {  // everything this warp needs is in registers: free the accumulator
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[ab]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = 0.f;
          }
          finish(v, col0);
        }
        if (nchunks == 1) ++ch;
      } else {
        // one chunk per K block: running fp32 sum in registers
        float run[64];
#pragma unroll
        for (int j = 0; j < 64; ++j) run[j] = 0.f;
        for (int c = 0; c < nchunks; ++c, ++ch) {
          const uint32_t ab = ch & 1;
          ok = mbar_wait(&acc_full[ab], (ch >> 1) & 1);
          if (!ok) set_error(status, ERR_WAIT_ACC);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(tmem_base + lane_addr + ab * BN + col_base, r0);
          tmem_ld_32x32(tmem_base + lane_addr + ab * BN + col_base + 32, r1);
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[ab]);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            run[j] += __uint_as_float(r0[j]);
            run[32 + j] += __uint_as_float(r1[j]);
          }
        }
        if (!ok) break;
        finish(run, col_base);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// Sums split-K partials and applies the epilogue.  One block handles a 32x32 patch of one tile:
// reads and direct stores are 128-byte coalesced, the mirrored store goes through shared memory.
// grid: (work items, 4 * BN / 32).
template <int BN>
__global__ void __launch_bounds__(256)
splitk_reduce2_kernel(const __grid_constant__ GemmProblem2 single, const GemmProblem2* __restrict__ probs,
                      const GemmWork2* __restrict__ work, const int* __restrict__ tile_prefix, int n_probs) {
  __shared__ float tile[32][33];
  GemmWork2 w;
  const GemmProblem2* Pp;
  if (work != nullptr) {
    w = work[blockIdx.x];
    Pp = probs + w.problem;
  } else if (probs != nullptr) {
    // batch mode: tile_prefix[p] is the first tile (over the problems that were split) of problem p
    int lo = 0, hi = n_probs;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tile_prefix[mid] <= static_cast<int>(blockIdx.x))
        lo = mid;
      else
        hi = mid;
    }
    Pp = probs + lo;
    w = g2_decode<BN>(*Pp, (static_cast<int>(blockIdx.x) - tile_prefix[lo]) * Pp->nsplit);
  } else {
    w = g2_decode<BN>(single, blockIdx.x * single.nsplit);
    Pp = &single;
  }
  const G2Epi P = g2_epi(*Pp);
  const bool sym = (P.flags & G2F_SYM) != 0;
  constexpr int PC = BN / 32;  // patches per tile row
  const int sub_r = blockIdx.y / PC, sub_c = blockIdx.y % PC;
  const int tm = w.c_row / G2_BM;
  const int cb = (w.c_col + sub_c * 32) / G2_BM;  // 128-wide column block of this patch
  if (sym && cb > tm) return;
  const bool diag_tile = sym && cb == tm;
  if (diag_tile && (w.c_col + sub_c * 32) > (w.c_row + sub_r * 32)) return;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  // patches that lie completely outside the matrix (edge tiles of small problems) have no work
  if (w.c_row + sub_r * 32 >= P.M || w.c_col + sub_c * 32 >= P.N) return;
  const float* base = P.ws + static_cast<size_t>(w.tile_id) * P.nsplit * (G2_BM * BN);
  const int gc = w.c_col + sub_c * 32 + tx;
  // sum the partials in split order; the loads of the four rows of a thread and of four splits are
  // issued together (16 independent loads in flight per thread)
  float accs[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const float* p0 = base + static_cast<size_t>(sub_r * 32 + ty) * BN + sub_c * 32 + tx;
    int s = 0;
    for (; s + 4 <= P.nsplit; s += 4) {
      float v[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u)
          v[i][u] = __ldcg(p0 + static_cast<size_t>(8 * i) * BN + static_cast<size_t>(s + u) * (G2_BM * BN));
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u) accs[i] += v[i][u];
    }
    for (; s < P.nsplit; ++s)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        accs[i] += __ldcg(p0 + static_cast<size_t>(8 * i) * BN + static_cast<size_t>(s) * (G2_BM * BN));
  }
  const bool mirror_bf16 = sym && !(P.flags & G2F_LOWER);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = ty + 8 * i;
    const int gr = w.c_row + sub_r * 32 + lr;
    float val = P.alpha * accs[i];
    const bool inb = gr < P.M && gc < P.N;
    if (inb && P.beta != 0.f) val += P.beta * P.Cin[static_cast<size_t>(gr) * P.ldc + gc];
    tile[lr][tx] = val;
    const bool keep = inb && !(diag_tile && gc > gr);
    if (keep) {
      if (P.C != nullptr) P.C[static_cast<size_t>(gr) * P.ldc + gc] = val;
      for (int e = 0; e < P.n_extra; ++e) {
        float* dst = P.full->C_extra[e] + static_cast<size_t>(gr) * P.ldc + gc;
        if (P.flags & G2F_MCAST)
          g2_multimem_st_f32(dst, val);
        else
          *dst = val;
      }
      if (P.out_hi != nullptr) {
        const size_t o = static_cast<size_t>(gr) * P.ld_out + gc;
        const size_t om = static_cast<size_t>(gc) * P.ld_out + gr;
        const bool mir = mirror_bf16 && gc != gr;
        const __nv_bfloat16 h = __float2bfloat16_rn(val);
        P.out_hi[o] = h;
        if (mir) P.out_hi[om] = h;
        if (P.out_lo != nullptr) {
          const float r1 = val - __bfloat162float(h);
          if (P.out_mid != nullptr) {
            const __nv_bfloat16 m = __float2bfloat16_rn(r1);
            const __nv_bfloat16 l = __float2bfloat16_rn(r1 - __bfloat162float(m));
            P.out_mid[o] = m;
            P.out_lo[o] = l;
            if (mir) {
              P.out_mid[om] = m;
              P.out_lo[om] = l;
            }
          } else {
            const __nv_bfloat16 l = __float2bfloat16_rn(r1);
            P.out_lo[o] = l;
            if (mir) P.out_lo[om] = l;
          }
        }
      }
    }
  }
  if (!sym || P.C == nullptr || (P.flags & G2F_LOWER)) return;
  __syncthreads();
  // mirrored store: element (r, c) of the patch goes to C[c][r]
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lc = ty + 8 * i;                       // patch column -> destination row
    const int dst_r = w.c_col + sub_c * 32 + lc;     // global column index of the source
    const int dst_c = w.c_row + sub_r * 32 + tx;     // global row index of the source
    if (dst_r < P.N && dst_c < P.M && dst_r < dst_c)
      P.C[static_cast<size_t>(dst_r) * P.ldc + dst_c] = tile[tx][lc];
  }
}

}  // namespace b200
