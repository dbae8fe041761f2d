// Host-side interface of the persistent tcgen05 GEMM (umma_gemm2.cuh) for the other translation
// units of the extension (the tensor-core Cholesky inverse builds its own problem tables and work
// lists and runs them through these launchers).
#pragma once
#include "host_utils.h"
#include "umma_gemm2.cuh"

namespace b200 {

enum G2Flavour { G2_PLAIN = 0, G2_WIDE = 1, G2_SPLIT3 = 2, G2_X3WIDE = 3, G2_PAIR = 4 };

// Tensor map of one bf16 operand.  `mn` x `k` logical extents; `kmajor`: stored [mn, k] row-major
// with pitch `ld` elements, otherwise stored [k, mn] row-major.  `box_mn`: tile extent along MN
// for K-major operands (128 for A, the tile width for B); MN-major operands are always loaded as
// 64 x 64 boxes.
void g2_encode_operand(CUtensorMap* tm, const void* base, int64_t mn, int64_t k, int64_t ld,
                       bool kmajor, int box_mn);

// SM count of a device (cached).
int g2_sm_count(int dev);

// One launch of a kernel flavour: either `single` (work == nullptr; its tiles are decoded from the
// work index), a device-resident problem table with a work list, or such a table with an item
// prefix per problem (`prefix`, `n_probs` <= G2_MAX_BATCH; `work` null).  Defined in gemm2_<flavour>.cu.
void g2_run_plain(const GemmProblem2& single, const GemmProblem2* probs, const GemmWork2* work, int n_work,
                  int n_sms, cudaStream_t stream, const int* prefix = nullptr, int n_probs = 0);
void g2_run_wide(const GemmProblem2& single, const GemmProblem2* probs, const GemmWork2* work, int n_work,
                 int n_sms, cudaStream_t stream, const int* prefix = nullptr, int n_probs = 0);
void g2_run_x3wide(const GemmProblem2& single, const GemmProblem2* probs, const GemmWork2* work, int n_work,
                   int n_sms, cudaStream_t stream, const int* prefix = nullptr, int n_probs = 0);
void g2_run_split3(const GemmProblem2& single, const GemmProblem2* probs, const GemmWork2* work, int n_work,
                   int n_sms, cudaStream_t stream, const int* prefix = nullptr, int n_probs = 0);

// CTA-pair flavour (tcgen05.mma.cta_group::2, umma_gemm2_pair.cuh): one problem by value, `n_work`
// pair tiles x split-K slices.  Defined in gemm2_pair.cu.
void g2_run_pair(const GemmProblem2& single, int n_work, int n_sms, cudaStream_t stream);
// number of 256 x 256 pair tiles of a problem laid out for this flavour
int g2_pair_tiles(const GemmProblem2& P);

// Runs `n_work` work items of a device-resident problem table on `stream`.
void g2_launch_list(const GemmProblem2* d_probs, const GemmWork2* d_work, int n_work, G2Flavour flavour,
                    int dev, cudaStream_t stream);

// Split-K reduction of the listed tiles (one work item per tile).
void g2_launch_reduce_list(const GemmProblem2* d_probs, const GemmWork2* d_work, int n_work, bool wide,
                           cudaStream_t stream);

}  // namespace b200
