// Collectives over NVLink peer memory for buffers that every rank allocated symmetrically (the
// same size at the same offset on every GPU, mapped into every rank's address space).
//
//   symm_barrier          all ranks meet: each rank stores an epoch into its slot on every peer
//                         (st.release.sys) and waits until all of its own slots carry that epoch
//                         (ld.acquire.sys).  Every wait is bounded in wall time (the caller
//                         passes the limit); on expiry the status word is set to
//                         ERR_WAIT_PEER and the kernel returns.
//   symm_reduce_segments  the calling rank pulls the listed segments from every peer with plain
//                         peer loads, sums them, scales, and stores the result locally
//                         (reduce-to-owner of gradients / statistics).
//   symm_bcast_segments   the calling rank stores the listed segments into every peer's copy
//                         (broadcast-from-owner of preconditioned gradients).
//   symm_scale_segments   local beta-scaling of segments (moving-average decay of owned factors).
//   symm_reduce_slots     owner-side sum of the per-rank slots that the peers' SYRK epilogues stored
//                         into (lower triangles), folded into the running factor and mirrored.
//   symm_pull_slots       the same sum with every rank's contribution read from that rank's own buffer
//                         (coalesced peer loads): the SYRK epilogues store locally.
//   symm_mirror_lower     upper triangle <- lower triangle of local matrices.
//   symm_bucket_reduce    one kernel per gradient bucket on a communication stream: every rank
//                         announces "my part of this bucket is in place", waits (bounded) for all
//                         ranks, and the owner of each listed segment pulls the sum - through the
//                         NVSwitch with one multimem.ld_reduce per 16 bytes where the buffer has a
//                         multicast mapping, with one plain peer load per rank otherwise.
//   symm_bcast_segments   with a multicast mapping one multimem.st per 16 bytes reaches every rank.
//
// The first SYMM_FLAG_WORDS 32-bit words of the symmetric buffer are reserved for the barrier
// slots: word [s * 64 + r] of rank q is "rank r has reached epoch of barrier stream s"; word
// [s * 64 + 63] counts the barriers this rank has entered on stream s.
// Peer data is always accessed with plain per-thread loads and stores; bulk-copy engines are
// not used on peer memory.
#include "host_utils.h"
#include "sm100_ptx.cuh"

namespace b200 {

constexpr int SYMM_FLAG_WORDS = 256;

struct Seg {
  long long off;    // element offset inside the symmetric buffer (fp32 elements)
  long long numel;  // multiple of 4
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_f4(float* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

// ---- NVLS: one instruction per 16 bytes reads the sum over all ranks / writes to all ranks --------
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

__global__ void symm_barrier_kernel(const long long* peers, int rank, int world, int slot,
                                    unsigned long long wait_ns, int* status) {
  // The epoch lives in this rank's own flag area (word 63 of the slot), so the kernel carries no
  // per-call argument and can be replayed from a CUDA graph.
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) {
    uint32_t* counter = reinterpret_cast<uint32_t*>(peers[rank]) + slot * 64 + 63;
    s_epoch = *counter + 1;
    *counter = s_epoch;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  uint32_t* remote = reinterpret_cast<uint32_t*>(peers[t]) + slot * 64 + rank;
  st_release_sys(remote, epoch);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(peers[rank]) + slot * 64 + t;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
    if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > wait_ns) {
      set_error(status, ERR_WAIT_PEER);
      return;
    }
  }
}

__global__ void symm_reduce_segments_kernel(const long long* peers, int rank, int world,
                                            const Seg* segs, float scale, const float* mc_base) {
  const Seg s = segs[blockIdx.y];
  float* local = reinterpret_cast<float*>(peers[rank]) + s.off;
  const long long n4 = s.numel >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mc_base != nullptr) {   // the switch adds the ranks' copies: one transaction per 16 bytes
      acc = multimem_ld_reduce_f4(mc_base + s.off + 4 * i);
    } else
    for (int r = 0; r < world; ++r) {
      const float4 v = ld_peer_f4(reinterpret_cast<const float*>(peers[r]) + s.off + 4 * i);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    acc.x *= scale;
    acc.y *= scale;
    acc.z *= scale;
    acc.w *= scale;
    *reinterpret_cast<float4*>(local + 4 * i) = acc;
  }
}

__global__ void symm_bcast_segments_kernel(const long long* peers, int rank, int world, const Seg* segs,
                                           float* mc_base) {
  const Seg s = segs[blockIdx.y];
  const float* local = reinterpret_cast<const float*>(peers[rank]) + s.off;
  const long long n4 = s.numel >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = *reinterpret_cast<const float4*>(local + 4 * i);
    if (mc_base != nullptr) {
      multimem_st_f4(mc_base + s.off + 4 * i, v);   // the switch delivers it to every rank (this one too)
    } else {
      for (int r = 0; r < world; ++r)
        if (r != rank) st_peer_f4(reinterpret_cast<float*>(peers[r]) + s.off + 4 * i, v);
    }
  }
}

// Flag exchange + owner pull of one gradient bucket in one kernel.  Flag words of barrier slot
// `slot` in this rank's buffer: [slot*64 + r] "rank r has reached epoch", [slot*64 + 63] the epoch
// of the last completed call, [slot*64 + 62] count of blocks that finished the current call.  The
// epoch word only changes when the last block of a call retires, so every block of a call reads
// the same value at its start and no per-call host argument is needed (CUDA-graph replay).
constexpr int BUCKET_UNROLL = 8;
constexpr int BUCKET_THREADS = 128;

__global__ void __launch_bounds__(BUCKET_THREADS) symm_bucket_reduce_kernel(const long long* peers, int rank, int world, int slot,
                                          const Seg* segs, int nsegs, float scale, const float* mc_base,
                                          unsigned long long wait_ns, int* status) {
  uint32_t* flags = reinterpret_cast<uint32_t*>(peers[rank]) + slot * 64;
  __shared__ int s_ok;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(flags + 63) + 1;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();   // this rank's bucket (written by earlier kernels of the stream) before the flag
    st_release_sys(reinterpret_cast<uint32_t*>(peers[threadIdx.x]) + slot * 64 + rank, epoch);
  }
  if (threadIdx.x < world) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > wait_ns) {
        set_error(status, ERR_WAIT_PEER);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (s_ok) {
    const float* peer[8];
    const int wcap = world < 8 ? world : 8;
    for (int r = 0; r < wcap; ++r) peer[r] = reinterpret_cast<const float*>(peers[r]);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (int sidx = 0; sidx < nsegs; ++sidx) {
      const Seg s = segs[sidx];
      float* local = reinterpret_cast<float*>(peers[rank]) + s.off;
      const long long n4 = s.numel >> 2;
      // BUCKET_UNROLL independent 16-byte transactions per thread and trip: the pull is bound by the
      // latency of the link, so the number of loads in flight sets its speed.  The blocks are small
      // (128 threads) on purpose: while a block waits for a peer it stays resident next to the
      // kernels of the backward pass, and a fat block would take registers those kernels need.
      for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < n4;
           i0 += BUCKET_UNROLL * stride) {
        float4 acc[BUCKET_UNROLL];
#pragma unroll
        for (int u = 0; u < BUCKET_UNROLL; ++u) {
          const long long i = i0 + u * stride;
          acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (i < n4) {
            if (mc_base != nullptr) {
              acc[u] = multimem_ld_reduce_f4(mc_base + s.off + 4 * i);
            } else if (world <= 8) {
#pragma unroll
              for (int r = 0; r < 8; ++r)
                if (r < world) {
                  const float4 v = ld_peer_f4(peer[r] + s.off + 4 * i);
                  acc[u].x += v.x;
                  acc[u].y += v.y;
                  acc[u].z += v.z;
                  acc[u].w += v.w;
                }
            } else {
              for (int r = 0; r < world; ++r) {
                const float4 v = ld_peer_f4(reinterpret_cast<const float*>(peers[r]) + s.off + 4 * i);
                acc[u].x += v.x;
                acc[u].y += v.y;
                acc[u].z += v.z;
                acc[u].w += v.w;
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < BUCKET_UNROLL; ++u) {
          const long long i = i0 + u * stride;
          if (i < n4)
            *reinterpret_cast<float4*>(local + 4 * i) =
                make_float4(acc[u].x * scale, acc[u].y * scale, acc[u].z * scale, acc[u].w * scale);
        }
      }
    }
  }
  // retire: the last block publishes the epoch for the next call
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(flags + 62, 1u) + 1;
    if (done == gridDim.x) {
      flags[62] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(flags + 63) = epoch;
    }
  }
}

__global__ void symm_scale_segments_kernel(float* base, const Seg* segs, float beta) {
  const Seg s = segs[blockIdx.y];
  float* p = base + s.off;
  const long long n4 = s.numel >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 v = *reinterpret_cast<float4*>(p + 4 * i);
    v.x *= beta;
    v.y *= beta;
    v.z *= beta;
    v.w *= beta;
    *reinterpret_cast<float4*>(p + 4 * i) = v;
  }
}


// upper triangle <- transpose of the lower triangle for square matrices inside the buffer
// (segment rows: offset, n).  One block per 32x32 tile on or below the diagonal.
__global__ void symm_mirror_lower_kernel(float* base, const Seg* mats, int tiles_max) {
  __shared__ float tile[32][33];
  const Seg m = mats[blockIdx.y];
  const int n = static_cast<int>(m.numel);
  const int nt = (n + 31) / 32;
  const int t = blockIdx.x;
  if (t >= nt * (nt + 1) / 2) return;
  int r = static_cast<int>((sqrtf(8.f * t + 1.f) - 1.f) * 0.5f);
  while ((r + 1) * (r + 2) / 2 <= t) ++r;
  while (r * (r + 1) / 2 > t) --r;
  const int tr = r, tc = t - r * (r + 1) / 2;  // tile row >= tile column
  float* a = base + m.off;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int gr = tr * 32 + i, gc = tc * 32 + tx;
    tile[i][tx] = (gr < n && gc < n) ? a[static_cast<size_t>(gr) * n + gc] : 0.f;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int dr = tc * 32 + i, dc = tr * 32 + tx;  // destination (row, col) = source (col, row)
    if (dr < n && dc < n && dc > dr) a[static_cast<size_t>(dr) * n + dc] = tile[tx][i];
  }
}

// Owner-side reduction of per-rank slots into a running factor, for square matrices:
//   F <- beta * F + sum_r slot_r     on the lower triangle, mirrored into the upper one.
// Row t of `table`: (offset of F, offset of slot 0, n); slot r starts `slot_stride` elements after
// slot r-1.  Everything is local memory: the peers stored their lower-triangular tiles into the
// slots with plain (coalesced) stores from their SYRK epilogues.
struct SlotRow {
  long long f_off, slot_off, n;
};

__global__ void symm_reduce_slots_kernel(float* base, const SlotRow* table, int world, long long slot_stride,
                                         float beta) {
  __shared__ float tile[32][33];
  const SlotRow m = table[blockIdx.y];
  const int n = static_cast<int>(m.n);
  const int nt = (n + 31) / 32;
  const int t = blockIdx.x;
  if (t >= nt * (nt + 1) / 2) return;
  int r = static_cast<int>((sqrtf(8.f * t + 1.f) - 1.f) * 0.5f);
  while ((r + 1) * (r + 2) / 2 <= t) ++r;
  while (r * (r + 1) / 2 > t) --r;
  const int tr = r, tc = t - r * (r + 1) / 2;  // tile row >= tile column
  float* f = base + m.f_off;
  const float* slot0 = base + m.slot_off;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int gr = tr * 32 + i, gc = tc * 32 + tx;
    float v = 0.f;
    if (gr < n && gc < n && gc <= gr) {
      const size_t idx = static_cast<size_t>(gr) * n + gc;
      for (int q = 0; q < world; ++q) v += slot0[q * slot_stride + idx];
      if (beta != 0.f) v = fmaf(beta, f[idx], v);
      f[idx] = v;
    }
    tile[i][tx] = v;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int dr = tc * 32 + i, dc = tr * 32 + tx;  // destination (row, col) = source (col, row)
    if (dr < n && dc < n && dc > dr) f[static_cast<size_t>(dr) * n + dc] = tile[tx][i];
  }
}

// Pull variant: every rank keeps its own contribution to a factor in ITS OWN buffer (the SYRK epilogue
// stores locally), at the same offset on every rank; the owner reads that offset from every rank with
// coalesced loads over NVLink (128 bytes per warp and row), sums in rank order and mirrors.  A lane-per-row
// epilogue store into a peer is sixteen bytes per lane and instruction; a pull moves whole lines.
__device__ __forceinline__ float ld_peer_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

__global__ void symm_pull_slots_kernel(float* base, const long long* __restrict__ peers, const SlotRow* table, int world,
                                       float beta) {
  __shared__ float tile[32][33];
  const SlotRow m = table[blockIdx.y];
  const int n = static_cast<int>(m.n);
  const int nt = (n + 31) / 32;
  const int t = blockIdx.x;
  if (t >= nt * (nt + 1) / 2) return;
  int r = static_cast<int>((sqrtf(8.f * t + 1.f) - 1.f) * 0.5f);
  while ((r + 1) * (r + 2) / 2 <= t) ++r;
  while (r * (r + 1) / 2 > t) --r;
  const int tr = r, tc = t - r * (r + 1) / 2;  // tile row >= tile column
  float* f = base + m.f_off;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  // the four rows of a thread and up to four ranks at a time: sixteen loads in flight per thread
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  bool live[4];
  size_t idx[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int gr = tr * 32 + ty + 8 * k, gc = tc * 32 + tx;
    live[k] = gr < n && gc < n && gc <= gr;
    idx[k] = static_cast<size_t>(gr) * n + gc;
  }
  for (int q0 = 0; q0 < world; q0 += 4) {
    float v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const bool have = q0 + u < world;
      const float* src = have ? reinterpret_cast<const float*>(peers[q0 + u]) + m.slot_off : nullptr;
#pragma unroll
      for (int k = 0; k < 4; ++k) v[u][k] = (have && live[k]) ? ld_peer_f32(src + idx[k]) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] += v[u][k];
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float v = acc[k];
    if (live[k]) {
      if (beta != 0.f) v = fmaf(beta, f[idx[k]], v);
      f[idx[k]] = v;
    }
    tile[ty + 8 * k][tx] = live[k] ? v : 0.f;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int dr = tc * 32 + i, dc = tr * 32 + tx;  // destination (row, col) = source (col, row)
    if (dr < n && dc < n && dc > dr) f[static_cast<size_t>(dr) * n + dc] = tile[tx][i];
  }
}

// ---- host ------------------------------------------------------------------------------------
static int sm_count(int dev) { return at::cuda::getDeviceProperties(dev)->multiProcessorCount; }

static void check_table(const at::Tensor& peers, int world) {
  TORCH_CHECK(peers.is_cuda() && peers.scalar_type() == at::kLong && peers.is_contiguous() &&
                  peers.numel() == world, "peers must be a CUDA int64 vector with one pointer per rank");
}
static void check_segs(const at::Tensor& segs) {
  TORCH_CHECK(segs.is_cuda() && segs.scalar_type() == at::kLong && segs.is_contiguous() &&
                  segs.dim() == 2 && segs.size(1) == 2, "segments must be a CUDA int64 [k, 2] tensor");
}

void symm_barrier(at::Tensor peers, int64_t rank, int64_t world, int64_t slot, int64_t wait_ms) {
  check_table(peers, static_cast<int>(world));
  TORCH_CHECK(world <= 63 && slot >= 0 && slot * 64 + 64 <= SYMM_FLAG_WORDS, "bad barrier slot");
  TORCH_CHECK(wait_ms > 0 && wait_ms <= 60000, "the barrier wait limit must be in (0, 60000] ms");
  const int dev = peers.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  symm_barrier_kernel<<<1, 64, 0, stream>>>(reinterpret_cast<const long long*>(peers.data_ptr<int64_t>()),
                                            static_cast<int>(rank), static_cast<int>(world),
                                            static_cast<int>(slot),
                                            static_cast<unsigned long long>(wait_ms) * 1000000ull,
                                            device_state(dev).status.data_ptr<int>());
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

void symm_reduce_segments(at::Tensor peers, int64_t rank, int64_t world, at::Tensor segs, double scale,
                          int64_t mc_ptr) {
  check_table(peers, static_cast<int>(world));
  check_segs(segs);
  if (segs.size(0) == 0) return;
  const int dev = peers.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  dim3 grid(sm_count(dev), static_cast<unsigned>(segs.size(0)));
  symm_reduce_segments_kernel<<<grid, 256, 0, stream>>>(
      reinterpret_cast<const long long*>(peers.data_ptr<int64_t>()), static_cast<int>(rank),
      static_cast<int>(world), reinterpret_cast<const Seg*>(segs.data_ptr<int64_t>()),
      static_cast<float>(scale), reinterpret_cast<const float*>(mc_ptr));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// `mc_ptr`: address of the buffer's multicast mapping (0: none, plain peer stores are used)
void symm_bcast_segments(at::Tensor peers, int64_t rank, int64_t world, at::Tensor segs, int64_t mc_ptr) {
  check_table(peers, static_cast<int>(world));
  check_segs(segs);
  if (segs.size(0) == 0) return;
  const int dev = peers.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  dim3 grid(sm_count(dev), static_cast<unsigned>(segs.size(0)));
  symm_bcast_segments_kernel<<<grid, 256, 0, stream>>>(
      reinterpret_cast<const long long*>(peers.data_ptr<int64_t>()), static_cast<int>(rank),
      static_cast<int>(world), reinterpret_cast<const Seg*>(segs.data_ptr<int64_t>()),
      reinterpret_cast<float*>(mc_ptr));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// One gradient bucket: flag exchange on barrier slot `slot`, then this rank pulls the sum of the
// listed segments (the ones it owns) scaled by `scale`.  Every rank has to make the call for every
// bucket, with an empty segment list if it owns nothing in it.  `blocks`: CTAs of the kernel (the
// pull shares the GPU with the backward pass it overlaps).
void symm_bucket_reduce(at::Tensor peers, int64_t rank, int64_t world, int64_t slot, at::Tensor segs, double scale,
                        int64_t mc_ptr, int64_t wait_ms, int64_t blocks) {
  check_table(peers, static_cast<int>(world));
  check_segs(segs);
  TORCH_CHECK(world <= 62 && slot >= 0 && slot * 64 + 64 <= SYMM_FLAG_WORDS, "bad barrier slot");
  TORCH_CHECK(wait_ms > 0 && wait_ms <= 60000, "the wait limit must be in (0, 60000] ms");
  TORCH_CHECK(blocks >= 1 && blocks <= 1024, "blocks out of range");
  const int dev = peers.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  symm_bucket_reduce_kernel<<<static_cast<unsigned>(blocks), BUCKET_THREADS, 0, stream>>>(
      reinterpret_cast<const long long*>(peers.data_ptr<int64_t>()), static_cast<int>(rank), static_cast<int>(world),
      static_cast<int>(slot), reinterpret_cast<const Seg*>(segs.data_ptr<int64_t>()), static_cast<int>(segs.size(0)),
      static_cast<float>(scale), reinterpret_cast<const float*>(mc_ptr),
      static_cast<unsigned long long>(wait_ms) * 1000000ull, device_state(dev).status.data_ptr<int>());
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

void symm_scale_segments(at::Tensor local, at::Tensor segs, double beta) {
  TORCH_CHECK(local.is_cuda() && local.scalar_type() == at::kFloat && local.is_contiguous(),
              "local must be a contiguous fp32 CUDA tensor");
  check_segs(segs);
  if (segs.size(0) == 0) return;
  const int dev = local.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  dim3 grid(sm_count(dev), static_cast<unsigned>(segs.size(0)));
  symm_scale_segments_kernel<<<grid, 256, 0, stream>>>(
      local.data_ptr<float>(), reinterpret_cast<const Seg*>(segs.data_ptr<int64_t>()),
      static_cast<float>(beta));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// mats: [k, 2] rows of (element offset inside `local`, matrix size n); n_max: the largest n (host value,
// so that the call needs no device read and can be captured in a CUDA graph).
void symm_mirror_lower(at::Tensor local, at::Tensor mats, int64_t n_max) {
  TORCH_CHECK(local.is_cuda() && local.scalar_type() == at::kFloat && local.is_contiguous(),
              "local must be a contiguous fp32 CUDA tensor");
  check_segs(mats);
  if (mats.size(0) == 0) return;
  TORCH_CHECK(n_max > 0, "n_max must be the largest matrix size");
  const int nt = static_cast<int>((n_max + 31) / 32);
  const int dev = local.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  dim3 grid(nt * (nt + 1) / 2, static_cast<unsigned>(mats.size(0)));
  symm_mirror_lower_kernel<<<grid, 256, 0, stream>>>(local.data_ptr<float>(),
                                                     reinterpret_cast<const Seg*>(mats.data_ptr<int64_t>()), nt);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// table: [k, 3] rows of (offset of the factor, offset of slot 0, n) inside `local`.
void symm_reduce_slots(at::Tensor local, at::Tensor table, int64_t world, int64_t slot_stride, int64_t n_max,
                       double beta) {
  TORCH_CHECK(local.is_cuda() && local.scalar_type() == at::kFloat && local.is_contiguous(),
              "local must be a contiguous fp32 CUDA tensor");
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.is_contiguous() && table.dim() == 2 &&
                  table.size(1) == 3, "table must be a CUDA int64 [k, 3] tensor");
  if (table.size(0) == 0) return;
  TORCH_CHECK(n_max > 0 && world > 0, "bad arguments");
  const int nt = static_cast<int>((n_max + 31) / 32);
  const int dev = local.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  dim3 grid(nt * (nt + 1) / 2, static_cast<unsigned>(table.size(0)));
  symm_reduce_slots_kernel<<<grid, 256, 0, stream>>>(local.data_ptr<float>(),
                                                     reinterpret_cast<const SlotRow*>(table.data_ptr<int64_t>()),
                                                     static_cast<int>(world), slot_stride, static_cast<float>(beta));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// table: [k, 3] rows of (offset of the local factor, offset of the contribution on EVERY rank, n); peers: one
// base pointer per rank.  factor <- beta * factor + sum over ranks of their contributions (lower triangles), mirrored.
void symm_pull_slots(at::Tensor local, at::Tensor peers, at::Tensor table, int64_t world, int64_t n_max, double beta) {
  TORCH_CHECK(local.is_cuda() && local.scalar_type() == at::kFloat && local.is_contiguous(),
              "local must be a contiguous fp32 CUDA tensor");
  check_table(peers, static_cast<int>(world));
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.is_contiguous() && table.dim() == 2 &&
                  table.size(1) == 3, "table must be a CUDA int64 [k, 3] tensor");
  if (table.size(0) == 0) return;
  TORCH_CHECK(n_max > 0 && world > 0, "bad arguments");
  const int nt = static_cast<int>((n_max + 31) / 32);
  const int dev = local.get_device();
  c10::cuda::CUDAGuard guard(dev);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  dim3 grid(nt * (nt + 1) / 2, static_cast<unsigned>(table.size(0)));
  symm_pull_slots_kernel<<<grid, 256, 0, stream>>>(local.data_ptr<float>(),
                                                   reinterpret_cast<const long long*>(peers.data_ptr<int64_t>()),
                                                   reinterpret_cast<const SlotRow*>(table.data_ptr<int64_t>()),
                                                   static_cast<int>(world), static_cast<float>(beta));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

}  // namespace b200
